from .blocks import (BSA_Config, BSA_Repr, Block_Comp_Volume, Block_Table_Type, Block_Type, CAUSAL,
                     EMPTY, FULL, coarsen, refine)
from .named import (by_name, causal, cmap_contiguous, cmap_strided, cmap_zigzag,
                    create_bsa_block_table, document, full, global_local, permute_pattern,
                    remap_permutation, star, streaming, strided)
from .oracle import dense_attention, dense_attention_with_grads
