"""Reference: orchestrated_attn/ (runtime)."""
from ultraattn_b200.runtime.orchestrated import (Input_Col_Bwd, Input_Col_Fwd, Input_Row_Bwd,  # noqa: F401
                                                 Input_Row_Fwd, Integrated_Data, Output_Col_Bwd,
                                                 Output_Col_Fwd, Output_Row_Bwd, Output_Row_Fwd,
                                                 OrchestratedAttnFunc, orchestrated_attn_backward,
                                                 orchestrated_attn_func)
