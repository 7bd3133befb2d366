"""Reference: orchestrated_attn/utils.py (data carriers :34-298, communication wrappers :300-380)."""
from ultraattn_b200.parallel.communicator import (InterComm, InterComm_fused, IntraComm,  # noqa: F401
                                                  IntraComm_fused)
from ultraattn_b200.runtime.orchestrated import (Input_Col_Bwd, Input_Col_Fwd, Input_Row_Bwd,  # noqa: F401
                                                 Input_Row_Fwd, Integrated_Data, Output_Col_Bwd,
                                                 Output_Col_Fwd, Output_Row_Bwd, Output_Row_Fwd)
