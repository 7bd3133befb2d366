"""Reference: search_algo/graph_transformation_engine.py."""
from ultraattn_b200.planner.fuse import (Comm_Rebuild_Engine, Comp_Fusion_Substitution,  # noqa: F401
                                         Comp_Fusion_Transformation, Graph_Substitution,
                                         Graph_Transformation, Graph_Transformation_Engine)
