"""Reference: search_algo/graph_transformation_engine.py."""
from ultraattn_b200.planner.fuse import (Comp_Fusion_Substitution, Comp_Fusion_Transformation,  # noqa: F401
                                         Graph_Transformation_Engine)
