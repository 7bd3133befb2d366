"""Reference: search_algo/dependent_graph.py."""
from ultraattn_b200.planner.graph import Comm_Kernel, Comp_Kernel, Cuda_Kernel, Dependent_Graph  # noqa: F401
