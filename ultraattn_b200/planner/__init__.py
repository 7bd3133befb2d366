from .allocate import (Allocation, brute_force_allocate, comm_volumes, comp_volumes,
                       naive_allocate_strategy, solve_sparse_from_bsa, tile_volumes)
from .cost import (Comm_Profile_Map, Dist_Attn_Config, Dist_Attn_Schedule, Evaluation_Configs,
                   FlashAttn_Profile_Map, Inter_Comp_Profile_Map, Machine_Config,
                   convert_shape_config_to_str, get_cc_optimal_schedule_from_table)
from .fuse import Comp_Fusion_Substitution, Comp_Fusion_Transformation, Graph_Transformation_Engine
from .graph import Comm_Kernel, Comp_Kernel, Cuda_Kernel, Dependent_Graph
from .schedule import Execution_Plan, Fused_Execution_Plan, create_one_node_exe_plan
from .pipeline import make_plan, make_plan_collective


def _bind_reference_class_paths() -> bool:
    """Make pickles of plans name their classes by the reference's module paths
    (``search_algo.execute_plan.Execution_Plan``, ``search_algo.dependent_graph.Comp_Kernel``,
    ``search_algo.bsa_config.BSA_Repr``, ...): a plan pickled here and one pickled by the reference
    are then bound to the same names, and either loads wherever those modules import. Done only
    when the ``search_algo`` modules of this distribution are importable and export these very
    classes (pickle checks that); otherwise the classes keep their own module paths."""
    import importlib
    from ..patterns import blocks as _blocks
    from . import cost as _cost, graph as _graph, schedule as _schedule
    table = {
        "search_algo.execute_plan": [_schedule.Execution_Plan, _schedule.Fused_Execution_Plan],
        "search_algo.dependent_graph": [_graph.Cuda_Kernel, _graph.Comp_Kernel, _graph.Comm_Kernel,
                                        _graph.Dependent_Graph],
        "search_algo.search_engine": [_cost.Dist_Attn_Config, _cost.Dist_Attn_Schedule, _cost.Evaluation_Configs,
                                      _cost.Machine_Config, _cost.Comp_Profile_Map, _cost.FlashAttn_Profile_Map,
                                      _cost.Inter_Comp_Profile_Map, _cost.Comm_Profile_Map],
        "search_algo.bsa_config": [_blocks.BSA_Config, _blocks.BSA_Repr],
        "search_algo.utils": [_blocks.Block_Type, _blocks.Block_Table_Type],
    }
    try:
        mods = {name: importlib.import_module(name) for name in table}
    except Exception:       # not installed next to this package: keep the native paths
        return False
    if not all(getattr(mods[name], cls.__name__, None) is cls for name, classes in table.items() for cls in classes):
        return False
    for name, classes in table.items():
        for cls in classes:
            cls.__module__ = name
    return True


REFERENCE_CLASS_PATHS = _bind_reference_class_paths()


def bind_reference_class_paths() -> bool:
    """Idempotent; the writers of pickles call it again because the first attempt, at import time,
    cannot succeed when one of the ``search_algo`` modules is itself what triggered this import."""
    global REFERENCE_CLASS_PATHS
    if not REFERENCE_CLASS_PATHS:
        REFERENCE_CLASS_PATHS = _bind_reference_class_paths()
    return REFERENCE_CLASS_PATHS
