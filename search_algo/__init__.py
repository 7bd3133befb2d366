"""Import-compatible names of the reference's planner package, backed by ``ultraattn_b200``.

Plans pickled by this framework use these module paths (``search_algo.execute_plan.Execution_Plan``
and friends), the same ones the reference's pickles are bound to.
"""
