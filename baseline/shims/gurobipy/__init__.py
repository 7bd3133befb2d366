"""Import-only stand-in for ``gurobipy`` (not installable here: no wheel, no licence).

The reference imports ``gurobipy`` at module level in its planner files although only its
integer-program paths use it. The benchmark arm drives the reference's solver-free choices (row-owner
allocation and the list scheduler), so nothing here may ever be *called*: every entry point raises.
"""


class GurobiUnavailable(RuntimeError):
    pass


def _refuse(*_a, **_k):
    raise GurobiUnavailable("gurobipy is an import-only stand-in on this machine; use the solver-free plan types")


class _Refusing:
    def __getattr__(self, name):
        _refuse()


class GRB:
    BINARY = "B"
    INTEGER = "I"
    CONTINUOUS = "C"
    MINIMIZE = 1
    MAXIMIZE = -1
    OPTIMAL = 2
    TIME_LIMIT = 9
    INFINITY = 1e100

    class Param:
        pass

    class Attr:
        pass


Model = Env = quicksum = _refuse
