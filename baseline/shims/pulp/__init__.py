"""Import-only stand-in for ``pulp`` (not installed here). See the ``gurobipy`` stand-in: the
reference imports it at module level; the benchmark arm never reaches a call."""


def _refuse(*_a, **_k):
    raise RuntimeError("pulp is an import-only stand-in on this machine; use the solver-free plan types")


LpProblem = LpVariable = lpSum = LpMinimize = LpMaximize = LpStatus = value = PULP_CBC_CMD = _refuse
LpBinary, LpInteger, LpContinuous = "Binary", "Integer", "Continuous"
