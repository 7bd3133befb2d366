"""A small solver-agnostic MILP layer.

The planner states its two integer programs (tile allocation, kernel scheduling) against this
interface; the default backend is HiGHS through ``scipy.optimize.milp``. ``gurobipy`` or ``pulp``
are used when importable and asked for (the reference requires Gurobi:
search_algo/workload_partition.py:19-20, 287-291; search_algo/execute_plan.py:214-219). A solve
that hits its time limit returns the incumbent, like the reference's ``TimeLimit`` runs.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional

import numpy as np


@dataclass
class Solution:
    status: str            # "optimal" | "feasible" (time limit, incumbent returned) | "infeasible" | "error"
    objective: float = float("nan")
    x: Optional[np.ndarray] = None
    message: str = ""

    @property
    def ok(self) -> bool:
        return self.status in ("optimal", "feasible") and self.x is not None

    def value(self, idx: int) -> float:
        return float(self.x[idx])


@dataclass
class Model:
    name: str = "model"
    lb: list = field(default_factory=list)
    ub: list = field(default_factory=list)
    integer: list = field(default_factory=list)
    names: list = field(default_factory=list)
    rows: list = field(default_factory=list)      # (cols, vals, lo, hi)
    obj: dict = field(default_factory=dict)

    def add_var(self, name: str = "", lb: float = 0.0, ub: float = float("inf"),
                integer: bool = False) -> int:
        self.lb.append(lb)
        self.ub.append(ub)
        self.integer.append(integer)
        self.names.append(name)
        return len(self.lb) - 1

    def add_binary(self, name: str = "") -> int:
        return self.add_var(name, 0.0, 1.0, True)

    def add_constr(self, coeffs: dict, sense: str, rhs: float) -> None:
        """sum(coeffs[i] * x[i]) {<=, >=, ==} rhs"""
        cols = list(coeffs.keys())
        vals = [coeffs[c] for c in cols]
        if sense == "<=":
            lo, hi = -np.inf, rhs
        elif sense == ">=":
            lo, hi = rhs, np.inf
        elif sense == "==":
            lo, hi = rhs, rhs
        else:
            raise ValueError(sense)
        self.rows.append((cols, vals, lo, hi))

    def minimize(self, coeffs: dict) -> None:
        self.obj = dict(coeffs)

    @property
    def n_vars(self) -> int:
        return len(self.lb)

    # ---------------------------------------------------------------------------------------
    def solve(self, time_limit: float = 60.0, backend: Optional[str] = None, threads: Optional[int] = None,
              mip_rel_gap: float = 1e-6) -> Solution:
        backend = backend or os.environ.get("UA_MILP_BACKEND", "highs")
        if backend == "gurobi":
            try:
                return self._solve_gurobi(time_limit, threads)
            except ImportError:
                backend = "highs"
        if backend == "pulp":
            try:
                return self._solve_pulp(time_limit)
            except ImportError:
                backend = "highs"
        return self._solve_highs(time_limit, mip_rel_gap)

    def _solve_highs(self, time_limit: float, mip_rel_gap: float) -> Solution:
        from scipy.optimize import Bounds, LinearConstraint, milp
        from scipy.sparse import csr_matrix
        n = self.n_vars
        c = np.zeros(n)
        for i, v in self.obj.items():
            c[i] = v
        cons = []
        if self.rows:
            data, ri, ci, lo, hi = [], [], [], [], []
            for r, (cols, vals, l, h) in enumerate(self.rows):
                data.extend(vals)
                ri.extend([r] * len(cols))
                ci.extend(cols)
                lo.append(l)
                hi.append(h)
            A = csr_matrix((data, (ri, ci)), shape=(len(self.rows), n))
            cons = [LinearConstraint(A, np.array(lo), np.array(hi))]
        res = milp(c, constraints=cons, integrality=np.array(self.integer, dtype=int),
                   bounds=Bounds(np.array(self.lb), np.array(self.ub)),
                   options={"time_limit": float(time_limit), "mip_rel_gap": mip_rel_gap, "disp": False})
        if res.x is not None:
            x = np.array(res.x)
            x[np.array(self.integer, dtype=bool)] = np.round(x[np.array(self.integer, dtype=bool)])
            return Solution("optimal" if res.status == 0 else "feasible", float(res.fun), x, res.message)
        if res.status == 2:
            return Solution("infeasible", message=res.message)
        return Solution("error", message=res.message)

    def _solve_gurobi(self, time_limit: float, threads: Optional[int]) -> Solution:
        import gurobipy as gp
        m = gp.Model(self.name)
        m.setParam("OutputFlag", 0)
        m.setParam("TimeLimit", time_limit)
        m.setParam("Seed", 42)
        m.setParam("Threads", threads or int(os.getenv("GUROBI_NUM_THREADS", "64")))
        xs = [m.addVar(lb=self.lb[i], ub=self.ub[i],
                       vtype=gp.GRB.INTEGER if self.integer[i] else gp.GRB.CONTINUOUS,
                       name=self.names[i] or f"v{i}") for i in range(self.n_vars)]
        for cols, vals, lo, hi in self.rows:
            expr = gp.quicksum(v * xs[c] for c, v in zip(cols, vals))
            if lo == hi:
                m.addConstr(expr == lo)
            else:
                if np.isfinite(lo):
                    m.addConstr(expr >= lo)
                if np.isfinite(hi):
                    m.addConstr(expr <= hi)
        m.setObjective(gp.quicksum(v * xs[i] for i, v in self.obj.items()), gp.GRB.MINIMIZE)
        m.optimize()
        if m.SolCount == 0:
            return Solution("infeasible" if m.status == gp.GRB.INFEASIBLE else "error")
        x = np.array([v.X for v in xs])
        return Solution("optimal" if m.status == gp.GRB.OPTIMAL else "feasible", float(m.objVal), x)

    def _solve_pulp(self, time_limit: float) -> Solution:
        import pulp
        prob = pulp.LpProblem(self.name, pulp.LpMinimize)
        xs = [pulp.LpVariable(self.names[i] or f"v{i}", lowBound=self.lb[i],
                              upBound=None if not np.isfinite(self.ub[i]) else self.ub[i],
                              cat="Integer" if self.integer[i] else "Continuous")
              for i in range(self.n_vars)]
        prob += pulp.lpSum(v * xs[i] for i, v in self.obj.items())
        for cols, vals, lo, hi in self.rows:
            expr = pulp.lpSum(v * xs[c] for c, v in zip(cols, vals))
            if lo == hi:
                prob += expr == lo
            else:
                if np.isfinite(lo):
                    prob += expr >= lo
                if np.isfinite(hi):
                    prob += expr <= hi
        prob.solve(pulp.PULP_CBC_CMD(msg=False, timeLimit=time_limit))
        if pulp.LpStatus[prob.status] not in ("Optimal", "Not Solved"):
            return Solution("infeasible")
        x = np.array([v.value() or 0.0 for v in xs])
        return Solution("optimal" if pulp.LpStatus[prob.status] == "Optimal" else "feasible",
                        float(pulp.value(prob.objective)), x)
