from .executor import FaultInjector, PlanExecutor
