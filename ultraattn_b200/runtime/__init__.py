from .context_parallel import ContextParallelAttention, plan_allocation
from .executor import FaultInjector, PlanExecutor
from .fused import FakeSpace, FusedContextParallel, PeerSpace, SymmMemSpace
from .grid import GridExecutor
from .verify import verify_fused_tables
from .heartbeat import StepHeartbeat
from .graphed import GraphedAttention
