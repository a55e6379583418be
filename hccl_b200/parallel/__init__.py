"""Parallelism helpers built on the operators: tensor / sequence parallel layers and the process-group binding."""
from .tp_layers import ColumnParallelLinear, RowParallelLinear, TPContext  # noqa: F401
from .context_parallel import ring_attention, ulysses_attention  # noqa: F401
from .data_parallel import GradientBucketer, ShardedOptimizer  # noqa: F401
from .expert_parallel import moe_forward  # noqa: F401
from .pipeline_parallel import gpipe_step  # noqa: F401
