"""Parallelism helpers built on the ``bccl`` backend: DDP communication hooks whose bucket all-reduce
is the backend's fused peer-memory kernel, FSDP2 glue, tensor-parallel fused cross entropy, expert parallelism
(``moe``), pipeline schedules (``pipeline``)."""
from .ddp import fused_allreduce_hook, bf16_compress_fused_hook, wrap_ddp  # noqa: F401
from . import fsdp  # noqa: F401
from .loss import parallel_fused_cross_entropy  # noqa: F401
from .sharded_grad_scaler import ShardedGradScaler  # noqa: F401
from .pipeline import PipelineStage, split_into_stages  # noqa: F401
