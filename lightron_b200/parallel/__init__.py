"""Parallel strategies.  Same public names as the reference's ``parallel/__init__.py:3-19``."""
from ..mesh import setup_distributed, get_context, get_parallel_info  # noqa: F401
from .tp import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding  # noqa: F401
from .cp import ContextParallelAttention, ring_attention, ulysses_attention  # noqa: F401
from .ep import ExpertParallel  # noqa: F401
from .pp import PipelineParallel, train_step_pipeline_afab, train_step_pipeline_1f1b  # noqa: F401
from .dp import DataParallel  # noqa: F401
from .fsdp import apply_fsdp1, apply_fsdp2  # noqa: F401
from .collectives import ring_all_reduce, ring_all_gather, ring_reduce_scatter, ring_p2p  # noqa: F401
