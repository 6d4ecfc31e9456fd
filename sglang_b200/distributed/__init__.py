"""Tensor-parallel block-FP8 linear layers (the part of ``python/sglang/srt/layers/linear.py`` and
``srt/distributed`` this path touches): column/row sharding of block-quantised weights and the
all-reduce after row-parallel layers, over ``torch.distributed`` (NCCL on GPUs)."""

from .expert_parallel import ep_fused_experts, ep_owner_tables  # noqa: F401
from .peer_allreduce import PeerExchange, fused_row_parallel_linear  # noqa: F401
from .peer_ep import PeerEpExchange, ep_fused_experts_peer  # noqa: F401
from .symm_mem import (SymmMemCommunicator, row_parallel_linear_symm_mem,  # noqa: F401
                       row_parallel_linear_symm_mem_fused, row_parallel_linear_symm_mem_overlapped)
from .parallel_linear import (  # noqa: F401
    ColumnParallelBlockFp8Linear,
    RowParallelBlockFp8Linear,
    row_parallel_linear_overlapped,
    shard_block_fp8_weight,
    tensor_model_parallel_all_reduce,
)
