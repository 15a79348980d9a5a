"""Choice of attention kernel for a step.

The 32-bit path and head sizes the tensor-core kernels are not built for run the
position-aligned fp32 kernel; bfloat16 with a supported head size runs the tensor-core
kernels: a tiled prefill kernel for long portions and a split-key kernel for short ones.
The reference dispatches the same way on the query length (decode vs prefill flash,
src/compute/cuda/GpuOps.cpp:2711-2731).
"""
from __future__ import annotations

import torch

from . import ops


def paged_attention(q, cache, out, ctx, num_heads: int, num_kv_heads: int, head_dim: int, window: int,
                    scale: float) -> torch.Tensor:
    if q.dtype == torch.bfloat16:
        from . import attention_bf16
        if attention_bf16.supports(head_dim, num_heads, num_kv_heads):
            return attention_bf16.run(q, cache, out, ctx, num_heads, num_kv_heads, head_dim, window, scale)
    return ops.attention_generic(q, cache.k_pages, cache.v_pages, out, ctx.positions, ctx.token_req,
                                 cache.block_table, cache.page_size, num_heads, num_kv_heads, head_dim, window, scale)
