"""bfloat16 matrix products y = x · Wᵀ (+ bias) on the tensor cores.

The plain product of a part that does not fuse anything into it.  Up to ``ops.GEMV_MAX_ROWS`` rows go to this
library's weight-streaming kernel (csrc/gemv_bf16.cu); beyond that the route is cuBLAS through ``torch.mm`` (the
reference's bf16 library route is cuBLASLt, src/compute/cuda/GpuMatmul.cpp:786-884); accumulation is fp32 inside
the product and the result is rounded once to the requested dtype.  The products with fused epilogues (the decode
layer's, csrc/gemv_bf16.cu and csrc/gemm_skinny_tcgen05.cu; the prefill gate/up product, csrc/gemm_tcgen05.cu) are
called by the parts directly.
"""
from __future__ import annotations

from typing import Optional

import torch


def matmul_nt(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    from . import ops
    if ops.gemv_supported(x.shape[0], weight.shape[0], weight.shape[1]):
        return ops.gemv_bf16(x, weight, bias, out_dtype)          # a handful of rows: weight streaming
    if out_dtype == torch.float32:
        y = torch.mm(x, weight.t(), out_dtype=torch.float32)
        if bias is not None:
            y += bias.float()
        return y
    if bias is not None:
        return torch.addmm(bias.to(x.dtype), x, weight.t())
    return torch.mm(x, weight.t())
