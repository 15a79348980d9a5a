"""bfloat16 matrix products y = x · Wᵀ (+ bias) on the tensor cores.

Up to 16 rows go to this library's weight-streaming kernel (csrc/gemv_bf16.cu).  Beyond that the
library route is cuBLAS through ``torch.mm`` (the reference's bf16 library route is
cuBLASLt, src/compute/cuda/GpuMatmul.cpp:786-884); accumulation is fp32 inside the
product and the result is rounded once to the requested dtype.
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
