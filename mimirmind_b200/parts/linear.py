"""Matrix products of the parts: y = x · Wᵀ (+ bias), W stored [out, in].

The reference computes ``Y[m,n] = Σ_k X[m,k]·W[n,k]`` (src/compute/Matmul.cpp:54-65) and,
on CUDA, picks a kernel by weight type and M, with cuBLASLt as its bf16 library path
(src/compute/cuda/GpuMatmul.cpp:786-884, 1095-1430).  Here the choice is by dtype only:

* fp32 activations or fp32 weights → this library's fp32-FMA kernel (true 32-bit, each
  output summed over k in ascending order, independent of the batch);
* bf16 × bf16 → the tensor-core route chosen by :mod:`mimirmind_b200.kernels.matmul_bf16`.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Runtime


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], rt: Runtime,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    out_dtype = out_dtype or x.dtype
    m, n = x.shape[0], weight.shape[0]
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and rt.matmul != "simt":
        from ..kernels import matmul_bf16
        return matmul_bf16.matmul_nt(x, weight, bias, out_dtype)
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    return ops.gemm_simt(x, weight, bias, out)
