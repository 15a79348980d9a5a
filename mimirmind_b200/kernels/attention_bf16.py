"""Tensor-core attention kernels for bfloat16 (bound when built)."""
from __future__ import annotations


def supports(head_dim: int, num_heads: int, num_kv_heads: int) -> bool:
    return False


def run(*args, **kwargs):
    raise NotImplementedError
