"""From a model folder (or a spec and a seed) to a Model on the device."""
from __future__ import annotations

from typing import Tuple

import torch

from ..config.spec import ModelSpec
from ..parts.base import Runtime
from ..registry import _ensure_builtin
from ..weights.store import load_spec, load_tensors, parse_dtype, random_tensors
from .model import Model


def require_cuda() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("mimirmind_b200 runs on a CUDA device (sm_100a); no GPU is visible and there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


def make_runtime(dtype, device=None, matmul: str = "auto") -> Runtime:
    if isinstance(dtype, str):
        dtype = parse_dtype(dtype)
    if dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("dtype must be bfloat16 or float32")
    # The 32-bit path must stay true fp32 everywhere, also inside library calls.
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    return Runtime(dtype=dtype, device=device or require_cuda(), matmul=matmul)


def load_model(model_dir: str, dtype="bfloat16", device=None, matmul: str = "auto") -> Tuple[Model, object]:
    """Reads config.json (which chooses the model class) and the safetensors weights."""
    _ensure_builtin()
    rt = make_runtime(dtype, device, matmul)
    cfg, spec = load_spec(model_dir)
    tensors = load_tensors(model_dir, spec, rt.dtype, rt.device)
    return Model(spec, tensors, rt), cfg


def random_model(spec: ModelSpec, seed: int, dtype="bfloat16", device=None, matmul: str = "auto") -> Model:
    """A model with seeded random weights made directly on the device (no folder written)."""
    _ensure_builtin()
    rt = make_runtime(dtype, device, matmul)
    tensors = random_tensors(spec, seed, rt.dtype, rt.device)
    return Model(spec, tensors, rt)
