"""Weights by tensor name: what a model expects, loading with one clear error, random init.

The reference indexes tensors by name with ``require`` throwing
"tensor '<name>' not in model" (src/core/gguf/WeightsMap.cpp:130-152) and discovers a
missing block tensor only at first use (src/runtime/arch/Qwen2Backend.cpp:174-181).  Here
the whole checkpoint is checked against the model's spec at load, and one error lists
every missing tensor, every unexpected tensor and every wrong shape.

Precision policy: floating tensors stored in 16 bits are kept as bfloat16; a tensor stored
in 32 bits stays fp32; integer tables become int32.  A float32 run upcasts everything to
fp32 (exact).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterable, Optional, Tuple

import torch

from ..config.model_config import read_config_json
from ..config.spec import ModelSpec, TensorSpec
from ..registry import (EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, get_architecture, part_class)
from .safetensors_io import SafetensorsFolder, write_safetensors


class WeightsError(ValueError):
    pass


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorSpec]:
    """Every tensor the model's parts declare, by full name."""
    out: Dict[str, TensorSpec] = {}

    def add(specs: Iterable[TensorSpec]):
        for ts in specs:
            prev = out.get(ts.name)
            if prev is not None and prev.shape != ts.shape:
                raise WeightsError(f"tensor '{ts.name}' is declared twice with shapes {prev.shape} and {ts.shape}")
            out[ts.name] = ts

    add(EMBEDDINGS.get(spec.embedding.kind).tensor_specs(spec.embedding, ""))
    for layer in spec.layers:
        add(NORMS.get(layer.mixer_norm.kind).tensor_specs(layer.mixer_norm, layer.prefix))
        add(MIXERS.get(layer.mixer.kind).tensor_specs(layer.mixer, layer.prefix))
        add(NORMS.get(layer.ffn_norm.kind).tensor_specs(layer.ffn_norm, layer.prefix))
        add(FEED_FORWARDS.get(layer.feed_forward.kind).tensor_specs(layer.feed_forward, layer.prefix))
        for extra in layer.extras.values():
            add(part_class(extra).tensor_specs(extra, layer.prefix))
    add(NORMS.get(spec.final_norm.kind).tensor_specs(spec.final_norm, ""))
    add(HEADS.get(spec.head.kind).tensor_specs(spec.head, ""))
    return out


def layer_tensor_shapes(spec: ModelSpec):
    """Per layer, the shapes of the tensors its parts declare (for estimates of a step's working memory)."""
    out = []
    for layer in spec.layers:
        specs = []
        for reg, part in ((NORMS, layer.mixer_norm), (MIXERS, layer.mixer), (NORMS, layer.ffn_norm), (FEED_FORWARDS, layer.feed_forward)):
            specs += reg.get(part.kind).tensor_specs(part, layer.prefix)
        for extra in layer.extras.values():
            specs += part_class(extra).tensor_specs(extra, layer.prefix)
        out.append([tuple(ts.shape) for ts in specs])
    return out


def _storage_dtype(t: torch.Tensor, run_dtype: torch.dtype) -> torch.dtype:
    if not t.dtype.is_floating_point:
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if t.dtype in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_spec(model_dir: str):
    """(typed config, ModelSpec) of a model folder; the class is chosen by config.json."""
    obj = read_config_json(model_dir)
    archs = obj.get("architectures")
    if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
        from ..config.model_config import ConfigError
        raise ConfigError(f"{model_dir}/config.json: missing 'architectures'")
    entry = get_architecture(archs[0])
    cfg = entry.parse_config(obj, os.path.join(model_dir, "config.json"))
    return cfg, entry.build_spec(cfg)


def load_tensors(model_dir: str, spec: ModelSpec, run_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """All tensors of the folder, validated against the spec, converted and moved to ``device``."""
    want = expected_tensors(spec)
    with SafetensorsFolder(model_dir) as folder:
        # the comparison and its one message are the container library's (csrc/host/safetensors.cpp)
        message = folder.mismatch({n: (tuple(ts.shape), ts.optional) for n, ts in want.items()}, model_dir)
        if message is not None:
            raise WeightsError(message)
        out: Dict[str, torch.Tensor] = {}
        for name in folder.names():
            t = folder.tensor(name)
            out[name] = t.to(device=device, dtype=_storage_dtype(t, run_dtype))
    return out


# ---- random weights ---------------------------------------------------------

MATRIX_STD = 0.02
BIAS_STD = 0.02
NORM_STD = 0.1


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(spec: ModelSpec, seed: int, dtype: torch.dtype, device="cpu") -> Dict[str, torch.Tensor]:
    """Seeded random weights for every declared tensor: matrices, tables and biases ~ N(0, 0.02),
    norm weights ~ 1 + N(0, 0.1).  Each tensor has its own stream keyed by (seed, name)."""
    device = torch.device(device)
    out: Dict[str, torch.Tensor] = {}
    for name, ts in expected_tensors(spec).items():
        if ts.optional:
            continue
        gen = torch.Generator(device=device)
        gen.manual_seed(_tensor_seed(seed, name))
        x = torch.randn(ts.shape, generator=gen, device=device, dtype=torch.float32)
        if ts.role == "norm":
            x = 1.0 + NORM_STD * x
        elif ts.role == "bias":
            x = BIAS_STD * x
        else:
            x = MATRIX_STD * x
        out[name] = x.to(dtype)
        del x
    return out


_DTYPE_NAMES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "fp32": torch.float32, "bf16": torch.bfloat16}


def parse_dtype(name: str) -> torch.dtype:
    try:
        return _DTYPE_NAMES[name]
    except KeyError:
        raise ValueError(f"dtype '{name}' is not one of bfloat16, float32") from None


def write_random_model(model_dir: str, config: Dict, seed: int, dtype: Optional[str] = None) -> ModelSpec:
    """Random-weights mode: writes ``config.json`` and ``model.safetensors`` for a configuration and a seed.

    ``config`` is the config.json object of the architecture; ``dtype`` (default: its torch_dtype)
    is the stored precision."""
    archs = config.get("architectures")
    entry = get_architecture(archs[0] if isinstance(archs, list) and archs else "")
    config = dict(config)
    if dtype is not None:
        config["torch_dtype"] = {"fp32": "float32", "bf16": "bfloat16"}.get(dtype, dtype)
    cfg = entry.parse_config(config, "config")
    spec = entry.build_spec(cfg)
    store_dtype = parse_dtype(config.get("torch_dtype", "bfloat16"))
    tensors = random_tensors(spec, seed, store_dtype, "cpu")
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config, f, indent=2)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return spec
