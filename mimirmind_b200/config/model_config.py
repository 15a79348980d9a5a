"""Typed model configuration read from a model folder's ``config.json``.

The reference fills one architecture-agnostic ``LlmConfig`` from container
metadata with "required key throws / optional key takes a logged default"
helpers (src/model/LlmConfig.cpp:64-93) and has an HF ``config.json`` reader of
the same style for another architecture
(src/runtime/nvfp4/Qwen3_5MoeConfig.cpp:20-114).  This module is that mechanism
for the Qwen2.5 dense decoder's own ``config.json`` keys.  Nothing here knows a
model size: every number comes from the file.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """Raised for a config.json that cannot describe a runnable model."""


class _Reader:
    """Required/optional typed access to a JSON object, collecting what was read."""

    def __init__(self, obj: Dict[str, Any], where: str):
        if not isinstance(obj, dict):
            raise ConfigError(f"{where}: not a JSON object")
        self.obj = obj
        self.where = where
        self.defaults_used: List[str] = []

    def _get(self, key: str):
        return self.obj.get(key, None)

    def req_int(self, key: str, minimum: int = 1) -> int:
        v = self._get(key)
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{self.where}: missing required integer '{key}'")
        if v < minimum:
            raise ConfigError(f"{self.where}: '{key}' = {v} must be >= {minimum}")
        return v

    def opt_int(self, key: str, default: Optional[int], minimum: int = 0) -> Optional[int]:
        v = self._get(key)
        if v is None:
            self.defaults_used.append(key)
            return default
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{self.where}: '{key}' must be an integer, got {v!r}")
        if v < minimum:
            raise ConfigError(f"{self.where}: '{key}' = {v} must be >= {minimum}")
        return v

    def opt_float(self, key: str, default: float) -> float:
        v = self._get(key)
        if v is None:
            self.defaults_used.append(key)
            return default
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: '{key}' must be a number, got {v!r}")
        return float(v)

    def opt_bool(self, key: str, default: bool) -> bool:
        v = self._get(key)
        if v is None:
            self.defaults_used.append(key)
            return default
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: '{key}' must be true or false, got {v!r}")
        return v

    def opt_str(self, key: str, default: Optional[str]) -> Optional[str]:
        v = self._get(key)
        if v is None:
            self.defaults_used.append(key)
            return default
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: '{key}' must be a string, got {v!r}")
        return v


@dataclass(frozen=True)
class Qwen2Config:
    """Hyper-parameters of one Qwen2.5 dense decoder, as its config.json states them.

    Key → meaning follows the reference's HF-key table
    (src/runtime/nvfp4/Qwen3_5MoeConfig.cpp:55-63, 79) and its defaults
    (src/model/LlmConfig.cpp:97-106, 159-161): ``num_key_value_heads`` defaults to
    the head count, ``head_dim`` to ``hidden_size / num_attention_heads``
    (src/model/LlmConfig.hpp:145-150), ``rms_norm_eps`` to 1e-6 and ``rope_theta``
    to 10000.
    """

    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    hidden_act: str
    # One entry per layer: 0 = the layer sees every earlier key, W > 0 = it sees the
    # last W keys (itself included), the reference's window rule
    # (src/compute/Attention.cpp:46-50).
    layer_windows: Tuple[int, ...]
    torch_dtype: str
    eos_token_ids: Tuple[int, ...] = ()
    defaults_used: Tuple[str, ...] = field(default=(), compare=False)

    # ---- derived sizes -------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def to_json_dict(self) -> Dict[str, Any]:
        """The config.json this configuration would be read back from."""
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
        }
        windows = set(w for w in self.layer_windows if w > 0)
        if windows:
            (w,) = windows
            d["use_sliding_window"] = True
            d["sliding_window"] = w
            d["layer_types"] = [
                "sliding_attention" if lw > 0 else "full_attention" for lw in self.layer_windows
            ]
        else:
            d["use_sliding_window"] = False
        if self.eos_token_ids:
            d["eos_token_id"] = (
                self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
            )
        return d


def parse_qwen2_config(obj: Dict[str, Any], where: str = "config.json") -> Qwen2Config:
    """Build a :class:`Qwen2Config` from the parsed JSON object of a config.json."""
    top = _Reader(obj, where)
    # Multimodal checkpoints nest the text model under "text_config"
    # (src/runtime/nvfp4/Qwen3_5MoeConfig.cpp:27-31).
    if isinstance(obj.get("text_config"), dict):
        r = _Reader(obj["text_config"], where + ":text_config")
    else:
        r = top

    archs = obj.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        architecture = archs[0]
    else:
        raise ConfigError(f"{where}: missing 'architectures' (a list naming the model class)")

    layers = r.req_int("num_hidden_layers")
    hidden = r.req_int("hidden_size")
    heads = r.req_int("num_attention_heads")
    inter = r.req_int("intermediate_size")
    vocab = r.req_int("vocab_size")
    kv_heads = r.opt_int("num_key_value_heads", heads, minimum=1)
    head_dim = r.opt_int("head_dim", None, minimum=1)
    if head_dim is None:
        if hidden % heads != 0:
            raise ConfigError(
                f"{where}: hidden_size {hidden} is not a multiple of num_attention_heads {heads} "
                "and no 'head_dim' is given"
            )
        head_dim = hidden // heads
    eps = r.opt_float("rms_norm_eps", 1e-6)
    theta = r.opt_float("rope_theta", 10000.0)
    max_pos = r.opt_int("max_position_embeddings", 32768, minimum=1)
    tied = r.opt_bool("tie_word_embeddings", False)
    act = r.opt_str("hidden_act", "silu")
    dtype = r.opt_str("torch_dtype", None) or r.opt_str("dtype", "bfloat16")

    if heads % kv_heads != 0:
        # src/compute/Attention.cpp:28-31
        raise ConfigError(
            f"{where}: num_attention_heads {heads} must be a multiple of num_key_value_heads {kv_heads}"
        )
    if head_dim % 2 != 0:
        # src/compute/Rope.cpp:20-22
        raise ConfigError(f"{where}: head_dim {head_dim} must be even for rotary position encoding")
    if eps <= 0.0:
        raise ConfigError(f"{where}: rms_norm_eps must be positive, got {eps}")
    if theta <= 0.0:
        raise ConfigError(f"{where}: rope_theta must be positive, got {theta}")
    if act != "silu":
        raise ConfigError(f"{where}: hidden_act '{act}' is not supported (this architecture uses 'silu')")
    if dtype not in ("bfloat16", "float32", "float16"):
        raise ConfigError(f"{where}: torch_dtype '{dtype}' is not one of bfloat16, float16, float32")

    scaling = r.obj.get("rope_scaling")
    if scaling is not None:
        # The reference runs plain rotary for this architecture: frequency factors are
        # applied only when a factor tensor exists (src/runtime/arch/Qwen2Backend.cpp:54-71).
        raise ConfigError(f"{where}: rope_scaling {scaling!r} is not supported (only plain rotary)")

    # Sliding window.  `layer_types` is authoritative when present (the reference treats
    # it so, src/runtime/nvfp4/Qwen3_5MoeConfig.cpp:101-106); otherwise the first
    # `max_window_layers` layers see every key and the rest see a window.
    use_window = r.opt_bool("use_sliding_window", False)
    window = r.opt_int("sliding_window", None, minimum=1)
    layer_types = r.obj.get("layer_types")
    windows: List[int]
    if not use_window:
        windows = [0] * layers
    else:
        if window is None:
            raise ConfigError(f"{where}: use_sliding_window is true but 'sliding_window' is missing")
        if layer_types is not None:
            if not isinstance(layer_types, list) or len(layer_types) != layers:
                raise ConfigError(f"{where}: 'layer_types' must list {layers} layers")
            windows = []
            for i, t in enumerate(layer_types):
                if t == "full_attention":
                    windows.append(0)
                elif t == "sliding_attention":
                    windows.append(window)
                else:
                    raise ConfigError(f"{where}: layer_types[{i}] = {t!r} is not a kind this architecture has")
        else:
            # no default: a guessed boundary would silently turn a windowed checkpoint into a full-attention one
            if "max_window_layers" not in r.obj:
                raise ConfigError(f"{where}: use_sliding_window is true but neither 'layer_types' nor "
                                  "'max_window_layers' says which layers are windowed")
            first_windowed = r.opt_int("max_window_layers", layers, minimum=0)
            windows = [0 if i < first_windowed else window for i in range(layers)]

    eos = r.obj.get("eos_token_id")
    if eos is None:
        eos_ids: Tuple[int, ...] = ()
    elif isinstance(eos, int) and not isinstance(eos, bool):
        eos_ids = (eos,)
    elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
        eos_ids = tuple(eos)
    else:
        raise ConfigError(f"{where}: 'eos_token_id' must be an integer or a list of integers")

    return Qwen2Config(
        architecture=architecture,
        vocab_size=vocab,
        hidden_size=hidden,
        intermediate_size=inter,
        num_hidden_layers=layers,
        num_attention_heads=heads,
        num_key_value_heads=kv_heads,
        head_dim=head_dim,
        rms_norm_eps=eps,
        rope_theta=theta,
        max_position_embeddings=max_pos,
        tie_word_embeddings=tied,
        hidden_act=act,
        layer_windows=tuple(windows),
        torch_dtype=dtype,
        eos_token_ids=eos_ids,
        defaults_used=tuple(r.defaults_used),
    )


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json in the model folder")
    with open(path, "r", encoding="utf-8") as f:
        try:
            obj = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(obj, dict):
        raise ConfigError(f"{path}: not a JSON object")
    return obj
