"""Typed model configuration read from a model folder's ``config.json`` (the reader is C++: ``csrc/host/model_config.cpp``).

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
from typing import Any, Dict, Tuple


class ConfigError(ValueError):
    """Raised for a config.json that cannot describe a runnable model."""


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
    """Build a :class:`Qwen2Config` from the parsed JSON object of a config.json.

    The reading itself (required and optional keys, defaults, the checks and their messages, the window of every layer)
    is the host library's (``csrc/host/model_config.cpp``); this is its Python face."""
    from ..cache import host
    if not isinstance(obj, dict):
        raise ConfigError(f"{where}: not a JSON object")
    try:
        text = json.dumps(obj).encode("utf-8")
    except (TypeError, ValueError) as e:
        raise ConfigError(f"{where}: not a JSON object ({e})") from None
    lib = host.load()
    answer = lib.mmh_config_qwen2(text, len(text), where.encode("utf-8"))
    if not answer:
        raise ConfigError(host.last_error())
    f = json.loads(answer.decode("utf-8"))
    return Qwen2Config(
        architecture=f["architecture"], vocab_size=f["vocab_size"], hidden_size=f["hidden_size"], intermediate_size=f["intermediate_size"],
        num_hidden_layers=f["num_hidden_layers"], num_attention_heads=f["num_attention_heads"], num_key_value_heads=f["num_key_value_heads"],
        head_dim=f["head_dim"], rms_norm_eps=float(f["rms_norm_eps"]), rope_theta=float(f["rope_theta"]),
        max_position_embeddings=f["max_position_embeddings"], tie_word_embeddings=f["tie_word_embeddings"], hidden_act=f["hidden_act"],
        layer_windows=tuple(f["layer_windows"]), torch_dtype=f["torch_dtype"], eos_token_ids=tuple(f["eos_token_ids"]),
        defaults_used=tuple(f["defaults_used"]),
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
