"""Process configuration: one strict JSON file, command-line values override it.

In the reference's manner (src/core/config/Config.hpp:362-415, config.example.json): a
``models`` list with ``id`` and ``path`` and a ``defaultModel``, a ``runtime`` section
(``maxContextTokens``), a ``serving`` section (``tokenBudget`` 1..8192 default 512,
``maxActiveRequests`` 1..256 default 32, ``blockSize`` 8/16/32 default 16) and a
``diagnostics`` section; an unknown key is an error, not a warning.  Keys the reference has
for servers, other backends, speculative decoding or host governors do not exist here.
Ours, beside the reference's: ``runtime.dtype``, ``runtime.cacheTokens`` (size of the page
pool in tokens; 0 sizes it from the free device memory, ``runtime.cacheMemoryFraction`` of it), ``serving.prefillChunk``, and ``models[].random`` (a config.json object and
a seed instead of a path).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class EngineConfigError(ValueError):
    pass


@dataclass
class ModelEntry:
    id: str = ""
    path: str = ""
    title: str = ""
    random: Optional[Dict[str, Any]] = None   # {"config": {...config.json...}, "seed": int}


@dataclass
class RuntimeSettings:
    dtype: str = "bfloat16"
    maxContextTokens: int = 8192
    cacheTokens: int = 0          # size of the page pool in tokens; 0: what fits in cacheMemoryFraction of the free device
                                  # memory once the weights are loaded, at most maxContextTokens * serving.maxActiveRequests
    cacheMemoryFraction: float = 0.9


@dataclass
class ServingSettings:
    tokenBudget: int = 512
    maxActiveRequests: int = 32
    blockSize: int = 16
    prefillChunk: int = 0


@dataclass
class DiagnosticsSettings:
    parityDump: str = ""          # prefix of the per-stage dump files of a prefill (reference: diagnostics.parityDump)
    traceDecodeFile: str = ""     # one JSON line per decode step (reference: diagnostics.traceDecodeFile)
    profile: bool = False         # the command line prints where a prefill and a decode step spend their time


@dataclass
class EngineConfig:
    defaultModel: str = ""
    models: List[ModelEntry] = field(default_factory=list)
    runtime: RuntimeSettings = field(default_factory=RuntimeSettings)
    serving: ServingSettings = field(default_factory=ServingSettings)
    diagnostics: DiagnosticsSettings = field(default_factory=DiagnosticsSettings)

    def model(self, model_id: Optional[str] = None) -> ModelEntry:
        mid = model_id or self.defaultModel
        for m in self.models:
            if m.id == mid:
                return m
        if not mid and self.models:
            return self.models[0]
        raise EngineConfigError(f"no model with id '{mid}' in the configuration")


def _fill(section: str, cls, obj: Any):
    if not isinstance(obj, dict):
        raise EngineConfigError(f"'{section}' must be an object")
    inst = cls()
    known = inst.__dataclass_fields__
    for k, v in obj.items():
        if k not in known:
            raise EngineConfigError(f"unknown key '{section}.{k}' (known: {', '.join(known)})")
        want = type(getattr(inst, k)) if getattr(inst, k) is not None else None
        if want is None and v is not None and not isinstance(v, dict):
            raise EngineConfigError(f"'{section}.{k}' must be an object")
        if want is bool and not isinstance(v, bool):
            raise EngineConfigError(f"'{section}.{k}' must be true or false")
        if want is int and (isinstance(v, bool) or not isinstance(v, int)):
            raise EngineConfigError(f"'{section}.{k}' must be an integer")
        if want is str and not isinstance(v, str):
            raise EngineConfigError(f"'{section}.{k}' must be a string")
        if want is float:
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                raise EngineConfigError(f"'{section}.{k}' must be a number")
            v = float(v)
        setattr(inst, k, v)
    return inst


def parse_engine_config(obj: Dict[str, Any]) -> EngineConfig:
    if not isinstance(obj, dict):
        raise EngineConfigError("configuration must be a JSON object")
    cfg = EngineConfig()
    for k, v in obj.items():
        if k == "defaultModel":
            if not isinstance(v, str):
                raise EngineConfigError("'defaultModel' must be a string")
            cfg.defaultModel = v
        elif k == "models":
            if not isinstance(v, list):
                raise EngineConfigError("'models' must be a list")
            cfg.models = [_fill(f"models[{i}]", ModelEntry, m) for i, m in enumerate(v)]
        elif k == "runtime":
            cfg.runtime = _fill("runtime", RuntimeSettings, v)
        elif k == "serving":
            cfg.serving = _fill("serving", ServingSettings, v)
        elif k == "diagnostics":
            cfg.diagnostics = _fill("diagnostics", DiagnosticsSettings, v)
        else:
            raise EngineConfigError(f"unknown key '{k}' (known: defaultModel, models, runtime, serving, diagnostics)")
    validate(cfg)
    return cfg


def validate(cfg: EngineConfig) -> None:
    s, r = cfg.serving, cfg.runtime
    # ranges of the reference (src/core/config/Config.hpp:285-351)
    if not (1 <= s.tokenBudget <= 8192):
        raise EngineConfigError("serving.tokenBudget must be in 1..8192")
    if not (1 <= s.maxActiveRequests <= 256):
        raise EngineConfigError("serving.maxActiveRequests must be in 1..256")
    if s.blockSize not in (8, 16, 32, 64):
        raise EngineConfigError("serving.blockSize must be 8, 16, 32 or 64")
    if s.prefillChunk < 0:
        raise EngineConfigError("serving.prefillChunk must be >= 0")
    if r.dtype not in ("bfloat16", "float32"):
        raise EngineConfigError("runtime.dtype must be bfloat16 or float32")
    if r.maxContextTokens < 1:
        raise EngineConfigError("runtime.maxContextTokens must be positive")
    if r.cacheTokens < 0:
        raise EngineConfigError("runtime.cacheTokens must be >= 0")
    if not (0.0 < r.cacheMemoryFraction <= 1.0):
        raise EngineConfigError("runtime.cacheMemoryFraction must be in (0, 1]")
    ids = [m.id for m in cfg.models]
    if len(set(ids)) != len(ids):
        raise EngineConfigError("model ids must be unique")
    for m in cfg.models:
        if not m.id:
            raise EngineConfigError("every model needs an 'id'")
        if bool(m.path) == bool(m.random):
            raise EngineConfigError(f"model '{m.id}' needs either 'path' or 'random'")


def load_engine_config(path: str) -> EngineConfig:
    """Fails hard when the file is missing or malformed, like the reference's --config
    (src/mimirmind/CliParser.cpp:34-36)."""
    if not os.path.isfile(path):
        raise EngineConfigError(f"config file '{path}' not found")
    with open(path, "r", encoding="utf-8") as f:
        try:
            obj = json.load(f)
        except json.JSONDecodeError as e:
            raise EngineConfigError(f"{path}: not valid JSON ({e})") from None
    return parse_engine_config(obj)
