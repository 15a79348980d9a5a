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
from dataclasses import asdict, dataclass, field
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


def _from_library(text: bytes, where: Optional[str]) -> EngineConfig:
    """Reading, the strict key check, the defaults and the ranges are the host library's (``csrc/host/engine_config.cpp``)."""
    from ..cache import host
    lib = host.load()
    answer = lib.mmh_engine_config(text, len(text), where.encode("utf-8") if where else None)
    if not answer:
        raise EngineConfigError(host.last_error())
    f = json.loads(answer.decode("utf-8"))
    f["runtime"]["cacheMemoryFraction"] = float(f["runtime"]["cacheMemoryFraction"])
    return EngineConfig(defaultModel=f["defaultModel"], models=[ModelEntry(**m) for m in f["models"]], runtime=RuntimeSettings(**f["runtime"]),
                        serving=ServingSettings(**f["serving"]), diagnostics=DiagnosticsSettings(**f["diagnostics"]))


def parse_engine_config(obj: Dict[str, Any]) -> EngineConfig:
    if not isinstance(obj, dict):
        raise EngineConfigError("configuration must be a JSON object")
    try:
        text = json.dumps(obj).encode("utf-8")
    except (TypeError, ValueError) as e:
        raise EngineConfigError(f"configuration is not JSON ({e})") from None
    return _from_library(text, None)


def validate(cfg: EngineConfig) -> None:
    """The same checks on a configuration that was changed after it was read (command-line values override the file)."""
    parse_engine_config(asdict(cfg))


def load_engine_config(path: str) -> EngineConfig:
    """Fails hard when the file is missing or malformed, like the reference's --config
    (src/mimirmind/CliParser.cpp:34-36)."""
    if not os.path.isfile(path):
        raise EngineConfigError(f"config file '{path}' not found")
    with open(path, "rb") as f:
        return _from_library(f.read(), path)
