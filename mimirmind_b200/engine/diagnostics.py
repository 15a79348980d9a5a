"""Diagnostics in the reference's manner: stage dumps of a prefill, and a per-step decode trace.

Stage dumps (``diagnostics.parityDump: "PREFIX"``): while a step holds a prompt portion, every layer writes
``PREFIX-blk<N>-<stage>.bin`` for the stages ``attn_norm``, ``Qcur``, ``Kcur``, ``Vcur``, ``attn_out``, ``ffn_mlp``
and ``l_out``, and layer 0 also ``inp_scaled`` (the embedded tokens); a file is three little-endian uint32
(block, rows, width) and then rows x width float32, the format of the reference's dumps and of its parity tool
(src/runtime/arch/Qwen2Backend.cpp:104-129, 207, 390-392, 431, 458, 462; src/runtime/InferenceEngine.cpp:1466-1543).
A later step overwrites the files of an earlier one, so this is for one prompt in one portion.  As in the reference
it synchronises at every stage and writes rows x width x 4 bytes per stage and layer: not for production traffic.

Decode trace (``diagnostics.traceDecodeFile: "PATH"``): one JSON object per line and decode step with the step's
wall time; the reference writes ``tok``, ``wall_ms``, ``cap_mhz``, ``pkg_c`` per token of its single session
(src/runtime/InferenceEngine.cpp:346-362, 2020-2040); here a step serves a batch, so a line is
``{"step", "tokens", "wall_ms", "sm_mhz", "gpu_c"}`` (clock and temperature from NVML when it can be loaded, else 0 / -1).
"""
from __future__ import annotations

import json
import struct

import torch


class StageDump:
    def __init__(self, prefix: str):
        self.prefix = prefix
        self.files_written = 0

    def write(self, block: int, stage: str, rows: torch.Tensor) -> None:
        if rows.dim() != 2:
            rows = rows.reshape(rows.shape[0], -1)
        host = rows.detach().to(torch.float32).cpu().contiguous().numpy()      # the copy waits for the kernels before it
        with open(f"{self.prefix}-blk{block}-{stage}.bin", "wb") as f:
            f.write(struct.pack("<III", block, host.shape[0], host.shape[1]))
            f.write(host.astype("<f4").tobytes())
        self.files_written += 1


def read_stage_dump(path: str):
    """(block, float32 array [rows, width]) of a dump file."""
    import numpy as np
    with open(path, "rb") as f:
        block, rows, width = struct.unpack("<III", f.read(12))
        data = np.frombuffer(f.read(), dtype="<f4")
    if data.size != rows * width:
        raise ValueError(f"{path}: header says {rows} x {width}, file holds {data.size} values")
    return block, data.reshape(rows, width)


class DecodeTrace:
    def __init__(self, path: str, device_index: int = 0):
        self._f = open(path, "w", encoding="utf-8")
        self._step = 0
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = (pynvml, pynvml.nvmlDeviceGetHandleByIndex(device_index))
        except Exception:
            self._nvml = None

    def _sensors(self):
        if self._nvml is None:
            return 0, -1.0
        nv, h = self._nvml
        try:
            return int(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), float(nv.nvmlDeviceGetTemperature(h, nv.NVML_TEMPERATURE_GPU))
        except Exception:
            return 0, -1.0

    def step(self, tokens: int, wall_ms: float) -> None:
        mhz, temp = self._sensors()
        self._f.write(json.dumps({"step": self._step, "tokens": int(tokens), "wall_ms": round(float(wall_ms), 3),
                                  "sm_mhz": mhz, "gpu_c": temp}) + "\n")
        self._step += 1

    def flush(self) -> None:
        self._f.flush()

    def close(self) -> None:
        if self._f is not None:
            self._f.close()
            self._f = None
