#!/usr/bin/env python3
"""Drives the unmodified reference program for ``bench.py --impl reference``.

The reference (OpenSourcePKG/mimirmind) is a C++/CMake program, not a Python package.  Its binary is built once,
offline, from the read-only source tree with its CUDA backend switched on::

    cmake <reference> -DMIMIRMIND_ENABLE_L0=OFF -DMIMIRMIND_ENABLE_CUDA=ON -DCMAKE_BUILD_TYPE=Release
    cmake --build . --target mimirmind -j 8        # -> baseline/_ref/bin/mimirmind and baseline/_ref/bin/ptx/

It reads GGUF files, and its engine for this architecture serves one session at a time
(src/runtime/engine/ServingSession.cpp:578-587), so what can be measured is a prompt of N tokens and decoding at
batch 1, through its own ``smoke`` mode, which prints ``prefill X ms`` and ``decode Y ms (Z ms/token)``
(src/mimirmind/diagnostics/SmokeSuite.cpp:878-895).  This script writes the model that the mode needs: a GGUF v3
file with random bfloat16 matrices of the requested Qwen2 shape (norms and biases in float32), the metadata keys
the loader requires (src/model/LlmConfig.cpp:97-160) and a tokenizer table in which every letter is a token of its
own and nothing merges, so that a prompt of N letters is N tokens (src/model/Tokenizer.cpp:162-216, 425-457).  It
then runs the binary and parses its timings.  None of this repository's kernels or engine code is on that path.
"""
import argparse
import json
import os
import re
import struct
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
BIN = os.path.join(HERE, "_ref", "bin", "mimirmind")
PTX = os.path.join(HERE, "_ref", "bin", "ptx")

GGUF_MAGIC, GGUF_VERSION, ALIGN = 0x46554747, 3, 32
T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR = 4, 5, 6, 7, 8, 9
GGML_F32, GGML_BF16 = 0, 30


def _s(text: str) -> bytes:
    b = text.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, vtype: int, payload: bytes) -> bytes:
    return _s(key) + struct.pack("<I", vtype) + payload


def write_gguf(path: str, cfg: dict, seed: int = 0) -> int:
    """Random weights of a Qwen2 shape as a GGUF file; returns its size in bytes."""
    import numpy as np
    import torch
    L, d, F, H, G, hd, V = (cfg[k] for k in ("layers", "hidden", "intermediate", "heads", "kv_heads", "head_dim", "vocab"))
    q, kv = H * hd, G * hd
    a = "qwen2"
    letters = [chr(c) for c in range(ord("a"), ord("z") + 1)]
    tokens = [letters[i] if i < 26 else f"<t{i}>" for i in range(V)]
    meta = [
        _kv("general.architecture", T_STR, _s(a)), _kv("general.name", T_STR, _s("random weights for timing")),
        _kv("general.alignment", T_U32, struct.pack("<I", ALIGN)),
        _kv(f"{a}.block_count", T_U32, struct.pack("<I", L)), _kv(f"{a}.context_length", T_U32, struct.pack("<I", cfg["context"])),
        _kv(f"{a}.embedding_length", T_U32, struct.pack("<I", d)), _kv(f"{a}.feed_forward_length", T_U32, struct.pack("<I", F)),
        _kv(f"{a}.attention.head_count", T_U32, struct.pack("<I", H)), _kv(f"{a}.attention.head_count_kv", T_U32, struct.pack("<I", G)),
        _kv(f"{a}.attention.key_length", T_U32, struct.pack("<I", hd)), _kv(f"{a}.attention.value_length", T_U32, struct.pack("<I", hd)),
        _kv(f"{a}.attention.layer_norm_rms_epsilon", T_F32, struct.pack("<f", cfg["eps"])),
        _kv(f"{a}.rope.freq_base", T_F32, struct.pack("<f", cfg["theta"])),
        _kv("tokenizer.ggml.model", T_STR, _s("llama")),
        _kv("tokenizer.ggml.tokens", T_ARR, struct.pack("<IQ", T_STR, V) + b"".join(_s(t) for t in tokens)),
        _kv("tokenizer.ggml.scores", T_ARR, struct.pack("<IQ", T_F32, V) + np.zeros(V, dtype="<f4").tobytes()),
        _kv("tokenizer.ggml.token_type", T_ARR, struct.pack("<IQ", T_I32, V) + np.ones(V, dtype="<i4").tobytes()),
        _kv("tokenizer.ggml.bos_token_id", T_U32, struct.pack("<I", V - 2)), _kv("tokenizer.ggml.eos_token_id", T_U32, struct.pack("<I", V - 1)),
        _kv("tokenizer.ggml.unknown_token_id", T_U32, struct.pack("<I", V - 3)),
        _kv("tokenizer.ggml.add_space_prefix", T_BOOL, struct.pack("<B", 0)), _kv("tokenizer.ggml.add_bos_token", T_BOOL, struct.pack("<B", 0)),
    ]
    # (name, dims innermost first, ggml type, kind)
    tensors = [("token_embd.weight", (d, V), GGML_BF16, "matrix")]
    for b in range(L):
        p = f"blk.{b}."
        tensors += [(p + "attn_norm.weight", (d,), GGML_F32, "norm"), (p + "attn_q.weight", (d, q), GGML_BF16, "matrix"), (p + "attn_q.bias", (q,), GGML_F32, "bias"),
                    (p + "attn_k.weight", (d, kv), GGML_BF16, "matrix"), (p + "attn_k.bias", (kv,), GGML_F32, "bias"),
                    (p + "attn_v.weight", (d, kv), GGML_BF16, "matrix"), (p + "attn_v.bias", (kv,), GGML_F32, "bias"),
                    (p + "attn_output.weight", (q, d), GGML_BF16, "matrix"), (p + "ffn_norm.weight", (d,), GGML_F32, "norm"),
                    (p + "ffn_gate.weight", (d, F), GGML_BF16, "matrix"), (p + "ffn_up.weight", (d, F), GGML_BF16, "matrix"),
                    (p + "ffn_down.weight", (F, d), GGML_BF16, "matrix")]
    tensors += [("output_norm.weight", (d,), GGML_F32, "norm"), ("output.weight", (d, V), GGML_BF16, "matrix")]
    infos, offset = [], 0
    for name, dims, gtype, _kind in tensors:
        n = 1
        for x in dims:
            n *= x
        infos.append(_s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", x) for x in dims) + struct.pack("<IQ", gtype, offset))
        offset += (n * (4 if gtype == GGML_F32 else 2) + ALIGN - 1) // ALIGN * ALIGN
    head = struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(tensors), len(meta)) + b"".join(meta) + b"".join(infos)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * ((ALIGN - len(head) % ALIGN) % ALIGN))
        for name, dims, gtype, kind in tensors:
            n = 1
            for x in dims:
                n *= x
            if kind == "norm":
                t = 1.0 + 0.1 * torch.randn(n, generator=gen, device=dev, dtype=torch.float32)
            else:
                t = 0.02 * torch.randn(n, generator=gen, device=dev, dtype=torch.float32)
            if gtype == GGML_BF16:
                raw = t.to(torch.bfloat16).view(torch.int16).cpu().numpy().tobytes()
            else:
                raw = t.cpu().numpy().astype("<f4").tobytes()
            f.write(raw)
            f.write(b"\0" * ((ALIGN - len(raw) % ALIGN) % ALIGN))
    return os.path.getsize(path)


def run(cfg: dict, prompt_len: int, max_new: int, workdir: str, timeout: int, backend: str = "auto") -> dict:
    """Writes the model, runs ``mimirmind smoke`` once, returns its timings (or why it could not)."""
    if not os.path.isfile(BIN):
        return {"unavailable": "the reference binary baseline/_ref/bin/mimirmind is not built (see the header of baseline/reference_arm.py)"}
    os.makedirs(workdir, exist_ok=True)
    gguf = os.path.join(workdir, "random-qwen2.gguf")
    t0 = time.time()
    size = write_gguf(gguf, cfg)
    conf = os.path.join(workdir, "config.json")
    with open(conf, "w") as f:
        json.dump({"defaultModel": "m", "models": [{"id": "m", "path": gguf, "backend": backend}],
                   "runtime": {"kvDtype": "f32", "maxContextTokens": cfg["context"]}}, f)
    prompt = "".join("abcdefghijklmnopqrstuvwxyz"[(7 * i + i // 26) % 26] for i in range(prompt_len))
    env = dict(os.environ, MIMIRMIND_HSACO_DIR=PTX)
    cmd = [BIN, "smoke", "--config", conf, "--model", gguf, "--prompt", prompt, "--max-new", str(max_new)]
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=timeout, cwd=workdir)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"the reference binary did not finish within {timeout} s", "command": " ".join(cmd[:6]) + " ..."}
    finally:
        try:
            os.remove(gguf)
        except OSError:
            pass
    out = proc.stdout + "\n" + proc.stderr
    res = {"returncode": proc.returncode, "gguf_bytes": size, "wall_s": time.time() - t0, "command": " ".join(cmd[:6]) + f" --prompt <{prompt_len} letters> --max-new {max_new}"}
    m = re.search(r"prefill\s+([0-9.]+)\s*ms\s*\((\d+)\s*tokens", out)
    if m:
        res["prefill_ms"], res["prefill_tokens"] = float(m.group(1)), int(m.group(2))
    m = re.search(r"decode\s+([0-9.]+)\s*ms\s*\(([0-9.]+)\s*ms/token\)", out)
    if m:
        res["decode_ms"], res["decode_ms_per_token"] = float(m.group(1)), float(m.group(2))
    m = re.search(r"generated\s+(\d+)", out)
    if m:
        res["generated"] = int(m.group(1))
    if proc.returncode != 0 or "decode_ms_per_token" not in res:
        res["unavailable"] = "the reference binary failed on this model: " + " | ".join(
            [ln.strip() for ln in out.splitlines() if re.search(r"ERROR|error|what\(\)|terminate|not implemented|cannot", ln)][-4:] or out.strip().splitlines()[-3:])
        res["tail"] = out.strip().splitlines()[-25:]
    return res


SHAPES = {
    "tiny": dict(layers=2, hidden=256, intermediate=512, heads=4, kv_heads=2, head_dim=64, vocab=1024, eps=1e-6, theta=10000.0, context=512),
    "7b": dict(layers=28, hidden=3584, intermediate=18944, heads=28, kv_heads=4, head_dim=128, vocab=152064, eps=1e-6, theta=1000000.0, context=4096),
}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="tiny", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--prompt-len", type=int, default=64)
    ap.add_argument("--max-new", type=int, default=16)
    ap.add_argument("--workdir", default="/tmp/mimirmind_reference_arm")
    ap.add_argument("--timeout", type=int, default=900)
    ap.add_argument("--backend", default="auto", help="the reference's backend token (auto, cpu, ...)")
    args = ap.parse_args()
    cfg = dict(SHAPES[args.shape])
    if args.layers:
        cfg["layers"] = args.layers
    print(json.dumps(run(cfg, args.prompt_len, args.max_new, args.workdir, args.timeout, args.backend)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
