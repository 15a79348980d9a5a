"""Plain, slow implementation of the Qwen2.5 dense decoder: whole sequences, no cache.

Written from the formulas of the reference (OpenSourcePKG/mimirmind); each function cites the
file and lines it restates.  numpy float64 throughout (the reference's CPU code keeps fp32
values and accumulates dot products, norms and softmax sums in double).  It shares no
code with the package under test: it reads ``config.json`` and ``model.safetensors``
itself.  It is the oracle of the tests; ``tests/golden`` compares it once with the
reference's own CPU code.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np


# ---- reading a model folder ----------------------------------------------------

def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """8-byte little-endian header length, JSON header, raw data
    (src/core/safetensors/SafetensorsHeader.cpp:33-153)."""
    with open(path, "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen])
    data = blob[8 + hlen:]
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        raw = data[b:en]
        if e["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif e["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            a = u.view(np.float32).astype(np.float64)
        elif e["dtype"] == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        else:
            raise ValueError(f"{name}: dtype {e['dtype']} not handled by the plain reader")
        out[name] = a.reshape(e["shape"])
    return out


class PlainModel:
    def __init__(self, model_dir: str):
        with open(os.path.join(model_dir, "config.json")) as f:
            c = json.load(f)
        self.cfg = c
        self.L = c["num_hidden_layers"]
        self.d = c["hidden_size"]
        self.H = c["num_attention_heads"]
        self.G = c.get("num_key_value_heads", self.H)                    # src/model/LlmConfig.cpp:106
        self.hd = c.get("head_dim") or self.d // self.H                  # src/model/LlmConfig.hpp:145-150
        self.eps = c.get("rms_norm_eps", 1e-6)                           # src/model/LlmConfig.cpp:159
        self.theta = c.get("rope_theta", 10000.0)                        # src/model/LlmConfig.cpp:161
        self.V = c["vocab_size"]
        self.windows = layer_windows(c)
        self.w = read_safetensors(os.path.join(model_dir, "model.safetensors"))

    def logits(self, tokens: Sequence[int]) -> np.ndarray:
        """Logits [T, V] of every position of one whole sequence."""
        return forward(self, list(tokens))


def layer_windows(c: dict) -> List[int]:
    """0 = full attention; W = the layer sees the last W keys.  ``layer_types`` decides when present,
    else the first ``max_window_layers`` layers are full."""
    L = c["num_hidden_layers"]
    if not c.get("use_sliding_window", False):
        return [0] * L
    W = c["sliding_window"]
    if c.get("layer_types") is not None:
        return [W if t == "sliding_attention" else 0 for t in c["layer_types"]]
    first = c.get("max_window_layers", L)
    return [0 if i < first else W for i in range(L)]


# ---- one function for each part ---------------------------------------------------

def embedding(table: np.ndarray, ids: Sequence[int]) -> np.ndarray:
    """x[t,:] = E[id_t,:]; an id outside [0,V) gives a zero row (src/compute/Embedding.cpp:46-67);
    no scaling for this architecture (src/runtime/arch/Qwen2Backend.hpp:50)."""
    V, d = table.shape
    x = np.zeros((len(ids), d))
    for t, i in enumerate(ids):
        if 0 <= i < V:
            x[t] = table[i]
    return x


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """y = x * w / sqrt(mean(x^2) + eps), eps inside the root (src/compute/Norm.cpp:21-37)."""
    ms = (x * x).mean(axis=-1, keepdims=True)
    return x * w / np.sqrt(ms + eps)


def linear(x: np.ndarray, W: np.ndarray, b: Optional[np.ndarray] = None) -> np.ndarray:
    """Y[m,n] = sum_k X[m,k] W[n,k] (src/compute/Matmul.cpp:54-65), bias per column (:67-78)."""
    y = x @ W.T
    return y + b if b is not None else y


def rope(x: np.ndarray, positions: np.ndarray, theta: float) -> np.ndarray:
    """Split-half rotary over [T, heads, hd]: pairs (i, i+hd/2), angle = pos * theta^(-2i/hd)
    (src/compute/Rope.cpp:23-41)."""
    T, nh, hd = x.shape
    half = hd // 2
    i = np.arange(half)
    freq = theta ** (-(2.0 * i) / hd)
    ang = positions[:, None].astype(np.float64) * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * c - b * s, a * s + b * c], axis=-1)


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, window: int) -> np.ndarray:
    """Causal attention, q [T,H,hd], k,v [T,G,hd] of one whole sequence (position offset 0).
    kv head = (h*G)//H; query a sees keys [max(0, a+1-W), a]; s = (q.k)/sqrt(hd); softmax; P.v
    (src/compute/Attention.cpp:43-94; scale src/runtime/arch/Qwen2Backend.cpp:415-416)."""
    T, H, hd = q.shape
    G = k.shape[1]
    scale = 1.0 / np.sqrt(float(hd))
    out = np.zeros_like(q)
    for h in range(H):
        g = (h * G) // H
        s = (q[:, h, :] @ k[:, g, :].T) * scale           # [T, T]
        a = np.arange(T)
        mask = a[None, :] <= a[:, None]
        if window > 0:
            mask &= a[None, :] >= (a[:, None] + 1 - window)
        s = np.where(mask, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=-1, keepdims=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def swiglu(x: np.ndarray, Wg: np.ndarray, Wu: np.ndarray, Wd: np.ndarray) -> np.ndarray:
    """y = (silu(x Wg^T) * (x Wu^T)) Wd^T, silu(g) = g / (1 + exp(-g))
    (src/runtime/arch/Qwen2Backend.cpp:443-458; src/compute/Activations.cpp:25-36)."""
    g = linear(x, Wg)
    u = linear(x, Wu)
    return linear(g / (1.0 + np.exp(-g)) * u, Wd)


def block(m: PlainModel, i: int, x: np.ndarray, positions: np.ndarray) -> np.ndarray:
    """norm -> qkv(+bias) -> rope(q,k) -> attention -> o -> +residual -> norm -> swiglu -> +residual
    (src/runtime/arch/Qwen2Backend.cpp:203-461)."""
    w, p = m.w, f"model.layers.{i}."
    T = x.shape[0]
    n = rms_norm(x, w[p + "input_layernorm.weight"], m.eps)
    q = linear(n, w[p + "self_attn.q_proj.weight"], w.get(p + "self_attn.q_proj.bias")).reshape(T, m.H, m.hd)
    k = linear(n, w[p + "self_attn.k_proj.weight"], w.get(p + "self_attn.k_proj.bias")).reshape(T, m.G, m.hd)
    v = linear(n, w[p + "self_attn.v_proj.weight"], w.get(p + "self_attn.v_proj.bias")).reshape(T, m.G, m.hd)
    q, k = rope(q, positions, m.theta), rope(k, positions, m.theta)
    o = attention(q, k, v, m.windows[i]).reshape(T, m.H * m.hd)
    x = x + linear(o, w[p + "self_attn.o_proj.weight"])
    n = rms_norm(x, w[p + "post_attention_layernorm.weight"], m.eps)
    return x + swiglu(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])


def block_stages(m: PlainModel, i: int, x: np.ndarray, positions: np.ndarray) -> Dict[str, np.ndarray]:
    """The intermediate results of :func:`block` under the names of the reference's stage dumps
    (src/runtime/arch/Qwen2Backend.cpp:207, 390-392, 431, 458, 462)."""
    w, p = m.w, f"model.layers.{i}."
    T = x.shape[0]
    st = {}
    st["attn_norm"] = n = rms_norm(x, w[p + "input_layernorm.weight"], m.eps)
    q = linear(n, w[p + "self_attn.q_proj.weight"], w.get(p + "self_attn.q_proj.bias")).reshape(T, m.H, m.hd)
    k = linear(n, w[p + "self_attn.k_proj.weight"], w.get(p + "self_attn.k_proj.bias")).reshape(T, m.G, m.hd)
    v = linear(n, w[p + "self_attn.v_proj.weight"], w.get(p + "self_attn.v_proj.bias")).reshape(T, m.G, m.hd)
    q, k = rope(q, positions, m.theta), rope(k, positions, m.theta)
    st["Qcur"], st["Kcur"], st["Vcur"] = q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)
    o = attention(q, k, v, m.windows[i]).reshape(T, m.H * m.hd)
    st["attn_out"] = linear(o, w[p + "self_attn.o_proj.weight"])
    x = x + st["attn_out"]
    n = rms_norm(x, w[p + "post_attention_layernorm.weight"], m.eps)
    st["ffn_mlp"] = swiglu(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    st["l_out"] = x + st["ffn_mlp"]
    return st


def forward(m: PlainModel, tokens: List[int], return_hidden: bool = False):
    """embedding -> L blocks -> final norm -> head; head = lm_head if present else the embedding table
    (src/runtime/InferenceEngine.cpp:1374-1377, 1685-1690)."""
    x = embedding(m.w["model.embed_tokens.weight"], tokens)
    pos = np.arange(len(tokens))
    hidden = [x]
    for i in range(m.L):
        x = block(m, i, x, pos)
        hidden.append(x)
    n = rms_norm(x, m.w["model.norm.weight"], m.eps)
    head = m.w.get("lm_head.weight", m.w["model.embed_tokens.weight"])
    logits = linear(n, head)
    return (logits, hidden) if return_hidden else logits


# ---- sampling ------------------------------------------------------------------------

def greedy(logits: np.ndarray) -> int:
    """First strict maximum: the lowest index among equal maxima (src/compute/Sampling.cpp:14-27)."""
    best, bv = 0, logits[0]
    for i in range(1, len(logits)):
        if logits[i] > bv:
            best, bv = i, logits[i]
    return best


_M64 = (1 << 64) - 1


def uniform_from(seed: int, counter: int) -> float:
    """The engine's counter-based uniform stream (splitmix64 finaliser), top 24 bits → [0,1)."""
    z = (seed + 0x9E3779B97F4A7C15 * (counter + 1)) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    z ^= z >> 31
    return float(z >> 40) / 16777216.0


def sample(logits: np.ndarray, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """Temperature / top-k / top-p draw in the reference's order (src/compute/Sampling.cpp:186-263):
    order by logit descending, p = exp(l/T - max/T), keep top-k, keep the smallest prefix whose share
    reaches top-p, walk the cumulative sum with one uniform u.  Probabilities are kept as 40-bit
    fixed point like the engine, equal logits are ordered by index, and a cut inside a run of equal
    logits keeps the run."""
    l32 = logits.astype(np.float32)
    if temperature <= 0.0 or top_k == 1:
        return greedy(l32)
    V = len(l32)
    inv_t = np.float32(1.0) / np.float32(temperature)
    order = sorted(range(V), key=lambda i: (-float(l32[i]), i))
    mx = np.float32(l32[order[0]] * inv_t)
    w = [int(np.float32(np.exp(np.float32(l32[i] * inv_t - mx))) * np.float32(2.0 ** 40)) for i in order]
    kept = V
    if 0 < top_k < V:
        kept = top_k
        while kept < V and l32[order[kept]] == l32[order[kept - 1]]:
            kept += 1
    total = sum(w[:kept])
    if total == 0:
        return order[0]
    if 0.0 < top_p < 1.0:
        need = min(max(int(np.ceil(np.float64(np.float32(top_p)) * float(total))), 1), total)
        cum, cut = 0, kept
        for i in range(kept):
            cum += w[i]
            if cum >= need:
                cut = i + 1
                break
        while cut < kept and l32[order[cut]] == l32[order[cut - 1]]:
            cut += 1
        kept = cut
        total = sum(w[:kept])
    target = min(int(np.float64(np.float32(u)) * float(total)), total - 1)
    cum = 0
    for i in range(kept):
        cum += w[i]
        if target < cum:
            return order[i]
    return order[kept - 1]


def generate_greedy(m: PlainModel, prompt: Sequence[int], n_new: int) -> List[int]:
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        t = greedy(forward(m, toks)[-1].astype(np.float32))
        out.append(t)
        toks.append(t)
    return out
