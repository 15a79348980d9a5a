#!/usr/bin/env python3
"""Makes the golden vectors under tests/golden/ from the reference's own CPU code.

For each tiny configuration it writes a random model folder (the package's random-weights
mode, seeded), builds ``ref_harness.cpp`` against the reference's sources (path given by
--reference, default the REFERENCE_ROOT environment variable), runs it on one token
sequence and stores ``<name>.npz``: the configuration, seed, tokens, and the reference's
logits and final hidden state as float32.  ``test_plain_vs_golden.py`` regenerates the same
weights from the seed and compares the plain implementation with these files.

The reference's block has no sliding window for this architecture
(src/runtime/arch/Qwen2Backend.cpp:424), so the golden configurations have none; its attention function has one
(src/compute/Attention.cpp:46-50), and ``golden_attention.npz`` holds its outputs for direct calls with a window
and a position offset.

    python tests/golden/make_golden.py --reference /path/to/mimirmind
"""
import argparse
import glob
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from golden_configs import GOLDEN, GOLDEN_ATTENTION, attention_inputs  # noqa: E402

SOURCES = [
    "runtime/arch/Qwen2Backend.cpp", "runtime/KvCache.cpp", "runtime/BlockBuffers.cpp", "compute/cpu/GpuOps.cpp",
    "compute/cpu/GpuMatmul.cpp", "compute/Norm.cpp", "compute/Rope.cpp", "compute/Attention.cpp",
    "compute/Activations.cpp", "compute/Matmul.cpp", "compute/Dequant.cpp", "compute/GatedDeltaNet.cpp",
    "compute/QuantTypeRegistry.cpp", "compute/Embedding.cpp", "core/cpu/CpuContext.cpp", "core/gguf/WeightsMap.cpp",
    "core/gguf/GgufTypes.cpp", "core/log/Log.cpp",
]


def build(ref_root: str, out: str) -> None:
    src = os.path.join(ref_root, "src")
    files = [os.path.join(src, s) for s in SOURCES] + sorted(glob.glob(os.path.join(src, "compute/quant/*.cpp")))
    cmd = ["g++", "-std=c++23", "-O1", "-I", src, "-I", os.path.join(ref_root, "third_party"),
           "-I", os.path.join(ref_root, "third_party/nlohmann"), os.path.join(HERE, "ref_harness.cpp")] + files + ["-o", out, "-lpthread"]
    subprocess.run(cmd, check=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("REFERENCE_ROOT", ""))
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(args.reference, "src")):
        sys.exit("give --reference: the root of the reference's source tree")
    from mimirmind_b200.weights import write_random_model
    import plain_qwen2 as plain

    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "ref_harness")
        build(args.reference, exe)
        for name, g in GOLDEN.items():
            mdir = os.path.join(tmp, name)
            write_random_model(mdir, g["config"], g["seed"], "float32")
            m = plain.PlainModel(mdir)
            tokens = np.random.RandomState(g["seed"] + 100).randint(0, m.V, size=g["tokens"]).astype(np.int32)
            order = ["model.embed_tokens.weight"]
            for i in range(m.L):
                p = f"model.layers.{i}."
                order += [p + s for s in (
                    "input_layernorm.weight", "self_attn.q_proj.weight", "self_attn.q_proj.bias", "self_attn.k_proj.weight",
                    "self_attn.k_proj.bias", "self_attn.v_proj.weight", "self_attn.v_proj.bias", "self_attn.o_proj.weight",
                    "post_attention_layernorm.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight")]
            order.append("model.norm.weight")
            tied = "lm_head.weight" not in m.w
            if not tied:
                order.append("lm_head.weight")
            inp, outp = os.path.join(tmp, name + ".in"), os.path.join(tmp, name + ".out")
            with open(inp, "wb") as f:
                f.write(struct.pack("<9I", m.L, m.d, m.cfg["intermediate_size"], m.H, m.G, m.hd, m.V, len(tokens), int(tied)))
                f.write(struct.pack("<2f", m.eps, m.theta))
                f.write(tokens.tobytes())
                for n in order:
                    f.write(m.w[n].astype("<f4").tobytes())
            subprocess.run([exe, inp, outp], check=True)
            raw = np.fromfile(outp, dtype="<f4")
            T = len(tokens)
            logits = raw[: T * m.V].reshape(T, m.V)
            hidden = raw[T * m.V:].reshape(T, m.d)
            np.savez_compressed(os.path.join(HERE, name + ".npz"), tokens=tokens, logits=logits, hidden=hidden)
            ours = plain.forward(m, tokens.tolist())
            print(name, "max|plain - reference| =", float(np.abs(ours - logits).max()), "max|logit| =", float(np.abs(logits).max()))
        outs = {}
        for i, case in enumerate(GOLDEN_ATTENTION):
            q, k, v = attention_inputs(case)
            inp, outp = os.path.join(tmp, f"att{i}.in"), os.path.join(tmp, f"att{i}.out")
            with open(inp, "wb") as f:
                f.write(struct.pack("<7I", case["Tq"], case["Tk"], case["H"], case["G"], case["hd"], case["offset"], case["window"]))
                f.write(q.astype("<f4").tobytes() + k.astype("<f4").tobytes() + v.astype("<f4").tobytes())
            subprocess.run([exe, "--attention", inp, outp], check=True)
            outs[f"case{i}"] = np.fromfile(outp, dtype="<f4").reshape(case["Tq"], case["H"], case["hd"])
            full = np.zeros((case["Tk"], case["H"], case["hd"]))
            full[case["offset"]:case["offset"] + case["Tq"]] = q
            ours = plain.attention(full, k.astype(np.float64), v.astype(np.float64), case["window"])[case["offset"]:case["offset"] + case["Tq"]]
            print(f"attention case {i}: max|plain - reference| =", float(np.abs(ours - outs[f'case{i}']).max()))
        np.savez_compressed(os.path.join(HERE, "golden_attention.npz"), **outs)


if __name__ == "__main__":
    main()
