#!/usr/bin/env python3
"""Benchmark: decode and prefill throughput of the Qwen2.5-7B-shaped model on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 (device-timed over K
graph replays of the decode step, 2,048-token prompts, context 4,096, page size 16, random
bfloat16 weights, seeded uniform-random token ids); ``e2e`` is the same through
``Engine.generate`` with host token lists in and out; ``prefill`` is one 2,048-token prompt in
one step; ``roofline`` relates the decode step to the measured HBM bandwidth; ``points`` adds
batch 1 and 64.  A "step" is one decode step.  This engine runs on one GPU: for N > 1 it says
so and exits with 2.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The Qwen2.5-7B-shaped benchmark model and workload (the third configuration of the baseline description).
MODEL_7B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=28, hidden_size=3584,
                num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064,
                rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096,
                use_sliding_window=False, torch_dtype="bfloat16")
# Other shapes of the same architecture for --only runs (--shape): sizes of the published configurations of that name.
SHAPES = {
    "7b": {},
    "0.5b": dict(num_hidden_layers=24, hidden_size=896, num_attention_heads=14, num_key_value_heads=2, head_dim=64, intermediate_size=4864,
                 vocab_size=151936, tie_word_embeddings=True),
    "14b": dict(num_hidden_layers=48, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=13824, rms_norm_eps=1e-5),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=27648),
}
PROMPT_LEN = 2048
CONTEXT = 4096
PAGE_SIZE = 16
BATCH = 8
SETTLE_STEPS = 48       # decode replays after the prompts' prefill and before the warm-up steps (see decode_run)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, since: int = 0):
        rows = self.samples[since:]
        sm = sorted(float(r[0]) for r in rows if r[0].replace(".", "").isdigit())
        reasons = []
        for i, name in enumerate(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")):
            if any(r[3 + i].lower().startswith("active") for r in rows):
                reasons.append(name)
        mx = max((float(r[1]) for r in rows if r[1].replace(".", "").isdigit()), default=0.0)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": reasons, "samples": len(rows)}


def run_workload(name: str, layers: int) -> int:
    """One of the larger workloads, end to end through the scheduler (prefill portions, mixed steps, captured decode)."""
    import time

    import numpy as np
    import torch
    from mimirmind_b200.engine.engine import Engine
    from mimirmind_b200.engine.loader import random_model
    from mimirmind_b200.kernels import ops
    from mimirmind_b200.registry import get_architecture
    cfg = dict(MODEL_7B, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8)
    rng = np.random.RandomState(0)
    if name == "14b-serving":
        cfg.update(num_hidden_layers=48, intermediate_size=13824, rms_norm_eps=1e-5, max_position_embeddings=4096)
        lens, new, ctx = rng.randint(128, 2049, size=64).tolist(), 256, 4096
    else:
        cfg.update(num_hidden_layers=64, intermediate_size=27648, rms_norm_eps=1e-6, max_position_embeddings=16384)
        lens, new, ctx = [8192] * 8, 128, 16384
    full_layers = cfg["num_hidden_layers"]
    if layers:
        cfg["num_hidden_layers"] = layers
    arch = get_architecture(cfg["architectures"][0])
    mcfg = arch.parse_config(cfg, "bench")
    model = random_model(arch.build_spec(mcfg), seed=0, dtype="bfloat16")
    engine = Engine(model, page_size=PAGE_SIZE, cache_tokens=sum(lens) + len(lens) * (new + 64), max_context=ctx,
                    token_budget=2048, max_active=64)
    prompts = [rng.randint(0, mcfg.vocab_size, size=n).tolist() for n in lens]
    # the first run also captures the CUDA graphs of the decode batches (about a tenth of a second each); the second
    # run is the steady state of a serving process
    times = []
    for _ in range(2):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = engine.generate(prompts, max_new_tokens=new, use_eos=False)
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
    dt = times[1]
    ops.check_tcgen05_errors(torch.device("cuda"))
    gen = sum(r.stats.generated_tokens for r in res)
    # What was timed is checked.  The shortest and the longest request are run again, alone and whole in one step
    # (another batch, other kernels, other pages), with the tokens they generated in the batch appended, and the logits
    # at every place where a token was chosen are read back: the token the batch chose must be that row's maximum, or
    # within the rounding noise of bfloat16 of it (random weights give flat rows, where a near-tie may go either way
    # between two batch shapes).  The noise between two bfloat16 paths of this engine on the same weights was measured
    # at these widths as 0.010 of a row's largest magnitude after one layer, 0.019 after 4 and 0.032 after 16: it grows
    # with the square root of the depth, so the bound is 0.01 * sqrt(layers).  Exact agreements are counted beside it.
    bound = 0.01 * float(np.sqrt(mcfg.num_hidden_layers))
    from mimirmind_b200.engine.runner import StepEntry
    check = {}
    verified = True
    for which, i in (("shortest", int(np.argmin(lens))), ("longest", int(np.argmax(lens)))):
        toks = list(prompts[i]) + list(res[i].tokens[:-1])
        places = list(range(lens[i] - 1, len(toks)))
        engine.runner.add_request(("check", i))
        rows = engine.runner.step([StepEntry(("check", i), toks, places)]).float().cpu().numpy()
        engine.runner.release(("check", i))
        chosen = rows[np.arange(len(places)), res[i].tokens]
        best = rows.max(axis=1)
        worst = float(((best - chosen) / np.abs(rows).max(axis=1)).max())
        check[which] = {"request": i, "prompt_tokens": lens[i], "tokens": len(places), "exactly_the_maximum": int((chosen == best).sum()),
                        "worst_gap_over_row_scale": worst}
        verified = verified and worst <= bound
    ops.check_tcgen05_errors(torch.device("cuda"))
    print(json.dumps({"workload": name, "layers": mcfg.num_hidden_layers, "layers_of_config": full_layers, "requests": len(lens),
                      "prompt_tokens": sum(lens), "generated_tokens": gen, "first_run_seconds": times[0], "seconds": dt, "tokens_per_s": (sum(lens) + gen) / dt,
                      "generated_per_s": gen / dt, "graph_steps": engine.graph_steps,
                      "finish": sorted({r.stats.finish_reason for r in res}), "verified": verified, "check_bound": bound, "check": check,
                      "device_gib": torch.cuda.max_memory_allocated() / 2 ** 30}))
    return 0 if verified else 1


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (named in config)")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--only", default="", choices=["", "decode", "prefill", "mixed"],
                    help="run one phase only and print its timing (for profiling small cases)")
    ap.add_argument("--batch", type=int, default=BATCH, help="decode batch size of --only decode")
    ap.add_argument("--workload", default="", choices=["", "14b-serving", "32b-long"],
                    help="instead of the default run: another workload of the baseline's list through Engine.generate "
                         "(14B-shaped, 64 requests of 128..2048 prompt tokens, 256 new tokens each, continuous batching; "
                         "32B-shaped, 8 requests of 8,192 prompt tokens, 128 new tokens each)")
    ap.add_argument("--mixed-portion", type=int, default=192, help="tokens of the prompt portion in the mixed step")
    ap.add_argument("--shape", default="7b", choices=sorted(SHAPES), help="with --only: another size of the architecture (random weights)")
    ap.add_argument("--pdl", type=int, default=-1, help="for measurements: dependent launches of the weight-streaming kernels on (1) or off (0)")
    ap.add_argument("--gemv-blocks", type=int, default=-1, help="for measurements: the build of the weight-streaming kernel, for 2 or 3 resident blocks per SM (0: by the grid)")
    ap.add_argument("--prompt-len", type=int, default=0,
                    help="with --only decode or prefill: prompts of this many tokens instead of 2,048 (the context grows with them)")
    ap.add_argument("--opt", action="append", default=[], metavar="NAME=VALUE",
                    help="set a tunable of the library's dispatch (csrc/exec/exec.h, Options) for this run, e.g. cluster_max_wanted=64")
    args = ap.parse_args()

    if args.impl == "reference":
        # The attempt is on record (baseline/reference_arm.py is what drove it): the reference's binary builds offline with
        # its CUDA backend, loads a bfloat16 GGUF of this shape, and its process ends with SIGSEGV in generate() on this GPU,
        # so it is not run again.
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference builds offline (cmake -DMIMIRMIND_ENABLE_CUDA=ON) and loads a random bfloat16 GGUF, but its "
                          "CUDA backend is written for an integrated GPU whose memory the host can read: on a B200 its 'smoke' "
                          "mode dies with SIGSEGV in generate(), where the token embedding is looked up on the CPU from device memory; "
                          "its code is not run again after that crash (pip cannot install it either: no setup.py/pyproject)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    global PROMPT_LEN, CONTEXT
    if args.shape != "7b" and not args.only:
        print("bench.py: --shape goes with --only", file=sys.stderr)
        return 2
    if args.prompt_len:
        if args.only not in ("decode", "prefill"):
            print("bench.py: --prompt-len goes with --only decode or --only prefill", file=sys.stderr)
            return 2
        PROMPT_LEN = args.prompt_len
        CONTEXT = max(CONTEXT, -(-(PROMPT_LEN + SETTLE_STEPS + warmup + steps) // 1024) * 1024)
    if PROMPT_LEN + SETTLE_STEPS + warmup + steps > CONTEXT:           # the requests must fit their context
        steps = CONTEXT - PROMPT_LEN - SETTLE_STEPS - warmup
        print(f"bench.py: --steps clamped to {steps} (prompts of {PROMPT_LEN} tokens in a context of {CONTEXT})", file=sys.stderr)
    if args.workload:
        return run_workload(args.workload, args.layers)

    import torch
    from mimirmind_b200.engine.decode_graph import decode_session
    from mimirmind_b200.engine.engine import Engine
    from mimirmind_b200.engine.loader import random_model
    from mimirmind_b200.engine.runner import StepEntry
    from mimirmind_b200.kernels import lib as kernel_lib
    from mimirmind_b200.registry import get_architecture
    import numpy as np

    torch.cuda.set_device(0)
    peaks = load_peaks()
    cfg_json = dict(MODEL_7B, max_position_embeddings=max(CONTEXT, MODEL_7B["max_position_embeddings"]))
    cfg_json.update(SHAPES[args.shape])
    full_layers = cfg_json["num_hidden_layers"]
    if args.layers:
        cfg_json["num_hidden_layers"] = args.layers
    arch = get_architecture(cfg_json["architectures"][0])
    mcfg = arch.parse_config(cfg_json, "bench")
    spec = arch.build_spec(mcfg)
    kernel_lib.load(verbose=True)
    if args.pdl >= 0:
        kernel_lib.load().mm_set_pdl(args.pdl)
    if args.gemv_blocks >= 0:
        kernel_lib.load().mm_set_gemv_blocks(args.gemv_blocks)
    for item in args.opt:
        from mimirmind_b200.engine import native as native_exec
        name, _, value = item.partition("=")
        native_exec.option(name, int(value))
    model = random_model(spec, seed=0, dtype="bfloat16")
    L, d, F, V = mcfg.num_hidden_layers, mcfg.hidden_size, mcfg.intermediate_size, mcfg.vocab_size
    qs, kvs = mcfg.q_size, mcfg.kv_size
    layer_params = d * (qs + 2 * kvs) + (qs + 2 * kvs) + qs * d + 3 * d * F + 2 * d
    weight_bytes = 2 * (L * layer_params + d + V * d)               # every weight a decode step uses, once
    kv_bytes_per_token = 2 * L * kvs * 2

    max_batch = max(args.batch, 1) if args.only == "decode" else (1 if args.only == "prefill" else 64)
    # token budget: all prompts of the batch are prefilled in one step, so that the end-to-end run is
    # pure decoding after the first token, like the device-timed run
    engine = Engine(model, page_size=PAGE_SIZE, cache_tokens=max(max_batch, 2) * CONTEXT, max_context=CONTEXT,
                    token_budget=min(BATCH * PROMPT_LEN, 8192 * 16), max_active=max(max_batch, 2))
    runner = engine.runner
    rng = np.random.RandomState(0)
    prompts = [rng.randint(0, V, size=PROMPT_LEN).tolist() for _ in range(max(max_batch, BATCH + 1 if args.only == "mixed" else 5))]

    def ev():
        return torch.cuda.Event(enable_timing=True)

    clocks = ClockSampler()
    clocks.start()

    # ---- prefill: one 2,048-token prompt in one step ---------------------------------------
    def prefill_once(rid, toks):
        runner.add_request(rid)
        return runner.step([StepEntry(rid, toks, [len(toks) - 1])])

    for i in range(0 if args.only in ("decode", "mixed") else 3):
        prefill_once(("warm", i), prompts[i])
        runner.release(("warm", i))
    torch.cuda.synchronize()
    times = []
    for i in range(1 if args.only else 5):
        a, b = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        prefill_once(("pf", i), prompts[i])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        runner.release(("pf", i))
    pf_ms = sorted(times)[len(times) // 2]
    T = PROMPT_LEN
    pf_flops = 2.0 * T * L * (d * (qs + 2 * kvs) + qs * d + 3 * d * F) + 2.0 * d * V \
        + L * 2.0 * 2.0 * qs * (T * (T + 1) / 2)                     # causal attention: QK^T and PV
    # frac: against the burst figure of the library product; the runs are back to back under the power cap, so the
    # seconds-long figure is given beside it
    prefill = {"value": T / (pf_ms * 1e-3), "tokens": T, "ms": pf_ms,
               "frac": pf_flops / (pf_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), "tflops": pf_flops / (pf_ms * 1e-3) / 1e12,
               "frac_of_sustained": pf_flops / (pf_ms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12),
               "ms_min": min(times)}

    # ---- decode at a batch size: prompts prefilled, then W + K steps of the captured step ---------
    def decode_run(batch, k_steps, w_steps):
        ids = [("dec", batch, i) for i in range(batch)]
        firsts = []
        for rid, toks in zip(ids, prompts[:batch]):
            lg = prefill_once(rid, toks)
            firsts.append(int(lg.argmax(-1).item()))
        sess = decode_session(runner, batch, CONTEXT, greedy=True, feed_back=True)
        sess.bind(ids, SETTLE_STEPS + w_steps + k_steps, firsts)
        before = kernel_lib.launch_count()
        sess.step()                                   # eager + capture: the step's kernels are launched twice
        per_step_calls = (kernel_lib.launch_count() - before) // 2
        torch.cuda.synchronize()
        # The prompts' prefill has just run the GPU into its power cap, and the SM clock stays low for some tens of
        # milliseconds afterwards (the first dozen decode steps after a prefill take 3.7 ms instead of 3.4).  Decoding is
        # measured in its steady state: SETTLE_STEPS steps of the same replays (about 150 ms) come first; they belong to
        # the set-up like the prefill, and are counted neither as warm-up nor as timed steps.
        for _ in range(SETTLE_STEPS - 1):
            sess.step()
        torch.cuda.synchronize()
        mark = len(clocks.samples)                    # the clock record covers the warm-up replays too: the timed region may be shorter than a sample
        for _ in range(w_steps):
            sess.step()
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for _ in range(k_steps):
            sess.step()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / k_steps
        kv_tokens = sum(runner.length(r) for r in ids) - batch * k_steps // 2   # mean over the timed steps
        for r in ids:
            runner.release(r)
        return ms, per_step_calls, kv_tokens, mark

    # ---- a mixed step, not captured: 8 decoded tokens beside a 192-token prompt portion ------------------
    # The steady state of continuous batching.  "host_ms" is how long the call takes to return (the step is put
    # together and every kernel launched); "ms" is the device time between events around it.
    def mixed_run(k_steps):
        portion = args.mixed_portion
        ids = [("mix", i) for i in range(BATCH)]
        for rid, toks in zip(ids, prompts[:BATCH]):
            prefill_once(rid, toks)
        runner.add_request("mix-long")
        host, dev = [], []
        for i in range(3 + k_steps):          # 192 * (3 + k_steps) tokens of the long prompt must exist
            entries = [StepEntry(rid, [int(prompts[j][i])], [0]) for j, rid in enumerate(ids)]
            entries.append(StepEntry("mix-long", prompts[BATCH][portion * i:portion * (i + 1)], []))
            torch.cuda.synchronize()
            a, b = ev(), ev()
            t0 = time.perf_counter()
            a.record()
            runner.step(entries)
            b.record()
            t1 = time.perf_counter()
            torch.cuda.synchronize()
            if i >= 3:
                host.append((t1 - t0) * 1e3)
                dev.append(a.elapsed_time(b))
        for rid in ids + ["mix-long"]:
            runner.release(rid)
        med = lambda v: sorted(v)[len(v) // 2]
        return {"tokens": BATCH + portion, "decode_tokens": BATCH, "portion_tokens": portion, "ms": med(dev), "host_ms": med(host),
                "steps": k_steps, "launched_by": "library executor" if runner.native is not None else "python parts"}
    if args.only == "mixed":
        clocks.stop()
        k = max(1, min(steps, 12, PROMPT_LEN // max(args.mixed_portion, 1) - 3))      # the long prompt must last for 3 + k portions
        if args.mixed_portion < 1 or PROMPT_LEN // args.mixed_portion < 4:
            print(f"bench.py: --mixed-portion must be in 1..{PROMPT_LEN // 4}", file=sys.stderr)
            return 2
        print(json.dumps(dict(mixed_run(k), only="mixed", layers=L)))
        return 0
    if args.only == "prefill":
        clocks.stop()
        print(json.dumps({"only": "prefill", "shape": args.shape, "tokens": T, "ms": pf_ms, "tflops": prefill["tflops"], "frac": prefill["frac"], "layers": L}))
        return 0
    if args.only == "decode":
        ms, calls, kv_b, _ = decode_run(args.batch, steps, warmup)
        clocks.stop()
        nbytes = weight_bytes + kv_b * kv_bytes_per_token + args.batch * d * 2
        print(json.dumps({"only": "decode", "shape": args.shape, "batch": args.batch, "prompt_len": PROMPT_LEN, "ms_per_step": ms, "launches_per_step": calls, "layers": L,
                          "bytes_per_step": nbytes, "cache_bytes_per_step": kv_b * kv_bytes_per_token,
                          "achieved_gbs": nbytes / (ms * 1e-3) / 1e9, "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}))
        return 0
    ms8, calls, kv_tokens, mark = decode_run(BATCH, steps, warmup)
    clock_summary = clocks.summary(mark)
    value = BATCH / (ms8 * 1e-3)
    step_bytes = weight_bytes + kv_tokens * kv_bytes_per_token + BATCH * d * 2
    achieved = step_bytes / (ms8 * 1e-3) / 1e9
    points, point_rooflines = {}, {}
    if not args.no_points:
        for b, k in ((1, max(16, steps // 4)), (64, max(16, steps // 4))):
            ms, _, kv_b, _ = decode_run(b, k, warmup)
            points[f"decode_b{b}"] = b / (ms * 1e-3)
            nbytes = weight_bytes + kv_b * kv_bytes_per_token + b * d * 2
            point_rooflines[f"decode_b{b}"] = {"ms_per_step": ms, "bytes_per_step": nbytes, "achieved": nbytes / (ms * 1e-3) / 1e9,
                                               "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}

    mixed = mixed_run(min(7, PROMPT_LEN // max(args.mixed_portion, 1) - 3))

    # ---- end to end: Engine.generate, host token lists in and out ------------------------------
    # at least 128 decoded tokens per request: the first dozen steps after the prompts' prefill run at a clock that the
    # prefill's power cap has pulled down, which a run of 20 tokens would measure instead of decoding
    n_new = max(min(steps, 1024), 128) + 1       # as many decode steps as the device-timed run where the context allows
    engine.generate(prompts[:BATCH], max_new_tokens=max(engine.graph_min_steps + 1, min(n_new, 12)), use_eos=False)   # warm-up: captures the graph
    h0, d0, g0 = engine.h2d_bytes, engine.d2h_bytes, engine.graph_steps
    res = engine.generate(prompts[:BATCH], max_new_tokens=n_new, use_eos=False)
    gen = sum(r.stats.generated_tokens - 1 for r in res)
    dec_ms = max(r.stats.decode_ms for r in res)
    graph_steps = max(1, engine.graph_steps - g0)
    e2e = {"value": gen / (dec_ms * 1e-3) if dec_ms > 0 else None, "unit": "tokens/s",
           "h2d_bytes_per_step": (engine.h2d_bytes - h0) / graph_steps, "d2h_bytes_per_step": (engine.d2h_bytes - d0) / graph_steps,
           "graph_steps": graph_steps}
    clocks.stop()

    out = {
        "metric": "decode tokens/s, Qwen2.5-7B-shaped bf16, batch 8, 2048-token prompts (context 4096)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms8,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random bf16 weights, uniform-random token ids",
        "config": {"model": "Qwen2.5-7B-shaped", "layers": L, "layers_of_config": full_layers, "hidden": d, "heads": mcfg.num_attention_heads,
                   "kv_heads": mcfg.num_key_value_heads, "head_dim": mcfg.head_dim, "intermediate": F, "vocab": V,
                   "global_batch": BATCH, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "page_size": PAGE_SIZE,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (weights 15 GB per step)",
                   "decode": "CUDA graph of the step, greedy sampling on device", "settle_steps_before_warmup": SETTLE_STEPS},
        "e2e": e2e, "gpu_launches": calls * steps, "launches_per_step": calls,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "bytes_per_step": step_bytes, "peaks": peaks["source"]},
        "points": points, "point_rooflines": point_rooflines, "mixed": mixed, "clocks": clock_summary,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
