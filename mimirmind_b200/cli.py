"""Command line in the reference's manner: ``mimirmind [smoke|replay] [options]``.

Option names, meanings and defaults are the reference's where it has them
(src/mimirmind/CliParser.cpp:20-56, src/mimirmind/CliArgs.hpp:47-70): ``--config PATH``
(default ./config.json, a hard error if the file is missing), ``--model PATH`` (overrides the
default model's path), ``--prompt``, ``--max-new N`` (20), ``--temperature F`` (0 = greedy),
``--top-k N`` (0 off), ``--top-p F`` (1.0 off), ``--seed N`` (0 = random), ``--log-level``, ``--dump-dir``.
This engine has no tokenizer (it takes token ids), so ``--prompt`` is a list of ids
("5 17 3" or "5,17,3"), as the reference's parity tool takes ``--tokens id,id,…``
(tools/llama-parity-dump.cpp:111-124); ``--prompt-len N`` makes N seeded random ids instead.
Server, chat and parity-against-llama.cpp modes of the reference do not exist here.
``random-weights --model-config CONFIG.JSON --seed N --out DIR [--dtype D]`` writes a model
folder with seeded random weights.

``smoke`` loads the model, generates and prints the timings the reference prints
(src/mimirmind/diagnostics/SmokeSuite.cpp:878-895): ``generated N (hit stop)``,
``prefill X ms (T tokens, L blocks)``, ``decode Y ms (Z ms/token)`` with
ms/token = decode ms / (generated − 1).
"""
from __future__ import annotations

import argparse
import re
import sys
from typing import List, Optional

USAGE_MODES = ("smoke", "replay", "random-weights")


def parse_prompt_ids(text: str) -> List[int]:
    parts = [p for p in re.split(r"[\s,]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit("--prompt must be token ids (\"5 17 3\" or \"5,17,3\"): this engine has no tokenizer") from None


def print_kernel_shares(prof, top: int = 12) -> None:
    """``diagnostics.profile``: where the GPU time of the run went, by kernel (the reference prints shares by category
    of operation with ``diagnostics.traceOpTimes``, src/runtime/perf/OpProfiler.hpp)."""
    import collections
    import torch
    agg = collections.defaultdict(lambda: [0.0, 0])
    for e in prof.events():
        if e.device_type == torch.autograd.DeviceType.CUDA:
            agg[e.name][0] += e.time_range.elapsed_us()
            agg[e.name][1] += 1
    total = sum(v[0] for v in agg.values()) or 1.0
    print(f"profile: {total / 1e3:.2f} ms of GPU time in {sum(v[1] for v in agg.values())} launches")
    for name, (us, n) in sorted(agg.items(), key=lambda kv: -kv[1][0])[:top]:
        print(f"  {100 * us / total:5.1f} %  {us / 1e3:9.3f} ms  {n:6d} x  {name[:90]}")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="mimirmind", description="B200-native inference engine (Qwen2.5 dense decoder)")
    ap.add_argument("mode", nargs="?", default="smoke", choices=USAGE_MODES)
    ap.add_argument("--config", default="./config.json", help="engine config file (default ./config.json)")
    ap.add_argument("--model", default="", help="model folder (overrides models[<defaultModel>].path)")
    ap.add_argument("--prompt", default="", help="prompt as token ids")
    ap.add_argument("--prompt-len", type=int, default=0, help="use N seeded random token ids as the prompt")
    ap.add_argument("--max-new", type=int, default=20, help="max new tokens (default 20)")
    ap.add_argument("--temperature", type=float, default=0.0, help="sampling temperature, 0 = greedy (default 0)")
    ap.add_argument("--top-k", type=int, default=0, help="top-K cutoff, 0 = disabled (default 0)")
    ap.add_argument("--top-p", type=float, default=1.0, help="top-P cutoff, 1.0 = disabled (default 1.0)")
    ap.add_argument("--seed", type=int, default=0, help="RNG seed, 0 = random (default 0)")
    ap.add_argument("--dtype", default="", choices=["", "bfloat16", "float32"], help="overrides runtime.dtype")
    ap.add_argument("--log-level", default="info", choices=["trace", "debug", "info", "warn", "error", "off"])
    ap.add_argument("--dump-dir", default="", help="directory for per-stage dumps of the prefill (sets diagnostics.parityDump to DIR/engine)")
    # replay mode
    ap.add_argument("--out", default="", help="(replay) folder for the logits files")
    ap.add_argument("--max-tokens", type=int, default=0, help="(replay) size of the cache pool in tokens")
    # random-weights mode
    ap.add_argument("--model-config", default="", help="(random-weights) a config.json of the architecture")
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.mode == "replay":
        from .replay import main as replay_main
        if not (args.model and args.out and args.max_tokens):
            raise SystemExit("replay needs --model, --out and --max-tokens")
        return replay_main(["--model", args.model, "--dtype", args.dtype or "bfloat16", "--out", args.out,
                            "--max-tokens", str(args.max_tokens)])
    if args.mode == "random-weights":
        # writes a model folder (config.json, model.safetensors) from a configuration and a seed
        import json
        from .registry import _ensure_builtin
        from .weights.store import write_random_model
        if not (args.model_config and args.out):
            raise SystemExit("random-weights needs --model-config CONFIG.JSON and --out DIR (and takes --seed, --dtype)")
        _ensure_builtin()
        with open(args.model_config, "r", encoding="utf-8") as f:
            write_random_model(args.out, json.load(f), args.seed, args.dtype or None)
        print(f"wrote {args.out}/config.json and {args.out}/model.safetensors (seed {args.seed})")
        return 0
    from .config.engine_config import EngineConfigError, ModelEntry, load_engine_config
    try:
        cfg = load_engine_config(args.config)
    except EngineConfigError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    # precedence: command line > file > default
    if args.model:
        if cfg.models:
            entry = cfg.model()
            entry.path, entry.random = args.model, None
        else:
            cfg.models.append(ModelEntry(id="primary", path=args.model))
            cfg.defaultModel = "primary"
    if args.dtype:
        cfg.runtime.dtype = args.dtype
    if args.dump_dir:
        import os
        os.makedirs(args.dump_dir, exist_ok=True)
        cfg.diagnostics.parityDump = os.path.join(args.dump_dir, "engine")
    from .engine.engine import Engine
    from .sampling import SamplingParams
    import numpy as np

    log = (lambda m: print(m, file=sys.stderr, flush=True)) if args.log_level in ("trace", "debug", "info") else (lambda m: None)
    log(f"loading model '{cfg.model().id}' ({cfg.runtime.dtype})")
    engine = Engine.from_config(cfg)
    vocab = engine.model.spec.vocab_size
    if args.prompt_len > 0:
        prompt = np.random.RandomState(args.seed or 1234).randint(0, vocab, size=args.prompt_len).tolist()
    elif args.prompt:
        prompt = parse_prompt_ids(args.prompt)
    else:
        raise SystemExit("give --prompt (token ids) or --prompt-len N")
    sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, seed=args.seed)

    def on_token(_i: int, tok: int) -> bool:
        print(tok, end=" ", flush=True)
        return True

    if cfg.diagnostics.parityDump:
        log(f"diagnostics.parityDump={cfg.diagnostics.parityDump}: every layer writes its stages during the prefill "
            f"({len(prompt)} tokens), synchronising at each")
    prof = None
    if cfg.diagnostics.profile:
        from torch.profiler import ProfilerActivity, profile
        prof = profile(activities=[ProfilerActivity.CUDA])
        prof.__enter__()
    res = engine.generate([prompt], max_new_tokens=args.max_new, sampling=sp, on_token=on_token)[0]
    print()
    if prof is not None:
        import torch
        torch.cuda.synchronize()
        prof.__exit__(None, None, None)
        print_kernel_shares(prof)
    st = res.stats
    n = st.generated_tokens
    if st.finish_reason.startswith("rejected") or st.finish_reason == "out_of_pages":
        print(f"error: {st.finish_reason}", file=sys.stderr)
        return 1
    print(f"generated {n}" + (" (hit stop)" if st.hit_stop else ""))
    print(f"prefill {st.prefill_ms:.1f} ms ({st.prompt_tokens} tokens, {len(engine.model.schedule)} blocks)")
    per = st.decode_ms / (n - 1) if n > 1 else 0.0
    print(f"decode {st.decode_ms:.1f} ms ({per:.2f} ms/token)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
