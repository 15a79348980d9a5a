"""Trace replay over the engine's own step function (the program behind ``bin/trace_run``)."""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List

PAGE_SIZE = 16
TOKEN_ROUNDING = 64   # a request's token count is rounded up to this when sizing the pool
MAX_LIVE = 4


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token ids step by step and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE)
    args = ap.parse_args(argv)

    print(f"trace_run: loading {args.model} ({args.dtype})", file=sys.stderr, flush=True)
    from .engine.loader import load_model
    from .engine.runner import ModelRunner, StepEntry
    from .kernels import lib as kernel_lib

    kernel_lib.load(verbose=True)           # compiles at first call, with progress lines
    model, _cfg = load_model(args.model, args.dtype)
    ps = args.page_size
    rounded = ((args.max_tokens + TOKEN_ROUNDING - 1) // TOKEN_ROUNDING) * TOKEN_ROUNDING
    num_pages = (rounded + ps - 1) // ps
    runner = ModelRunner(model, page_size=ps, num_pages=num_pages, max_requests=MAX_LIVE * 2)
    os.makedirs(args.out, exist_ok=True)
    print(f"trace_run: ready, {num_pages} pages of {ps} tokens per cache group", file=sys.stderr, flush=True)

    import torch
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        step = obj["step"]
        entries: List[StepEntry] = []
        for e in obj.get("entries", []):
            rid = e["id"]
            if not runner.manager.has(rid):
                if not runner.add_request(rid):
                    raise RuntimeError(f"step {step}: no free request slot for '{rid}'")
            entries.append(StepEntry(rid, e["tokens"], e.get("want", [])))
        logits = runner.step(entries) if entries else None
        if logits is not None:
            host = logits.to(torch.float32).cpu().contiguous().numpy()
            runner.check_errors()           # no file is written from the output of a kernel that gave up a wait
            tmp = os.path.join(args.out, f".{step}.f32.tmp")
            host.astype("<f4").tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        else:
            torch.cuda.synchronize()
        for rid in obj.get("end", []):
            if runner.manager.has(rid):
                runner.release(rid)
        print(f"done {step}", flush=True)
    return 0
