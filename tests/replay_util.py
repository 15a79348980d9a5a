"""Builds replay traces (the JSON steps that bin/trace_run reads) for the ways of cutting the same
requests, runs them in process or through the program, and maps every returned logits row to its
(request, position)."""
import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def rounded(n: int, to: int = 64) -> int:
    return (n + to - 1) // to * to


class Trace:
    def __init__(self):
        self.steps: List[dict] = []
        self.rows: Dict[int, List[Tuple[str, int]]] = {}   # step → [(request, position)] in output order
        self._fed: Dict[str, int] = {}

    def step(self, entries: Sequence[Tuple[str, Sequence[int], Sequence[int]]], end: Sequence[str] = ()):
        """entries: (request id, tokens, wanted places among these tokens)."""
        i = len(self.steps)
        obj = {"step": i, "entries": [], "end": list(end)}
        rows = []
        for rid, toks, want in entries:
            base = self._fed.get(rid, 0)
            obj["entries"].append({"id": rid, "tokens": [int(t) for t in toks], "want": [int(w) for w in want]})
            rows += [(rid, base + w) for w in want]
            self._fed[rid] = base + len(toks)
        for rid in end:
            self._fed.pop(rid, None)
        self.steps.append(obj)
        if rows:
            self.rows[i] = rows
        return i

    def max_live_tokens(self) -> int:
        """Most tokens live requests hold at any time, each rounded up to a multiple of 64."""
        held: Dict[str, int] = {}
        worst = 0
        for s in self.steps:
            for e in s["entries"]:
                held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
            worst = max(worst, sum(rounded(v) for v in held.values()))
            for rid in s["end"]:
                held.pop(rid, None)
        return worst


def whole(trace: Trace, rid: str, toks: Sequence[int], end=True):
    trace.step([(rid, toks, list(range(len(toks))))], end=[rid] if end else [])


def tail_one_by_one(trace: Trace, rid: str, toks: Sequence[int], tail: int = 32):
    n = len(toks)
    head = max(n - tail, 1)
    trace.step([(rid, toks[:head], list(range(head)))])
    for p in range(head, n):
        trace.step([(rid, toks[p:p + 1], [0])], end=[rid] if p == n - 1 else [])
    if head == n:
        trace.steps[-1]["end"] = [rid]


def chunks(trace: Trace, rid: str, toks: Sequence[int], sizes: Sequence[int]):
    p, i, n = 0, 0, len(toks)
    while p < n:
        c = min(sizes[i % len(sizes)], n - p)
        trace.step([(rid, toks[p:p + c], list(range(c)))], end=[rid] if p + c == n else [])
        p += c
        i += 1


def mixed(trace: Trace, requests: Dict[str, Sequence[int]], seed: int, max_live: int = 4, decode_tail: int = 12):
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others; a request
    sometimes sits a step out; finished requests leave and later ones take their pages."""
    rng = np.random.RandomState(seed)
    waiting = list(requests.items())
    live: Dict[str, int] = {}
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.rand() < 0.6):
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, ends = [], []
        for rid in list(live):
            toks = requests[rid]
            fed, n = live[rid], len(toks)
            if len(live) > 1 and rng.rand() < 0.2:
                continue                                   # left out of this step, goes on later
            left = n - fed
            if left <= decode_tail:
                c = 1
            else:
                c = int(min(left - decode_tail, rng.choice([2, 3, 5, 16, 17, 31, 64])))
            entries.append((rid, toks[fed:fed + c], list(range(c))))
            live[rid] = fed + c
            if live[rid] == n:
                ends.append(rid)
        if entries:
            trace.step(entries, end=ends)
        for rid in ends:
            del live[rid]


def run_in_process(model_dir: str, dtype: str, trace: Trace, max_tokens: int, page_size: int = 16):
    """Same objects bin/trace_run drives.  Returns ({step: logits}, runner)."""
    from mimirmind_b200.engine.loader import load_model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    model, _ = load_model(model_dir, dtype)
    num_pages = (rounded(max_tokens) + page_size - 1) // page_size
    runner = ModelRunner(model, page_size=page_size, num_pages=num_pages, max_requests=8)
    out = {}
    for s in trace.steps:
        entries = []
        for e in s["entries"]:
            if not runner.manager.has(e["id"]):
                assert runner.add_request(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        lg = runner.step(entries)
        if lg is not None:
            out[s["step"]] = lg.float().cpu().numpy()
        for rid in s["end"]:
            runner.release(rid)
        runner.manager.check()
    return out, runner


def run_program(model_dir: str, dtype: str, trace: Trace, max_tokens: int, out_dir: str, vocab: int, env=None):
    """Through bin/trace_run as a user would: one JSON line per step, wait for ``done <step>``."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for s in trace.steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"expected 'done {s['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    out = {}
    for i, rows in trace.rows.items():
        a = np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4")
        out[i] = a.reshape(len(rows), vocab)
    assert sorted(int(f[:-4]) for f in os.listdir(out_dir) if f.endswith(".f32")) == sorted(trace.rows)
    return out


def collect(trace: Trace, outputs: Dict[int, np.ndarray]) -> Dict[Tuple[str, int], np.ndarray]:
    got = {}
    for i, rows in trace.rows.items():
        assert outputs[i].shape[0] == len(rows)
        for r, key in enumerate(rows):
            assert key not in got, f"position {key} returned twice"
            got[key] = outputs[i][r]
    return got
