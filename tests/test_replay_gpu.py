"""Replay on the GPU: the same requests whole, with the last 32 tokens one by one, in portions of
changing size, and mixed with other requests over a pool so small that pages are used again; in
32-bit and in bfloat16; every returned row against the plain implementation."""
import numpy as np
import pytest

import replay_util as ru
from conftest import TINY, random_tokens

pytestmark = pytest.mark.gpu

# |engine - plain| bounds, set from the formats: fp32 sums of a few hundred terms of size <= 1
# against float64; bfloat16 rounds activations to 8 bits of mantissa between the kernels.
TOL = {"float32": dict(max_abs=3e-5, mean_abs=3e-6), "bfloat16": dict(max_abs=4e-2, mean_abs=6e-3)}

LENGTHS = {"A": [5, 70, 133, 260], "B": [1, 9, 77, 300], "C": [33, 64, 150], "D": [40, 129, 257], "E": [17, 230, 301],
           "F": [1, 9, 40, 77, 128, 200], "G": [9, 70, 150], "H": [9, 70, 150], "I": [9, 70, 150]}


def requests_for(name, plain_model):
    V = plain_model.V
    return {f"{name}{i}": random_tokens(V, n, 100 * i + n) for i, n in enumerate(LENGTHS[name])}


def check(trace, outputs, reqs, ref, dtype, what):
    got = ru.collect(trace, outputs)
    tol = TOL[dtype]
    for rid, toks in reqs.items():
        rows = np.stack([got[(rid, p)] for p in range(len(toks))])
        err = np.abs(rows - ref[rid])
        scale = max(np.abs(ref[rid]).max(), 1.0)
        worst = np.unravel_index(err.argmax(), err.shape)
        assert err.max() <= tol["max_abs"] * scale, (
            f"{what} {dtype} request {rid}: max error {err.max():.3g} at position {worst[0]} (of {len(toks)}), "
            f"first position above the bound: {int(np.argmax(err.max(axis=1) > tol['max_abs'] * scale))}")
        assert err.mean() <= tol["mean_abs"] * scale, f"{what} {dtype} request {rid}: mean error {err.mean():.3g}"
    return got


def every_way_of_cutting(folder, dtype, reqs, ref, page_size=16, seed=7):
    """The same requests whole, with the last 32 tokens one by one, in portions of changing size and mixed with
    each other (each request twice, up to four live, in the smallest pool that holds them), every returned row
    against ``ref``; in float32 every cutting must give the whole run's rows bit for bit."""
    results = {}
    # each request alone and whole
    t = ru.Trace()
    for rid, toks in reqs.items():
        ru.whole(t, rid, toks)
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    results["whole"] = check(t, out, reqs, ref, dtype, "whole")
    # most of it in one step, the last 32 tokens one by one
    t = ru.Trace()
    for rid, toks in reqs.items():
        ru.tail_one_by_one(t, rid, toks, 32)
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    results["tail"] = check(t, out, reqs, ref, dtype, "tail one by one")
    # portions of changing size, down to two tokens
    t = ru.Trace()
    for i, (rid, toks) in enumerate(reqs.items()):
        ru.chunks(t, rid, toks, [[17, 7, 5, 3, 2], [2, 64, 3, 31], [33, 2, 2, 16]][i % 3])
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    results["chunks"] = check(t, out, reqs, ref, dtype, "portions")
    # mixed, up to four live, in the smallest pool that holds them: pages are used again
    t = ru.Trace()
    twice = dict(reqs)
    twice.update({rid + "x": toks for rid, toks in reqs.items()})       # the same requests a second time, later
    ru.mixed(t, twice, seed=seed)
    out, runner = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    ref2 = dict(ref)
    ref2.update({rid + "x": ref[rid] for rid in reqs})
    results["mixed"] = check(t, out, twice, ref2, dtype, "mixed")
    assert runner.manager.reuses() > 0, "the pool was large enough that no page was used again"
    for g in runner.manager.groups:
        assert runner.manager.free_pages(g) == runner.manager.total_pages(g)

    if dtype == "float32":
        # the 32-bit kernels sum in an order fixed by position: cutting changes nothing at all
        for mode in ("tail", "chunks", "mixed"):
            for key, row in results["whole"].items():
                assert np.array_equal(results[mode][key], row), f"{mode}: {key} differs from the whole run"
        for rid in reqs:
            for p in range(len(reqs[rid])):
                assert np.array_equal(results["mixed"][(rid + "x", p)], results["whole"][(rid, p)])
    return results


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_every_way_of_cutting_matches_the_plain_implementation(name, dtype, model_folders, plain_models):
    pm = plain_models(name, dtype)
    reqs = requests_for(name, pm)
    ref = {rid: pm.logits(t) for rid, t in reqs.items()}
    every_way_of_cutting(model_folders(name, dtype), dtype, reqs, ref, seed=len(name) + 7)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("D", 8), ("B", 32), ("E", 64), ("A", 8)])
def test_every_way_of_cutting_at_other_page_sizes(name, page_size, dtype, model_folders, plain_models):
    """The engine's other page sizes (8, 32, 64): a window over pages of 32 and 64, head sizes 128 and 64 on the
    tensor-core kernels, the generic kernel at 16 and 32."""
    pm = plain_models(name, dtype)
    reqs = requests_for(name, pm)
    ref = {rid: pm.logits(t) for rid, t in reqs.items()}
    every_way_of_cutting(model_folders(name, dtype), dtype, reqs, ref, page_size=page_size, seed=page_size)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_program_itself(dtype, model_folders, plain_models, tmp_path):
    """bin/trace_run as a user runs it: protocol, files, and the same numbers."""
    name = "B"
    folder = model_folders(name, dtype)
    pm = plain_models(name, dtype)
    reqs = {f"r{i}": random_tokens(pm.V, n, 11 + i) for i, n in enumerate([3, 90, 41, 150, 64])}
    ref = {rid: pm.logits(t) for rid, t in reqs.items()}
    t = ru.Trace()
    ru.mixed(t, reqs, seed=3)
    # a step that wants nothing writes no file
    t.step([("last", [1, 2, 3], [])], end=["last"])
    out = ru.run_program(folder, dtype, t, t.max_live_tokens(), str(tmp_path / "out"), pm.V)
    check(t, out, reqs, ref, dtype, "program")


def test_long_decoding_and_first_tokens(model_folders, plain_models):
    """One token at a time from the very first token on, over many pages."""
    for name, dtype in (("A", "float32"), ("E", "bfloat16")):
        pm = plain_models(name, dtype)
        toks = random_tokens(pm.V, 200, 5)
        ref = {"d": pm.logits(toks)}
        t = ru.Trace()
        ru.chunks(t, "d", toks, [1])
        out, _ = ru.run_in_process(model_folders(name, dtype), dtype, t, t.max_live_tokens())
        check(t, out, {"d": toks}, ref, dtype, "decode from the first token")


def test_step_refuses_what_it_cannot_run(model_folders):
    from mimirmind_b200.engine.loader import load_model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry, StepError
    model, _ = load_model(model_folders("A"), "float32")
    r = ModelRunner(model, 16, 4, 4)
    r.add_request("a")
    with pytest.raises(StepError, match="out of cache pages"):
        r.step([StepEntry("a", [1] * 65, [0])])
    assert r.manager.free_pages() == 4 and r.length("a") == 0       # nothing was taken
    with pytest.raises(StepError, match="token id"):
        r.step([StepEntry("a", [1, 256], [0])])
    with pytest.raises(StepError, match="unknown request"):
        r.step([StepEntry("zz", [1], [0])])
    with pytest.raises(StepError, match="wanted place"):
        r.step([StepEntry("a", [1, 2], [2])])
    assert r.step([StepEntry("a", [1, 2], [])]) is None
    assert r.length("a") == 2
