"""Generation through the Python entry point and the command line: greedy tokens equal the plain
implementation's, sampling is seeded per request, running out of pages changes no output."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_qwen2 as plain
from conftest import ROOT, TINY, random_tokens

pytestmark = pytest.mark.gpu


def check_greedy(pm, prompt, tokens, margin):
    """Every generated token is the plain implementation's argmax given the same history, or lies within
    ``margin`` of it (a near-tie may legitimately flip in reduced precision).  Returns exact matches."""
    toks, exact = list(prompt), 0
    for i, tok in enumerate(tokens):
        row = pm.logits(toks)[-1]
        best = int(plain.greedy(row.astype(np.float32)))
        assert row[tok] >= row[best] - margin, f"token {i}: engine chose {tok} ({row[tok]:.4f}), plain {best} ({row[best]:.4f})"
        exact += tok == best
        toks.append(tok)
    return exact


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("D", "bfloat16"), ("E", "bfloat16")])
def test_greedy_generation_equals_plain(name, dtype, model_folders, plain_models):
    from mimirmind_b200 import Engine
    pm = plain_models(name, dtype)
    prompts = [random_tokens(pm.V, n, 40 + n) for n in (5, 17, 33, 64)]
    eng = Engine.from_folder(model_folders(name, dtype), dtype=dtype, page_size=16, cache_tokens=1024, max_context=512,
                             token_budget=48, max_active=4)
    res = eng.generate(prompts, max_new_tokens=16)
    margin = 1e-4 if dtype == "float32" else 0.08
    exact = 0
    for p, r in zip(prompts, res):
        assert r.stats.generated_tokens == 16 and r.stats.finish_reason == "length"
        exact += check_greedy(pm, p, r.tokens, margin)
    assert exact >= (64 if dtype == "float32" else 56)
    assert eng.runner.manager.free_pages() == eng.runner.manager.total_pages()


def test_chunked_mixed_temperature_run_is_seeded_and_batch_independent(model_folders, plain_models):
    """Six requests, prompt portions of 32 mixed with decoding, temperature 0.8 with fixed seeds."""
    from mimirmind_b200 import Engine, SamplingParams
    pm = plain_models("B", "float32")
    prompts = [random_tokens(pm.V, n, n) for n in (1, 9, 40, 77, 128, 200)]
    sp = [SamplingParams(temperature=0.8, seed=1000 + i) for i in range(6)]
    kw = dict(dtype="float32", page_size=16, max_context=512)
    eng = Engine.from_folder(model_folders("B", "float32"), cache_tokens=4096, token_budget=64, max_active=6, prefill_chunk=32, **kw)
    a = eng.generate(prompts, max_new_tokens=24, sampling=sp)
    b = eng.generate(prompts, max_new_tokens=24, sampling=sp)
    assert [r.tokens for r in a] == [r.tokens for r in b]
    assert len({tuple(r.tokens) for r in a}) == 6
    # one request alone gives the same stream as in the batch
    solo = Engine.from_folder(model_folders("B", "float32"), cache_tokens=1024, token_budget=512, max_active=1, **kw)
    for i in (0, 3, 5):
        assert solo.generate([prompts[i]], max_new_tokens=24, sampling=sp[i])[0].tokens == a[i].tokens
    # every sampled token is what the plain sampler draws from the plain logits (when not a near-tie)
    toks = list(prompts[2])
    for step, tok in enumerate(a[2].tokens[:6]):
        row = pm.logits(toks)[-1]
        assert tok == plain.sample(row, 0.8, 0, 1.0, plain.uniform_from(1002, step))
        toks.append(tok)


def test_the_baselines_second_tiny_workload_as_written(model_folders, plain_models):
    """The baseline's second tiny configuration as it stands there (no window, context 256): six requests with prompts
    of 1, 9, 40, 77, 128 and 200 tokens, prompt portions of 32 beside decoding, 24 tokens each at temperature 0.8 with
    fixed seeds, in float32.  Every sampled token of every request is the one the plain sampler draws from the plain
    implementation's logits for the same history."""
    from mimirmind_b200 import Engine, SamplingParams
    pm = plain_models("F", "float32")
    prompts = [random_tokens(pm.V, n, 7 * n + 1) for n in (1, 9, 40, 77, 128, 200)]
    sp = [SamplingParams(temperature=0.8, seed=4000 + i) for i in range(6)]
    eng = Engine.from_folder(model_folders("F", "float32"), dtype="float32", page_size=16, max_context=256, cache_tokens=6 * 256,
                             token_budget=64, max_active=6, prefill_chunk=32)
    res = eng.generate(prompts, max_new_tokens=24, sampling=sp, use_eos=False)
    assert eng.last_metrics.steps > 12                      # portions of 32 under a budget of 64: the prompts took many steps
    for i, (p, r) in enumerate(zip(prompts, res)):
        assert r.stats.finish_reason == "length" and len(r.tokens) == 24
        toks = list(p)
        for step, tok in enumerate(r.tokens):
            row = pm.logits(toks)[-1]
            assert tok == plain.sample(row, 0.8, 0, 1.0, plain.uniform_from(4000 + i, step)), f"request {i}, token {step}"
            toks.append(tok)
    assert eng.runner.manager.free_pages() == eng.runner.manager.total_pages()


def test_running_out_of_pages_changes_no_output(model_folders):
    from mimirmind_b200 import Engine
    folder = model_folders("A", "float32")
    prompts = [random_tokens(256, n, n) for n in (30, 45, 20, 50)]
    roomy = Engine.from_folder(folder, dtype="float32", cache_tokens=2048, max_context=256, token_budget=64, max_active=4)
    tight = Engine.from_folder(folder, dtype="float32", cache_tokens=160, max_context=256, token_budget=64, max_active=4)
    a = roomy.generate(prompts, max_new_tokens=40)
    b = tight.generate(prompts, max_new_tokens=40)
    assert tight.last_metrics.preempted > 0 and roomy.last_metrics.preempted == 0
    assert [r.tokens for r in a] == [r.tokens for r in b]
    assert sum(r.stats.preemptions for r in b) == tight.last_metrics.preempted
    # a request that can never fit is reported, not hung
    lone = Engine.from_folder(folder, dtype="float32", cache_tokens=64, max_context=256, token_budget=64, max_active=2)
    r = lone.generate([random_tokens(256, 60, 1)], max_new_tokens=40)[0]
    assert r.stats.finish_reason == "out_of_pages" and 1 <= len(r.tokens) < 40
    r = lone.generate([random_tokens(256, 100, 1)], max_new_tokens=4)[0]
    assert r.stats.finish_reason.startswith("rejected")


def test_stop_ids_and_callback(model_folders):
    from mimirmind_b200 import Engine
    eng = Engine.from_folder(model_folders("A", "float32"), dtype="float32", cache_tokens=512, max_context=256)
    p = random_tokens(256, 12, 3)
    free = eng.generate([p], max_new_tokens=10)[0].tokens
    stopped = eng.generate([p], max_new_tokens=10, stop_ids=[free[3]])[0]
    first = free.index(free[3])
    assert stopped.tokens == free[:first + 1] and stopped.stats.hit_stop      # the stop token is part of the output
    seen = []
    eng.generate([p], max_new_tokens=10, on_token=lambda i, t: (seen.append(t), len(seen) < 4)[1])
    assert seen == free[:4]


def test_command_line_smoke(model_folders, tmp_path):
    cfg = {"defaultModel": "m", "models": [{"id": "m", "path": model_folders("A", "float32")}],
           "runtime": {"dtype": "float32", "maxContextTokens": 256, "cacheTokens": 512}}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    cmd = [sys.executable, os.path.join(ROOT, "bin", "mimirmind"), "smoke", "--config", str(tmp_path / "config.json"),
           "--prompt", "5 17 3 200", "--max-new", "6"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()
    assert len(lines[0].split()) == 6 and lines[1] == "generated 6"
    assert lines[2].startswith("prefill ") and "(4 tokens, 2 blocks)" in lines[2] and lines[3].startswith("decode ")
    missing = subprocess.run(cmd[:3] + ["--config", str(tmp_path / "nope.json")] + cmd[5:], capture_output=True, text=True, timeout=300)
    assert missing.returncode == 2 and "not found" in missing.stderr
    # random-weights mode writes a folder the engine loads
    (tmp_path / "mc.json").write_text(json.dumps(TINY["C"]))
    rw = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mimirmind"), "random-weights", "--model-config",
                         str(tmp_path / "mc.json"), "--seed", "9", "--out", str(tmp_path / "rw"), "--dtype", "bfloat16"],
                        capture_output=True, text=True, timeout=300)
    assert rw.returncode == 0, rw.stderr
    assert os.path.isfile(tmp_path / "rw" / "model.safetensors") and json.load(open(tmp_path / "rw" / "config.json"))["torch_dtype"] == "bfloat16"


def test_many_requests_small_pool_graphs_and_preemption_agree_with_plain_stepping(model_folders):
    """Twenty requests of random lengths through a pool that holds about four of them, with graph replay on:
    admissions, portions, decode runs, horizons cut short by missing pages and preemptions interleave; every
    request must produce exactly what it produces alone without graphs."""
    import random
    from mimirmind_b200 import Engine
    folder = model_folders("D", "bfloat16")
    rng = random.Random(11)
    prompts = [random_tokens(331, rng.randint(3, 150), 1000 + i) for i in range(20)]
    news = 40
    busy = Engine.from_folder(folder, dtype="bfloat16", cache_tokens=640, max_context=512, token_budget=96, max_active=6,
                              prefill_chunk=48, use_graphs=True)
    busy.graph_min_steps = 4
    got = busy.generate(prompts, max_new_tokens=news)
    assert busy.last_metrics.preempted > 0 and busy.graph_steps > 0
    assert all(r.stats.finish_reason == "length" and len(r.tokens) == news for r in got)
    assert busy.runner.manager.free_pages() == busy.runner.manager.total_pages()
    busy.runner.manager.check()
    alone = Engine.from_folder(folder, dtype="bfloat16", cache_tokens=1024, max_context=512, token_budget=512, max_active=1, use_graphs=False)
    same = 0
    for p, r in zip(prompts, got):
        want = alone.generate([p], max_new_tokens=news)[0].tokens
        same += want == r.tokens
    # bfloat16: a prompt cut into other portions, or a token decoded by the other attention kernel, may round a
    # near-tie the other way; most streams must still be identical token for token
    assert same >= 14, f"only {same} of 20 streams identical"


def test_many_requests_in_32_bit_are_identical_token_for_token(model_folders):
    """The same storm in float32, where no kernel's result depends on cutting or batching: every stream is equal."""
    import random
    from mimirmind_b200 import Engine
    folder = model_folders("B", "float32")
    rng = random.Random(5)
    prompts = [random_tokens(384, rng.randint(1, 120), 2000 + i) for i in range(16)]
    busy = Engine.from_folder(folder, dtype="float32", cache_tokens=512, max_context=512, token_budget=64, max_active=5,
                              prefill_chunk=32, use_graphs=True)
    busy.graph_min_steps = 4
    got = busy.generate(prompts, max_new_tokens=30)
    assert busy.last_metrics.preempted > 0 and busy.graph_steps > 0
    alone = Engine.from_folder(folder, dtype="float32", cache_tokens=1024, max_context=512, token_budget=512, max_active=1, use_graphs=False)
    for i, (p, r) in enumerate(zip(prompts, got)):
        assert alone.generate([p], max_new_tokens=30)[0].tokens == r.tokens, f"request {i}"


def _wide_tiny_model(tmp_path, dtype, layers=2, hidden=256):
    from mimirmind_b200.engine.loader import load_model
    from mimirmind_b200.weights import write_random_model
    cfg = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=400, hidden_size=hidden, intermediate_size=352,
               num_hidden_layers=layers, num_attention_heads=4, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6,
               rope_theta=10000.0, max_position_embeddings=8192, tie_word_embeddings=False)
    write_random_model(str(tmp_path), cfg, 21, dtype)
    return load_model(str(tmp_path), dtype=dtype)[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_library_executor_equals_the_python_part_classes(tmp_path, dtype):
    """A model whose parts all have native classes steps inside the library (one call per step); the same model with
    the executor switched off steps through the Python part classes.  Both launch the same kernels of this library, so
    mixed steps (a portion beside decoded tokens, portions of two requests, decoding alone) give equal logits: bit for
    bit in float32 and for steps of at most 64 tokens in bfloat16 (own kernels only); where the plain products of
    longer steps go to the library product (cuBLASLt here, through torch there) they agree to bfloat16 rounding."""
    import torch
    from mimirmind_b200.engine import native
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    from mimirmind_b200.kernels import ops
    model = _wide_tiny_model(tmp_path, dtype)
    a, b, c = random_tokens(400, 700, 1), random_tokens(400, 300, 2), random_tokens(400, 90, 3)
    steps = [
        [("a", a[:600], [599])],                                   # a long portion alone
        [("a", a[600:640], [0, 39]), ("b", b[:9], [8])],           # 49 tokens: the fused small-step kernels
        [("a", a[640:641], [0]), ("b", b[9:10], [0]), ("c", c[:30], [29])],
        [("b", b[10:300], [289]), ("c", c[30:90], []), ("a", a[641:642], [0])],   # two portions beside a decoded token
        [("a", a[642:643], [0]), ("b", [7], [0]), ("c", [9], [0])],                # decoding only
    ]

    def run(runner):
        outs = []
        for rid in "abc":
            runner.add_request(rid)
        for step in steps:
            out = runner.step([StepEntry(r, t, w) for r, t, w in step])
            outs.append(out.cpu().numpy())
        runner.manager.check()
        return outs

    lib_runner = ModelRunner(model, 16, 256, 4, max_seq_len=4096)
    assert lib_runner.native is not None
    got = run(lib_runner)
    assert lib_runner.native.steps() == len(steps)
    old = native.ENABLED
    try:
        native.ENABLED = False
        py_runner = ModelRunner(model, 16, 256, 4, max_seq_len=4096)
    finally:
        native.ENABLED = old
    assert py_runner.native is None
    want = run(py_runner)
    ops.check_tcgen05_errors(torch.device("cuda"))
    for i, (g, w) in enumerate(zip(got, want)):
        small = sum(len(t) for _, t, _ in steps[i]) <= 64
        if dtype == "float32" or small:
            assert np.array_equal(g, w), f"step {i}"
        else:
            assert np.abs(g - w).max() <= 2.0 ** -6 * np.abs(w).max(), f"step {i}"


def test_portions_back_to_back_never_overtake_their_staging_buffers(tmp_path):
    """Portions whose logits nobody reads are launched without the host ever waiting for the device, so the host runs
    many steps ahead; every step's integers go through one of a few pinned buffers, which must not be rewritten before
    the copy that reads it has run.  Twelve portions back to back and then the last one: its logits equal, bit for
    bit, those of the same steps with a synchronisation after each."""
    import torch
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    model = _wide_tiny_model(tmp_path, "bfloat16", layers=8, hidden=1024)
    toks = random_tokens(400, 13 * 256 + 40, 5)

    def run(sync):
        runner = ModelRunner(model, 16, 512, 2, max_seq_len=8192)
        assert runner.native is not None
        runner.add_request("r")
        for i in range(13):
            assert runner.step([StepEntry("r", toks[256 * i:256 * (i + 1)], [])]) is None
            if sync:
                torch.cuda.synchronize()
        out = runner.step([StepEntry("r", toks[13 * 256:], [39])])
        return out.cpu().numpy()

    assert np.array_equal(run(False), run(True))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_penalties_and_softcap_inside_the_captured_step_equal_the_eager_steps(model_folders, dtype):
    """Repetition / frequency / presence penalties and the soft-cap run inside the decode graph over rings of recent
    tokens kept on the device: same tokens as stepping eagerly, where the host rebuilds the window every step.
    Windows shorter and longer than the histories, a request without penalties beside them, greedy and sampled."""
    from mimirmind_b200 import Engine, SamplingParams
    name = "B" if dtype == "float32" else "E"
    eng = Engine.from_folder(model_folders(name, dtype), dtype=dtype, cache_tokens=2048, max_context=TINY[name]["max_position_embeddings"],
                             token_budget=64, max_active=4)
    V = TINY[name]["vocab_size"]
    prompts = [random_tokens(V, n, 40 + n) for n in (9, 30, 5, 17)]
    for greedy in (True, False):
        t = 0.0 if greedy else 0.9
        params = [SamplingParams(temperature=t, seed=5, repetition_penalty=1.3, penalty_window=8),
                  SamplingParams(temperature=t, seed=6, frequency_penalty=0.4, presence_penalty=0.2, penalty_window=200, final_logit_softcap=30.0),
                  SamplingParams(temperature=t, seed=7),
                  SamplingParams(temperature=t, seed=8, top_k=20, repetition_penalty=0.8, frequency_penalty=0.1, penalty_window=33)]
        outs = {}
        for graphs in (False, True):
            eng.use_graphs = graphs
            before = eng.graph_steps
            res = eng.generate(prompts, max_new_tokens=40, sampling=params, use_eos=False)
            outs[graphs] = [r.tokens for r in res]
            assert (eng.graph_steps > before) == graphs
        assert outs[True] == outs[False], greedy
        # the penalties matter: without them the first request repeats more
        eng.use_graphs = True
        plain_run = eng.generate(prompts[:1], max_new_tokens=40, sampling=SamplingParams(temperature=t, seed=5), use_eos=False)[0].tokens
        assert plain_run != outs[True][0]


def test_requests_added_while_others_run_get_the_tokens_they_get_alone(model_folders):
    """The serving loop: two requests start, a third and a fourth are submitted between steps (one while the others
    decode in captured steps), one is cancelled by its callback.  In float32 every request's tokens equal those it
    gets alone, token for token."""
    from mimirmind_b200 import Engine, SamplingParams
    eng = Engine.from_folder(model_folders("A", "float32"), dtype="float32", cache_tokens=1024,
                             max_context=TINY["A"]["max_position_embeddings"], token_budget=32, max_active=4)
    V = TINY["A"]["vocab_size"]
    prompts = [random_tokens(V, n, 70 + n) for n in (20, 7, 45, 3)]
    alone = [eng.generate([p], max_new_tokens=30, use_eos=False)[0].tokens for p in prompts]
    loop = eng.serve(max_graph_steps=8)
    seen = {i: [] for i in range(4)}
    stop_third_after = 5

    def cb(i):
        def on_token(tok):
            seen[i].append(tok)
            return not (i == 2 and len(seen[i]) >= stop_third_after)
        return on_token

    h = [loop.submit(prompts[0], 30, use_eos=False, on_token=cb(0)), loop.submit(prompts[1], 30, use_eos=False, on_token=cb(1))]
    for _ in range(3):
        assert loop.step()
    h.append(loop.submit(prompts[2], 30, use_eos=False, on_token=cb(2)))
    while not (loop.sched.all_decoding() and len(seen[0]) >= 10):
        assert loop.step()
    h.append(loop.submit(prompts[3], 30, SamplingParams(), use_eos=False, on_token=cb(3)))      # arrives during decoding
    loop.run_until_idle()
    assert not loop.has_work() and all(loop.finished(x) for x in h)
    res = [loop.result(x) for x in h]
    for i in (0, 1, 3):
        assert res[i].tokens == alone[i] == seen[i], i
        assert res[i].stats.finish_reason == "length" and res[i].stats.generated_tokens == 30
    assert res[2].tokens == alone[2][:stop_third_after] and res[2].stats.finish_reason == "cancelled"
    assert eng.graph_steps > 0
    eng.runner.manager.check()
    assert not eng.runner.manager.live_requests()


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("D", "bfloat16")])
def test_stage_dumps_of_a_prefill_and_the_decode_trace(name, dtype, model_folders, plain_models, tmp_path):
    """diagnostics.parityDump: every layer's stages of the prefill in the reference's file format, against the
    plain implementation's stages; diagnostics.traceDecodeFile: a line per decode step.  The tokens generated with the
    diagnostics on are those generated without them."""
    import plain_qwen2 as plain
    from mimirmind_b200 import Engine
    from mimirmind_b200.engine.diagnostics import read_stage_dump
    pm = plain_models(name, dtype)
    prompt = random_tokens(pm.V, 45, 3)
    eng = Engine.from_folder(model_folders(name, dtype), dtype=dtype, cache_tokens=512,
                             max_context=TINY[name]["max_position_embeddings"], token_budget=64, max_active=2)
    want = eng.generate([prompt], max_new_tokens=12, use_eos=False)[0].tokens
    prefix, trace = str(tmp_path / "dump"), str(tmp_path / "trace.ndjson")
    eng.set_diagnostics(parity_dump=prefix, trace_decode_file=trace)
    got = eng.generate([prompt], max_new_tokens=12, use_eos=False)[0].tokens
    eng.set_diagnostics()
    assert got == want
    x = plain.embedding(pm.w["model.embed_tokens.weight"], prompt)
    block, rows = read_stage_dump(prefix + "-blk0-inp_scaled.bin")
    assert block == 0 and rows.shape == x.shape
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert np.abs(rows - x).max() <= tol * max(1.0, np.abs(x).max())
    pos = np.arange(len(prompt))
    for i in range(pm.L):
        st = plain.block_stages(pm, i, x, pos)
        for stage, ref in st.items():
            block, rows = read_stage_dump(f"{prefix}-blk{i}-{stage}.bin")
            assert block == i and rows.shape == ref.shape, (i, stage, rows.shape, ref.shape)
            assert np.abs(rows - ref).max() <= tol * max(1.0, np.abs(ref).max()), (i, stage)
        x = st["l_out"]
    lines = [json.loads(l) for l in open(trace)]
    assert len(lines) == 11 and [l["step"] for l in lines] == list(range(11))        # the first token comes from the prefill
    assert all(l["tokens"] == 1 and l["wall_ms"] > 0 and {"sm_mhz", "gpu_c"} <= set(l) for l in lines)


def test_command_line_dump_dir_and_profile(model_folders, tmp_path):
    cfg = {"defaultModel": "m", "models": [{"id": "m", "path": model_folders("A", "float32")}],
           "runtime": {"dtype": "float32", "maxContextTokens": 256, "cacheTokens": 512}, "diagnostics": {"profile": True}}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    cmd = [sys.executable, os.path.join(ROOT, "bin", "mimirmind"), "smoke", "--config", str(tmp_path / "config.json"),
           "--prompt", "5 17 3 200 9", "--max-new", "4", "--dump-dir", str(tmp_path / "dumps")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert "profile:" in out.stdout and "% " in out.stdout
    names = sorted(os.listdir(tmp_path / "dumps"))
    assert "engine-blk0-inp_scaled.bin" in names and "engine-blk1-l_out.bin" in names and len(names) == 1 + 2 * 7


def test_a_step_that_fails_ends_its_requests_and_nothing_else(model_folders):
    """An exception out of a step: the requests in it finish with "error: ...", their pages go back, a request that was
    still waiting runs afterwards, and so does the next call."""
    from mimirmind_b200 import Engine
    from mimirmind_b200.engine import native
    old = native.ENABLED
    try:
        native.ENABLED = False        # the failure is injected into the Python loop's step; the library's step is failed in the next test
        eng = Engine.from_folder(model_folders("A", "float32"), dtype="float32", cache_tokens=512, max_context=256,
                                 token_budget=64, max_active=2)
    finally:
        native.ENABLED = old
    prompts = [random_tokens(256, n, n) for n in (20, 30, 10)]
    alone = [eng.generate([p], max_new_tokens=8, use_eos=False)[0].tokens for p in prompts]
    loop = eng.serve()
    h = [loop.submit(p, 8, use_eos=False) for p in prompts]          # two run, the third waits (max_active=2)
    real, calls = eng._run_plan, []

    def failing(plan):
        calls.append(len(plan))
        if len(calls) == 1:
            raise RuntimeError("injected")
        return real(plan)
    eng._run_plan = failing
    with pytest.raises(RuntimeError, match="injected"):
        loop.step()
    assert loop.finished(h[0]) and loop.finished(h[1]) and not loop.finished(h[2])
    assert loop.result(h[0]).stats.finish_reason.startswith("error: RuntimeError: injected")
    loop.run_until_idle()
    eng._run_plan = real
    assert loop.result(h[2]).tokens == alone[2] and loop.result(h[2]).stats.finish_reason == "length"
    assert eng.runner.manager.free_pages() == eng.runner.manager.total_pages()
    assert eng.generate([prompts[0]], max_new_tokens=8, use_eos=False)[0].tokens == alone[0]


@pytest.mark.parametrize("native_steps", [True, False])
def test_a_kernel_that_gave_up_a_wait_fails_the_steps_requests(model_folders, native_steps):
    """The kernels with bounded waits set a flag on the device when a wait runs out.  The flag comes back to the host with
    every step's tokens; when it is set the step fails like any step that raised: its requests end with "error: ...",
    their pages go back, the flag is cleared and the loop goes on.  No kernel is made to give up here: the test sets
    the flag itself, before an eager step and before a captured decode step."""
    import torch
    from mimirmind_b200 import Engine
    from mimirmind_b200.engine import native
    from mimirmind_b200.kernels import ops
    from mimirmind_b200.kernels.lib import KernelError
    old = native.ENABLED
    try:
        native.ENABLED = native_steps
        eng = Engine.from_folder(model_folders("D", "bfloat16"), dtype="bfloat16", cache_tokens=1024, max_context=256,
                                 token_budget=64, max_active=2)
    finally:
        native.ENABLED = old
    assert (eng.runner.native is not None) == native_steps
    eng.graph_min_steps = 4
    flag = ops.tcgen05_error_flag(torch.device("cuda", torch.cuda.current_device()))
    prompts = [random_tokens(331, n, n) for n in (20, 30, 10)]
    alone = [eng.generate([p], max_new_tokens=12, use_eos=False)[0].tokens for p in prompts]
    # an eager step (two prompts in one step, the third waits)
    loop = eng.serve()
    h = [loop.submit(p, 12, use_eos=False) for p in prompts]
    flag.fill_(1)
    with pytest.raises(KernelError, match="gave up"):
        loop.step()
    assert int(flag.item()) == 0
    assert loop.finished(h[0]) and loop.finished(h[1]) and not loop.finished(h[2])
    assert loop.result(h[0]).stats.finish_reason.startswith("error: KernelError")
    loop.run_until_idle()
    assert loop.result(h[2]).tokens == alone[2]
    assert eng.runner.manager.free_pages() == eng.runner.manager.total_pages()
    # a captured decode step: the flag rides with the tokens of the step
    loop = eng.serve()
    h = [loop.submit(p, 12, use_eos=False) for p in prompts[:2]]
    loop.step()                                   # both prompts, first tokens
    assert loop.sched.all_decoding()
    flag.fill_(1)
    graph_steps = eng.graph_steps
    with pytest.raises(KernelError, match="gave up"):
        loop.step()
    assert eng.graph_steps > graph_steps and int(flag.item()) == 0
    assert all(loop.finished(x) and loop.result(x).stats.finish_reason.startswith("error: KernelError") for x in h)
    assert eng.runner.manager.free_pages() == eng.runner.manager.total_pages()
    again = eng.generate(prompts, max_new_tokens=12, use_eos=False)           # the engine is as usable as before
    assert [r.stats.finish_reason for r in again] == ["length"] * 3 and again[0].tokens[:3] == alone[0][:3]


def test_random_settings_many_engines_in_one_process(model_folders):
    """Engines come and go in one process, each with random batch, budget, pool, portion cap and sampling (greedy or
    sampled, with and without top-k, top-p and penalties); captured decode runs, preemption and admission interleave.
    In float32 every request's tokens equal those it gets alone without graphs."""
    import gc
    import random
    from mimirmind_b200 import Engine, SamplingParams
    rng = random.Random(5)
    graph_steps = preempted = 0
    for it in range(12):
        name = rng.choice(["A", "B", "C"])
        V, ctx = TINY[name]["vocab_size"], min(512, TINY[name]["max_position_embeddings"])
        n, news, sampled = rng.randint(1, 9), rng.randint(2, 36), rng.random() < 0.5
        prompts = [random_tokens(V, rng.randint(1, 110), rng.randint(0, 10 ** 6)) for _ in range(n)]

        def params(i):
            if not sampled:
                return SamplingParams()
            kw = dict(temperature=rng.choice([0.7, 1.0]), seed=100 + i)
            if rng.random() < 0.4:
                kw.update(top_k=rng.choice([5, 40]))
            if rng.random() < 0.4:
                kw.update(top_p=0.9)
            if rng.random() < 0.3:
                kw.update(repetition_penalty=1.2, penalty_window=rng.choice([8, 64]))
            return SamplingParams(**kw)
        sp = [params(i) for i in range(n)]
        kw = dict(dtype="float32", max_context=ctx, token_budget=rng.choice([16, 48, 96, 512]), prefill_chunk=rng.choice([0, 0, 32]))
        busy = Engine.from_folder(model_folders(name, "float32"), cache_tokens=rng.choice([256, 640, 4096]),
                                  max_active=rng.choice([1, 2, 4, 8]), **kw)
        got = busy.generate(prompts, max_new_tokens=news, sampling=sp, use_eos=False)
        alone = Engine.from_folder(model_folders(name, "float32"), cache_tokens=4096, max_active=1, use_graphs=False, **kw)
        for i, p in enumerate(prompts):
            if got[i].stats.finish_reason.startswith("rejected") or got[i].stats.finish_reason == "out_of_pages":
                continue
            want = alone.generate([p], max_new_tokens=news, sampling=sp[i], use_eos=False)[0].tokens
            assert got[i].tokens == want, (it, name, i, kw)
        assert busy.runner.manager.free_pages() == busy.runner.manager.total_pages()
        graph_steps += busy.graph_steps
        preempted += busy.last_metrics.preempted
        del busy, alone
        if it % 3 == 0:
            gc.collect()
    assert graph_steps > 0


def test_captured_decode_steps_are_kept_up_to_a_limit(model_folders):
    from mimirmind_b200 import Engine
    eng = Engine.from_folder(model_folders("A", "float32"), dtype="float32", cache_tokens=2048, max_context=256,
                             token_budget=256, max_active=8)
    eng.max_decode_graphs = 2
    outs = {}
    for n in (1, 2, 3, 1, 3):
        prompts = [random_tokens(256, 10 + i, i) for i in range(n)]
        res = [r.tokens for r in eng.generate(prompts, max_new_tokens=12, use_eos=False)]
        assert outs.setdefault(n, res) == res                   # a batch size that comes back (recaptured or kept) gives the same tokens
        assert len(eng._sessions) <= 2
    assert [k[0] for k in eng._sessions] == [1, 3]              # least recently used went first
