"""The widths of the benchmark models against the plain implementation.

The tiny configurations never reach the kernels that only large shapes use: weight-streaming products with 8 row
tiles per CTA, the tcgen05 products with many tiles per CTA pair, K splits over clusters, the head over a wide
vocabulary.  Here one layer with the widths of the 7B-shaped model, one with those of the 14B-shaped one and one
with the feed-forward width of the 32B-shaped one (40 query heads over 8 KV heads: 5 per group) run every way of
cutting the replay test has (whole, last 32 tokens one by one, portions of changing size down to two tokens, mixed
with up to four live requests in the smallest pool, pages used again), in float32 and bfloat16, every returned
row against ``tests/plain_qwen2.py`` (numpy float64 on the same weights); float32 bit-equal between the cuttings.
"""
import numpy as np
import pytest
import torch

from conftest import random_tokens
from test_replay_gpu import every_way_of_cutting

pytestmark = pytest.mark.gpu


def _cfg(hidden, heads, kv_heads, intermediate, vocab, eps):
    return dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=vocab, hidden_size=hidden, intermediate_size=intermediate,
                num_hidden_layers=1, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=128, rms_norm_eps=eps,
                rope_theta=1000000.0, max_position_embeddings=4096, tie_word_embeddings=False)


SHAPES = {
    "7b": (_cfg(3584, 28, 4, 18944, 8192, 1e-6), 5, [40, 300, 700]),
    "14b": (_cfg(5120, 40, 8, 13824, 8200, 1e-5), 6, [33, 270, 520]),
    "32b": (_cfg(5120, 40, 8, 27648, 8192, 1e-6), 7, [17, 290]),
}
_folders = {}


@pytest.fixture(scope="module")
def wide_folders(tmp_path_factory):
    from mimirmind_b200.weights import write_random_model

    def get(name, dtype):
        if (name, dtype) not in _folders:
            d = tmp_path_factory.mktemp(f"wide_{name}_{dtype}")
            write_random_model(str(d), SHAPES[name][0], SHAPES[name][1], dtype)
            _folders[(name, dtype)] = str(d)
        return _folders[(name, dtype)]
    return get


@pytest.mark.parametrize("name,dtype", [("7b", "float32"), ("7b", "bfloat16"), ("14b", "float32"), ("14b", "bfloat16"), ("32b", "bfloat16")])
def test_wide_layers_every_way_of_cutting_against_the_plain_implementation(name, dtype, wide_folders):
    import plain_qwen2 as plain
    from mimirmind_b200.kernels import ops
    folder = wide_folders(name, dtype)
    pm = plain.PlainModel(folder)
    reqs = {f"{name}{i}": random_tokens(pm.V, n, 31 * i + n) for i, n in enumerate(SHAPES[name][2])}
    ref = {rid: pm.logits(t) for rid, t in reqs.items()}
    del pm
    every_way_of_cutting(folder, dtype, reqs, ref, seed=11)
    ops.check_tcgen05_errors(torch.device("cuda"))
    torch.cuda.empty_cache()


def test_wide_layer_graph_decode_equals_eager_decode(wide_folders):
    from mimirmind_b200 import Engine
    folder = wide_folders("7b", "bfloat16")
    prompts = [random_tokens(8192, n, n) for n in (700, 33, 1200)]
    eager = Engine.from_folder(folder, dtype="bfloat16", cache_tokens=8192, max_context=2048, token_budget=2048, max_active=4, use_graphs=False)
    a = eager.generate(prompts, max_new_tokens=24)
    del eager
    torch.cuda.empty_cache()
    graphs = Engine.from_folder(folder, dtype="bfloat16", cache_tokens=8192, max_context=2048, token_budget=2048, max_active=4, use_graphs=True)
    b = graphs.generate(prompts, max_new_tokens=24)
    assert graphs.graph_steps > 0
    # same kernels on the same inputs: the replayed graph gives the same tokens as stepping eagerly
    assert [r.tokens for r in a] == [r.tokens for r in b]


def test_the_pool_is_sized_from_the_device_when_nothing_is_configured(wide_folders):
    """With no cache size given the pool takes what the free memory allows, at most every active request at the full
    context: on this GPU, with one layer of the 7B width, that cap (32 requests of 4,096 tokens) is reached, so a full
    house never preempts."""
    from mimirmind_b200 import Engine
    eng = Engine.from_folder(wide_folders("7b", "bfloat16"), dtype="bfloat16", max_context=4096, token_budget=512, max_active=32)
    mgr = eng.runner.manager
    assert mgr.total_pages() * mgr.page_size == 32 * 4096
    free, _ = torch.cuda.mem_get_info()
    assert free > 0


def test_long_portions_beside_single_tokens(wide_folders):
    """Steps that hold prompt portions of 128 tokens and more beside single decoded tokens of other requests: the two
    attention kernels of such a step run side by side on two streams.  Every row against the plain implementation, and
    the same bits with the second stream switched off."""
    import plain_qwen2 as plain
    import replay_util as ru
    from mimirmind_b200.engine import native
    from mimirmind_b200.kernels import ops
    from test_replay_gpu import check
    folder = wide_folders("7b", "bfloat16")
    pm = plain.PlainModel(folder)
    reqs = {"a": random_tokens(pm.V, 230, 1), "b": random_tokens(pm.V, 150, 2), "c": random_tokens(pm.V, 420, 3), "d": random_tokens(pm.V, 200, 4)}
    ref = {rid: pm.logits(t) for rid, t in reqs.items()}
    del pm
    t = ru.Trace()
    all_of = lambda n: list(range(n))
    t.step([("a", reqs["a"][:200], all_of(200)), ("b", reqs["b"][:120], all_of(120))])
    fed = {"a": 200, "b": 120, "c": 0, "d": 0}

    def mixed_step(portions, end=()):
        entries = []
        for rid in ("a", "b"):
            if fed[rid] < len(reqs[rid]):
                entries.append((rid, reqs[rid][fed[rid]:fed[rid] + 1], [0]))
                fed[rid] += 1
        for rid, n in portions:
            entries.append((rid, reqs[rid][fed[rid]:fed[rid] + n], all_of(n)))
            fed[rid] += n
        t.step(entries, end=end)

    mixed_step([("c", 160)])                       # one portion of 160 beside two single tokens
    mixed_step([("c", 129), ("d", 70)])            # two portions, 199 tokens together
    mixed_step([("d", 130), ("c", 2)])
    mixed_step([("c", 129)], end=["c", "d"])
    while fed["a"] < len(reqs["a"]) or fed["b"] < len(reqs["b"]):
        mixed_step([])
    assert all(fed[r] == len(reqs[r]) for r in reqs)
    outs = []
    for side in (1, 0):
        old = native.option("use_side_stream", side)
        try:
            out, _ = ru.run_in_process(folder, "bfloat16", t, t.max_live_tokens())
        finally:
            native.option("use_side_stream", old)
        ops.check_tcgen05_errors(torch.device("cuda"))
        check(t, out, reqs, ref, "bfloat16", f"long portions beside single tokens (side stream {side})")
        outs.append(out)
    for i in outs[0]:
        assert np.array_equal(outs[0][i], outs[1][i]), f"step {i}"
    torch.cuda.empty_cache()
