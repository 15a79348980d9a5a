"""The plain implementation itself (no GPU): against the reference's own CPU code through the committed
golden vectors, and its parts against hand-computed cases (after the reference's formula-level unit
tests, tests/arch_tests.cpp:68-292 and tests/compute_tests.cpp:922-1042)."""
import os

import numpy as np
import pytest

import plain_qwen2 as plain
from golden.golden_configs import GOLDEN, GOLDEN_ATTENTION, attention_inputs

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_plain_matches_reference_cpu_code(name, tmp_path):
    from mimirmind_b200.weights import write_random_model
    g = GOLDEN[name]
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    write_random_model(str(tmp_path), g["config"], g["seed"], "float32")
    m = plain.PlainModel(str(tmp_path))
    logits, hidden = plain.forward(m, z["tokens"].tolist(), return_hidden=True)
    scale = np.abs(z["logits"]).max()
    assert np.abs(logits - z["logits"]).max() < 2e-6 * max(scale, 1.0)
    assert np.abs(hidden[-1] - z["hidden"]).max() < 2e-6 * max(np.abs(z["hidden"]).max(), 1.0)
    assert [plain.greedy(r) for r in logits.astype(np.float32)] == [int(np.argmax(r)) for r in z["logits"]]


@pytest.mark.parametrize("i", range(len(GOLDEN_ATTENTION)))
def test_plain_attention_window_matches_the_reference_function(i):
    """The sliding window and the position offset of the reference's own attention function
    (src/compute/Attention.cpp:46-50), which its block for this architecture never passes: a query at absolute
    position a sees keys [max(0, a + 1 - W), a].  Committed outputs of direct calls, four cases."""
    case = GOLDEN_ATTENTION[i]
    want = np.load(os.path.join(GOLDEN_DIR, "golden_attention.npz"))[f"case{i}"]
    q, k, v = attention_inputs(case)
    lo, hi = case["offset"], case["offset"] + case["Tq"]
    full = np.zeros((case["Tk"], case["H"], case["hd"]))       # the plain function takes whole sequences: rows before the queries are unused
    full[lo:hi] = q
    got = plain.attention(full, k.astype(np.float64), v.astype(np.float64), case["window"])[lo:hi]
    assert want.shape == got.shape and np.abs(got - want).max() < 5e-7


def test_rms_norm_formula():
    x = np.array([[3.0, 4.0]])
    y = plain.rms_norm(x, np.array([1.0, 2.0]), 0.5)
    assert np.allclose(y, x * [1.0, 2.0] / np.sqrt(12.5 + 0.5))


def test_rope_identities():
    x = np.random.RandomState(0).randn(3, 2, 8)
    assert np.allclose(plain.rope(x, np.zeros(3, dtype=int), 10000.0), x)         # position 0 is the identity
    y = plain.rope(x, np.array([5, 6, 7]), 10000.0)
    assert np.allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1))   # a rotation keeps the norm
    # pair (0, 4) of an 8-wide head turns by pos * theta^0 = pos
    a, b = x[0, 0, 0], x[0, 0, 4]
    assert np.allclose([y[0, 0, 0], y[0, 0, 4]], [a * np.cos(5) - b * np.sin(5), a * np.sin(5) + b * np.cos(5)])


def test_attention_causal_two_tokens_and_gqa():
    q = np.zeros((2, 2, 2)); k = np.zeros((2, 1, 2)); v = np.array([[[1.0, 0.0]], [[0.0, 1.0]]])
    o = plain.attention(q, k, v, 0)
    assert np.allclose(o[0], [[1, 0], [1, 0]])            # the first token sees only itself
    assert np.allclose(o[1], [[0.5, 0.5], [0.5, 0.5]])    # equal scores: the mean; both heads share the KV head


def test_attention_window():
    T = 6
    q = np.zeros((T, 1, 2)); k = np.zeros((T, 1, 2)); v = np.arange(T, dtype=float).reshape(T, 1, 1).repeat(2, -1)
    o = plain.attention(q, k, v, 3)
    assert np.allclose(o[:, 0, 0], [0, 0.5, 1, 2, 3, 4])  # mean of the last 3 positions


def test_kv_head_mapping_is_integer_division():
    rng = np.random.RandomState(1)
    q = rng.randn(4, 6, 4); k = rng.randn(4, 3, 4); v = rng.randn(4, 3, 4)
    o = plain.attention(q, k, v, 0)
    for h in range(6):
        solo = plain.attention(q[:, h:h + 1], k[:, h // 2:h // 2 + 1], v[:, h // 2:h // 2 + 1], 0)
        assert np.allclose(o[:, h], solo[:, 0])


def test_embedding_out_of_range_gives_zero_row():
    t = np.arange(6.0).reshape(3, 2)
    assert np.allclose(plain.embedding(t, [2, 5, -1]), [[4, 5], [0, 0], [0, 0]])


def test_greedy_lowest_index_on_ties():
    assert plain.greedy(np.array([1.0, 3.0, 3.0, 2.0])) == 1


def test_sampler_support_sets_and_limits():
    logits = np.array([0.0, 1.0, 2.0, 3.0, 4.0])
    us = [i / 50 for i in range(50)]
    assert {plain.sample(logits, 1.0, 2, 1.0, u) for u in us} == {3, 4}                 # top-k support
    assert {plain.sample(logits, 1.0, 0, 0.5, u) for u in us} == {4}                    # 4 alone holds 0.64 > 0.5
    assert {plain.sample(logits, 1.0, 0, 0.7, u) for u in us} == {3, 4}
    assert all(plain.sample(logits, 1e-4, 0, 1.0, u) == 4 for u in us)                  # very low temperature
    assert all(plain.sample(logits, 1.0, 1, 1.0, u) == 4 for u in us)                   # top_k 1 is greedy
    assert all(plain.sample(logits, 0.0, 0, 1.0, u) == 4 for u in us)
    counts = np.bincount([plain.sample(logits, 1.0, 0, 1.0, (i + 0.5) / 4000) for i in range(4000)], minlength=5)
    p = np.exp(logits - 4); p /= p.sum()
    assert np.abs(counts / 4000 - p).max() < 2e-3


def test_uniform_stream_is_deterministic():
    a = [plain.uniform_from(7, i) for i in range(1000)]
    assert a == [plain.uniform_from(7, i) for i in range(1000)] and len(set(a)) > 990
    assert 0.45 < np.mean(a) < 0.55 and min(a) >= 0.0 and max(a) < 1.0
