"""The kernels that only large shapes reach (weight-streaming products with 8 row tiles per CTA, the tcgen05
product with the SwiGLU epilogue, tcgen05 prefill attention, split-key decode attention over thousands of keys,
decode as a replayed graph) inside the whole engine: one layer with the widths of the benchmark model, bfloat16
against the engine's own 32-bit path on the same weights (that path is checked against the plain implementation
on the tiny models)."""
import numpy as np
import pytest
import torch

from conftest import random_tokens

pytestmark = pytest.mark.gpu

WIDE = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=2048, hidden_size=3584, intermediate_size=18944,
            num_hidden_layers=1, num_attention_heads=28, num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6,
            rope_theta=1000000.0, max_position_embeddings=4096, tie_word_embeddings=False)


@pytest.fixture(scope="module")
def wide_folder(tmp_path_factory):
    from mimirmind_b200.weights import write_random_model
    d = tmp_path_factory.mktemp("wide")
    write_random_model(str(d), WIDE, 5, "bfloat16")
    return str(d)


def run_steps(folder, dtype, cuts, toks):
    from mimirmind_b200.engine.loader import load_model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    from mimirmind_b200.kernels import ops
    model, _ = load_model(folder, dtype)
    runner = ModelRunner(model, 16, 4096 // 16, 4)
    runner.add_request("a")
    outs, p = [], 0
    for c in cuts:
        want = [c - 1]
        outs.append(runner.step([StepEntry("a", toks[p:p + c], want)]).float().cpu().numpy())
        p += c
    ops.check_tcgen05_errors(model.rt.device)
    del runner, model
    torch.cuda.empty_cache()
    return np.concatenate(outs)


def test_wide_layer_bf16_kernels_agree_with_the_32_bit_path(wide_folder):
    toks = random_tokens(2048, 1500 + 40, 9)
    # a 1,500-token portion (tcgen05 product and attention), a 24-token portion, then single tokens (streaming products)
    cuts = [1500, 24] + [1] * 16
    ref = run_steps(wide_folder, "float32", cuts, toks)
    got = run_steps(wide_folder, "bfloat16", cuts, toks)
    scale = np.abs(ref).max()
    err = np.abs(got - ref)
    assert err.max() <= 4e-2 * scale, f"max error {err.max():.4f} of scale {scale:.3f} at row {err.max(axis=1).argmax()}"
    assert err.mean() <= 6e-3 * scale


def test_wide_layer_graph_decode_equals_eager_decode(wide_folder):
    from mimirmind_b200 import Engine
    prompts = [random_tokens(2048, n, n) for n in (700, 33, 1200)]
    eager = Engine.from_folder(wide_folder, dtype="bfloat16", cache_tokens=8192, max_context=2048, token_budget=2048, max_active=4, use_graphs=False)
    a = eager.generate(prompts, max_new_tokens=24)
    del eager
    torch.cuda.empty_cache()
    graphs = Engine.from_folder(wide_folder, dtype="bfloat16", cache_tokens=8192, max_context=2048, token_budget=2048, max_active=4, use_graphs=True)
    b = graphs.generate(prompts, max_new_tokens=24)
    assert graphs.graph_steps > 0
    # same kernels on the same inputs: the replayed graph gives the same tokens as stepping eagerly
    assert [r.tokens for r in a] == [r.tokens for r in b]
