"""The tiny configurations whose reference outputs are committed beside this file."""

GOLDEN = {
    "golden_a": {
        "seed": 0, "tokens": 40,
        "config": dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=256, hidden_size=64,
                       intermediate_size=176, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=128, tie_word_embeddings=True,
                       torch_dtype="float32"),
    },
    "golden_b": {
        "seed": 1, "tokens": 24,
        "config": dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=384, hidden_size=192,
                       intermediate_size=352, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1,
                       head_dim=32, rms_norm_eps=1e-5, rope_theta=1000000.0, max_position_embeddings=256,
                       tie_word_embeddings=False, torch_dtype="float32"),
    },
    # head_dim * heads != hidden (explicit key length, src/model/LlmConfig.hpp:145-150)
    "golden_c": {
        "seed": 2, "tokens": 19,
        "config": dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=200, hidden_size=80,
                       intermediate_size=112, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=3,
                       head_dim=48, rms_norm_eps=1e-5, rope_theta=50000.0, max_position_embeddings=64,
                       tie_word_embeddings=False, torch_dtype="float32"),
    },
}

# Direct calls of the reference's attention with a sliding window and a position offset (queries are the last Tq
# positions of a sequence whose Tk keys may reach beyond them): dims, window, offset and the seed of q, k, v.
GOLDEN_ATTENTION = [
    dict(seed=11, Tq=7, Tk=40, H=6, G=2, hd=16, offset=33, window=9),      # a window inside the sequence, queries at its end
    dict(seed=12, Tq=40, Tk=40, H=4, G=1, hd=32, offset=0, window=5),      # a whole sequence: the window opens at position 5
    dict(seed=13, Tq=3, Tk=50, H=8, G=4, hd=8, offset=20, window=64),      # a window wider than the sequence, keys beyond the queries
    dict(seed=14, Tq=5, Tk=30, H=3, G=3, hd=24, offset=12, window=1),      # every query sees only itself
]


def attention_inputs(case):
    """q [Tq, H, hd], k and v [Tk, G, hd] of a case, float32, from its seed."""
    import numpy as np
    rng = np.random.RandomState(case["seed"])
    q = rng.randn(case["Tq"], case["H"], case["hd"]).astype(np.float32)
    k = rng.randn(case["Tk"], case["G"], case["hd"]).astype(np.float32)
    v = rng.randn(case["Tk"], case["G"], case["hd"]).astype(np.float32)
    return q, k, v
