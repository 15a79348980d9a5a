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
