"""Shared fixtures: tiny configurations, model folders in temporary directories, the plain oracle."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def _base(**kw):
    d = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_act="silu")
    d.update(kw)
    return d


# Two tiny configurations that differ in every size and option, plus variants for the head
# sizes the tensor-core attention kernels are built for.
TINY = {
    # no window, tied head, group of 2, head 16
    "A": _base(vocab_size=256, hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=1024,
               tie_word_embeddings=True, use_sliding_window=False),
    # window on layers 1 and 2, untied head, one KV head for 6 query heads, head 32, explicit head_dim
    "B": _base(vocab_size=384, hidden_size=192, intermediate_size=352, num_hidden_layers=3, num_attention_heads=6,
               num_key_value_heads=1, head_dim=32, rms_norm_eps=1e-5, rope_theta=1000000.0,
               max_position_embeddings=2048, tie_word_embeddings=False, use_sliding_window=True, sliding_window=72,
               max_window_layers=1),
    # heads * head_dim != hidden, head 48 (no power of two), three KV heads, odd vocabulary
    "C": _base(vocab_size=203, hidden_size=80, intermediate_size=112, num_hidden_layers=2, num_attention_heads=6,
               num_key_value_heads=3, head_dim=48, rms_norm_eps=1e-5, rope_theta=50000.0,
               max_position_embeddings=1024, tie_word_embeddings=False),
    # head 128 and 7 query heads per KV head (the group size of the benchmark model)
    "D": _base(vocab_size=331, hidden_size=160, intermediate_size=208, num_hidden_layers=2, num_attention_heads=7,
               num_key_value_heads=1, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
               max_position_embeddings=2048, tie_word_embeddings=False),
    # head 64, window on every layer
    "E": _base(vocab_size=300, hidden_size=128, intermediate_size=144, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=10000.0,
               max_position_embeddings=2048, tie_word_embeddings=True, use_sliding_window=True, sliding_window=100,
               max_window_layers=0),
    # the second tiny configuration of the baseline's list as it is written there: B without a window, context 256
    "F": _base(vocab_size=384, hidden_size=192, intermediate_size=352, num_hidden_layers=3, num_attention_heads=6,
               num_key_value_heads=1, head_dim=32, rms_norm_eps=1e-5, rope_theta=1000000.0,
               max_position_embeddings=256, tie_word_embeddings=False, use_sliding_window=False),
    # sizes that fit no kernel's tile: a width of 50 (rows of bfloat16 that are not 16-byte aligned), a feed-forward width of 33,
    # a vocabulary of 77, as many KV heads as query heads
    "G": _base(vocab_size=77, hidden_size=50, intermediate_size=33, num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5,
               head_dim=32, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=512, tie_word_embeddings=False),
    # 17 query heads on one KV head of size 64 (more than the tensor-core attention kernels group), one layer
    "H": _base(vocab_size=200, hidden_size=128, intermediate_size=256, num_hidden_layers=1, num_attention_heads=17, num_key_value_heads=1,
               head_dim=64, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512, tie_word_embeddings=False),
    # a head size that is no multiple of 16 (18: the fused rotary kernels refuse it, the generic ones take it)
    "I": _base(vocab_size=64, hidden_size=72, intermediate_size=80, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
               head_dim=18, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512, tie_word_embeddings=False),
}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4, "F": 1, "G": 6, "H": 7, "I": 8}


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name, dtype → folder with config.json and model.safetensors (made once per session)."""
    from mimirmind_b200.weights import write_random_model
    cache = {}

    def get(name: str, dtype: str = "float32") -> str:
        key = (name, dtype)
        if key not in cache:
            d = tmp_path_factory.mktemp(f"model_{name}_{dtype}")
            write_random_model(str(d), TINY[name], SEEDS[name], dtype)
            cache[key] = str(d)
        return cache[key]

    return get


@pytest.fixture(scope="session")
def plain_models(model_folders):
    import plain_qwen2 as plain
    cache = {}

    def get(name: str, dtype: str = "float32"):
        key = (name, dtype)
        if key not in cache:
            cache[key] = plain.PlainModel(model_folders(name, dtype))
        return cache[key]

    return get


def random_tokens(vocab: int, n: int, seed: int):
    return np.random.RandomState(seed).randint(0, vocab, size=n).tolist()


def has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False
