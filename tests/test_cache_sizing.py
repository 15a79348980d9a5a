"""The arithmetic that sizes the page pool from free device memory (no GPU)."""
from types import SimpleNamespace

import pytest

from conftest import TINY
from mimirmind_b200.cache import sizing
from mimirmind_b200.cache.manager import GroupSpec
from mimirmind_b200.config.engine_config import EngineConfigError, parse_engine_config
from mimirmind_b200.registry import get_architecture
from mimirmind_b200.weights.store import layer_tensor_shapes

GIB = 1 << 30


def test_bytes_per_token_counts_every_entry_of_every_group():
    groups = [GroupSpec("full", (0, 2), 4, 128, 0), GroupSpec("win", (1,), 2, 64, 100)]
    assert sizing.cache_bytes_per_token(groups, 2) == 2 * 2 * 4 * 128 * 2 + 1 * 2 * 2 * 64 * 2
    assert sizing.cache_bytes_per_token([], 2) == 0


def test_pool_is_what_fits_capped_by_what_can_be_in_use():
    per_token = 57344            # a 7B-shaped model in bfloat16: 28 layers x 2 x 4 heads x 128 x 2 bytes
    # plenty of memory: the cap (every active request at the full context) decides
    assert sizing.pool_tokens(150 * GIB, 0.9, 2 * GIB, per_token, 16, 4096, 32) == 32 * 4096
    # little memory: what fits decides, in whole pages
    got = sizing.pool_tokens(4 * GIB, 0.5, 1 * GIB, per_token, 16, 4096, 32)
    assert got == (1 * GIB // per_token) // 16 * 16 and got % 16 == 0
    # a context that is no multiple of the page is rounded up per request
    assert sizing.pool_tokens(150 * GIB, 0.9, 0, per_token, 16, 100, 3) == 112 * 3
    with pytest.raises(sizing.CacheSizingError, match="no room"):
        sizing.pool_tokens(1 * GIB, 0.9, 2 * GIB, per_token, 16, 4096, 32)
    with pytest.raises(sizing.CacheSizingError, match="fraction"):
        sizing.pool_tokens(1 * GIB, 0.0, 0, per_token, 16, 4096, 32)
    assert sizing.pool_tokens(1 * GIB, 0.9, 0, 0, 16, 4096, 4) == 64        # nothing cached per token


def test_step_reserve_grows_with_the_budget_and_the_widest_layer():
    arch = get_architecture("Qwen2ForCausalLM")
    spec = arch.build_spec(arch.parse_config(TINY["B"], "test"))
    shapes = layer_tensor_shapes(spec)
    assert len(shapes) == 3 and all(any(len(s) == 2 for s in layer) for layer in shapes)
    per_token = sizing.step_bytes_per_token(spec, shapes, 2)
    widest = (6 + 2) * 32 + 192 + 2 * 352 + 192          # q,k,v rows + o rows + gate,up rows + down rows
    assert per_token == 2 * 4 * 192 + 2 * 2 * widest
    small = sizing.step_reserve_bytes(spec, shapes, 2, 64, 4)
    large = sizing.step_reserve_bytes(spec, shapes, 2, 512, 4)
    assert large - small == (512 - 64) * per_token


def test_engine_config_takes_the_fraction():
    cfg = parse_engine_config({"models": [{"id": "m", "path": "/x"}], "runtime": {"cacheMemoryFraction": 0.5}})
    assert cfg.runtime.cacheMemoryFraction == 0.5 and cfg.runtime.cacheTokens == 0
    with pytest.raises(EngineConfigError, match="cacheMemoryFraction"):
        parse_engine_config({"models": [{"id": "m", "path": "/x"}], "runtime": {"cacheMemoryFraction": 1.5}})
    with pytest.raises(EngineConfigError, match="number"):
        parse_engine_config({"models": [{"id": "m", "path": "/x"}], "runtime": {"cacheMemoryFraction": "half"}})
