"""How many tokens the page pool holds when the configuration does not say: as many as the device has room for.

The reference sizes its cache from the runtime setting alone (``maxContextTokens``,
src/runtime/InferenceEngine.hpp:967); a paged pool shared by many requests is better sized from the memory that
is left once the weights are loaded.  Pure arithmetic, so that it can be tested without a device:

    usable  = free bytes x fraction - what a step needs beside the cache
    tokens  = usable / bytes that one token takes in every cache group
    capped at maxContextTokens x maxActiveRequests (more can never be in use), in whole pages
"""
from __future__ import annotations

from typing import Iterable, Sequence

from ..config.spec import ModelSpec


class CacheSizingError(RuntimeError):
    pass


def cache_bytes_per_token(groups: Iterable, element_bytes: int) -> int:
    """Bytes one cached token takes over all groups (every per-token array of every schedule entry of a group)."""
    sizes = {None: element_bytes, "float32": 4, "bfloat16": 2, "float16": 2, "int32": 4, "int8": 1}
    total = 0
    for g in groups:
        for _name, shape, dtype in g.token_arrays():
            n = 1
            for s in shape:
                n *= int(s)
            total += len(g.entries) * n * sizes[dtype]
    return total


def step_bytes_per_token(spec: ModelSpec, layer_tensor_shapes: Sequence[Sequence[Sequence[int]]], element_bytes: int) -> int:
    """Estimate of a step's working memory per token: the fp32 residual stream (and a copy for the norm's
    output) plus every output row of the widest layer's matrices, twice over, because the memory of two
    consecutive layers is live at a time.  ``layer_tensor_shapes``: per layer, the shapes of its tensors."""
    widest = 0
    for shapes in layer_tensor_shapes:
        widest = max(widest, sum(int(s[0]) for s in shapes if len(s) == 2))
    return 2 * 4 * spec.hidden_size + 2 * element_bytes * widest


def step_reserve_bytes(spec: ModelSpec, layer_tensor_shapes, element_bytes: int, token_budget: int, max_active: int) -> int:
    """What is kept free for a step of ``token_budget + max_active`` tokens: activations, logits of every active
    request (three copies: the step's, the sampler's, a captured graph's) and 128 MiB for library workspaces."""
    tokens = token_budget + max_active
    return tokens * step_bytes_per_token(spec, layer_tensor_shapes, element_bytes) + 3 * 4 * max_active * spec.vocab_size + (128 << 20)


def pool_tokens(free_bytes: int, fraction: float, reserve_bytes: int, bytes_per_token: int, page_size: int, max_context: int,
                max_active: int) -> int:
    """Tokens for the page pool, a multiple of ``page_size``.  Raises CacheSizingError when not even one request's
    first page fits."""
    if not (0.0 < fraction <= 1.0):
        raise CacheSizingError("the memory fraction must be in (0, 1]")
    if bytes_per_token <= 0:
        return page_size * max(1, max_active)            # no layer keeps keys and values: a token costs nothing
    usable = int(free_bytes * fraction) - reserve_bytes
    tokens = max(0, usable) // bytes_per_token
    cap = -(-max_context // page_size) * page_size * max_active
    tokens = min(tokens, cap) // page_size * page_size
    if tokens < page_size:
        raise CacheSizingError(
            f"no room for a cache: {free_bytes / 2 ** 30:.2f} GiB free x {fraction} leaves {max(0, usable) / 2 ** 30:.2f} GiB after "
            f"{reserve_bytes / 2 ** 30:.2f} GiB kept for a step, and a page of {page_size} tokens takes {page_size * bytes_per_token / 2 ** 20:.2f} MiB")
    return tokens
