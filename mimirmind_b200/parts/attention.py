"""Causal self-attention with grouped KV heads over a paged cache.

Per layer (src/runtime/arch/Qwen2Backend.cpp:203-430): ``q,k,v = n·Wᵀ + b`` (bias on
q/k/v only, none on the output projection), position encoding on q and k, k and v
appended to the cache *before* attention, ``s = (q·k)·scale`` with ``scale = 1/sqrt(hd)``
(:415-416), softmax over the keys a query may see, ``o = P·v``, then the output
projection.  Query head h reads KV head ``(h·G)/H`` (src/compute/Attention.cpp:43); a
query at absolute position a sees keys ``[max(0, a+1−W), a]`` (:46-50, W = 0: all).

Head counts, head size, window, scale, biases and the position encoding are parameters of
the part; the three projections are concatenated at load so one product feeds the fused
bias + rotary + cache-write kernel.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import MIXERS, POSITION_ENCODINGS
from .base import FactoredRows, KVCacheSpec, LayerCache, Mixer, NativeDesc, ResidualSink, Runtime, StepContext, WeightView
from .linear import linear


@MIXERS.register("gqa_attention")
class GQAAttention(Mixer):
    """spec params: hidden, num_heads, num_kv_heads, head_dim, window, scale (None: 1/sqrt(head_dim)),
    qkv_bias, position (PartSpec), q, k, v, o (projection name stems under the prefix)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        d, hd = spec["hidden"], spec["head_dim"]
        qs, kvs = spec["num_heads"] * hd, spec["num_kv_heads"] * hd
        out = [
            TensorSpec(prefix + spec["q"] + ".weight", (qs, d)),
            TensorSpec(prefix + spec["k"] + ".weight", (kvs, d)),
            TensorSpec(prefix + spec["v"] + ".weight", (kvs, d)),
            TensorSpec(prefix + spec["o"] + ".weight", (d, qs)),
        ]
        if spec.get("qkv_bias", False):
            out += [
                TensorSpec(prefix + spec["q"] + ".bias", (qs,), role="bias"),
                TensorSpec(prefix + spec["k"] + ".bias", (kvs,), role="bias"),
                TensorSpec(prefix + spec["v"] + ".bias", (kvs,), role="bias"),
            ]
        return out

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.hidden = int(spec["hidden"])
        self.num_heads = int(spec["num_heads"])
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.window = int(spec.get("window", 0) or 0)
        scale = spec.get("scale")
        # computed in fp32 like the reference (src/runtime/arch/Qwen2Backend.cpp:415-416)
        self.scale = float(scale) if scale is not None else float(
            torch.tensor(1.0, dtype=torch.float32) / torch.sqrt(torch.tensor(float(self.head_dim), dtype=torch.float32)))
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        pos_spec: PartSpec = spec["position"]
        self.position = POSITION_ENCODINGS.get(pos_spec.kind)(pos_spec, weights, rt)

        ws = [weights.take(spec[n] + ".weight") for n in ("q", "k", "v")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        self.w_qkv = torch.cat(ws, dim=0).contiguous()
        del ws
        self.b_qkv: Optional[torch.Tensor] = None
        if spec.get("qkv_bias", False):
            bs = [weights.take(spec[n] + ".bias") for n in ("q", "k", "v")]
            if len({b.dtype for b in bs}) > 1:
                bs = [b.float() for b in bs]
            self.b_qkv = torch.cat(bs, dim=0).contiguous()
        self.w_o = weights.take(spec["o"] + ".weight").contiguous()
        # With a rotation of the whole head that the kernels can apply, the q and k rows of the projection are
        # stored with each head's halves interleaved in blocks of 8: the weight-streaming product of a decode
        # step then holds rotation partners in one thread and encodes and caches in its epilogue.
        fused = self.position.fused_rotary()
        self.interleaved = bool(
            fused is not None and fused[0] == self.head_dim and self.head_dim % 16 == 0 and rt.dtype == torch.bfloat16
            and self.w_qkv.dtype == torch.bfloat16 and self.w_o.dtype == torch.bfloat16 and rt.matmul != "simt")
        if rt.dtype == torch.bfloat16:
            self._say_what_runs_slowly(fused)
        if self.interleaved:
            rot_heads = self.num_heads + self.num_kv_heads
            self.w_qkv = ops.interleave_halves(self.w_qkv, rot_heads, self.head_dim)
            if self.b_qkv is not None:
                self.b_qkv = ops.interleave_halves(self.b_qkv, rot_heads, self.head_dim)

    _told = set()

    def _say_what_runs_slowly(self, fused) -> None:
        """One warning per head geometry that the tensor-core attention kernels or the fused projection are not built for:
        the model still runs, correctly, on the generic kernels, far from the speed of the built-for shapes."""
        import warnings
        from ..kernels import attention_bf16
        H, G, hd = self.num_heads, self.num_kv_heads, self.head_dim
        reasons = []
        if not attention_bf16.supports(hd, H, G):
            reasons.append(f"attention with head size {hd} and {H // G} query heads per KV head runs the generic kernel "
                           "(the tensor-core kernels take head sizes 64 and 128 and up to 16 query heads per KV head)")
        if fused is None or fused[0] != hd or hd % 16:
            reasons.append("the position encoding is not a rotation of the whole head in steps of 16, so small steps run the projection, "
                           "the encoding and the cache write as separate kernels")
        key = (H, G, hd, tuple(reasons))
        if reasons and key not in GQAAttention._told:
            GQAAttention._told.add(key)
            warnings.warn("mimirmind_b200: " + "; ".join(reasons), RuntimeWarning, stacklevel=3)

    def _encode_unfused(self, qkv: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """A position encoding the fused kernel cannot apply: add the bias with the same kernel into contiguous
        buffers (a pool of one-token pages addressed by token index, no rotation), let the encoding's own
        ``apply`` work on q [n, H, hd] and k [n, G, hd] in place, and hand back one [n, (H+2G)*hd] buffer."""
        n = qkv.shape[0]
        H, G, hd = self.num_heads, self.num_kv_heads, self.head_dim
        q = torch.empty((n, H * hd), dtype=qkv.dtype, device=qkv.device)
        k = torch.empty((n, G, 1, hd), dtype=qkv.dtype, device=qkv.device)
        v = torch.empty_like(k)
        index = torch.arange(n, dtype=torch.int32, device=qkv.device)
        ops.qkv_rope_kvwrite(qkv, self.b_qkv, q, k, v, index, torch.zeros_like(index), index.view(1, n).contiguous(), 1, H, G, hd, 0, 1.0)
        self.position.apply(q.view(n, H, hd), k.view(n, G, hd), ctx.positions)
        return torch.cat([q, k.view(n, G * hd), v.view(n, G * hd)], dim=1)

    def _dump_qkv(self, q: torch.Tensor, cache: LayerCache, ctx: StepContext) -> None:
        """The reference's Qcur / Kcur / Vcur stages (src/runtime/arch/Qwen2Backend.cpp:390-392): q after bias and
        rotation, and this step's keys and values as they stand in the cache (read back from their pages)."""
        ctx.dump("Qcur", q)
        if not cache.writes:
            return
        slots = ops.slot_mapping(ctx.positions, ctx.token_req, cache.block_table, cache.page_size).long()
        ok = slots >= 0
        page, place = (slots.clamp(min=0) // cache.page_size), (slots.clamp(min=0) % cache.page_size)
        for stage, pool in (("Kcur", cache.k_pages), ("Vcur", cache.v_pages)):
            rows = pool[page, :, place, :].reshape(q.shape[0], -1).clone()
            rows[~ok] = 0
            ctx.dump(stage, rows)

    def kv_cache_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def native(self):
        position = self.position.native()
        if type(self) is not GQAAttention or position is None or self.position.fused_rotary() is None:
            return None
        tensors = {"w_qkv": self.w_qkv, "w_o": self.w_o}
        if self.b_qkv is not None:
            tensors["b_qkv"] = self.b_qkv
        return NativeDesc("gqa_attention", {
            "hidden": self.hidden, "num_heads": self.num_heads, "num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim,
            "window": self.window, "scale": self.scale, "interleaved": int(self.interleaved)}, tensors, {"position": position})

    def fuses(self, n_tokens: int) -> bool:
        width = (self.num_heads + 2 * self.num_kv_heads) * self.head_dim
        return (self.interleaved and ops.small_batch_supported(n_tokens, width, self.hidden)
                and ops.small_batch_supported(n_tokens, self.hidden, self.num_heads * self.head_dim))

    def forward(self, x, ctx: StepContext, cache: LayerCache, sink: Optional[ResidualSink] = None):
        n = x.shape[0]
        H, G, hd = self.num_heads, self.num_kv_heads, self.head_dim
        k_pages, v_pages = (cache.k_pages, cache.v_pages) if cache.writes else (None, None)
        fused = self.position.fused_rotary()
        fuses = self.fuses(n) and not ctx.plain_only
        q = torch.empty((n, H * hd), dtype=self.rt.dtype, device=x.xw.device if isinstance(x, FactoredRows) else x.device)
        # rotation factors and cache places are the same in every layer that shares them: made once per step
        tables = fused is not None and fused[0] == hd and hd % 16 == 0 and self.rt.dtype == torch.bfloat16
        table = slots = None
        if tables:
            key = ("rope_table", hd, fused[1])
            if key not in ctx.derived:
                ctx.derived[key] = ops.rope_table(ctx.positions, hd, fused[1])
            table = ctx.derived[key]
            if k_pages is not None:
                skey = ("slots", cache.block_table.data_ptr(), cache.page_size)
                if skey not in ctx.derived:
                    ctx.derived[skey] = ops.slot_mapping(ctx.positions, ctx.token_req, cache.block_table, cache.page_size)
                slots = ctx.derived[skey]
        if fuses:
            # a few tokens: projection, 1/rms of a factored input, bias, rotation and cache write in one launch
            xin, scale = (x.xw, x.scale) if isinstance(x, FactoredRows) else (x, None)
            ops.gemv_bf16_qkv_rope(xin, self.w_qkv, self.b_qkv, q, k_pages, v_pages, table, slots,
                                   cache.page_size, H, G, hd, scale=scale)
        else:
            qkv = linear(x, self.w_qkv, None, self.rt)
            if tables and qkv.dtype == torch.bfloat16:
                ops.qkv_rope_tables(qkv, self.b_qkv, q, k_pages, v_pages, table, slots, cache.page_size, H, G, hd,
                                    interleave=self.interleaved)
            elif fused is not None:
                rotary_dim, theta = fused
                ops.qkv_rope_kvwrite(qkv, self.b_qkv, q, k_pages, v_pages, ctx.positions, ctx.token_req, cache.block_table,
                                     cache.page_size, H, G, hd, rotary_dim, theta, interleave=self.interleaved)
            else:
                qkv = self._encode_unfused(qkv, ctx)
                ops.qkv_rope_kvwrite(qkv, None, q, k_pages, v_pages, ctx.positions, ctx.token_req, cache.block_table,
                                     cache.page_size, H, G, hd, 0, 1.0)
        if ctx.dump is not None:
            self._dump_qkv(q, cache, ctx)
        out = torch.empty_like(q)
        from ..kernels import attention as attn_kernels
        attn_kernels.paged_attention(q, cache, out, ctx, H, G, hd, self.window, self.scale)
        if sink is None:
            return linear(out, self.w_o, None, self.rt)
        made = ops.gemv_bf16_residual(out, self.w_o, sink.residual, sink.norm_weight, sink.eps)
        return FactoredRows(*made) if made is not None else None
