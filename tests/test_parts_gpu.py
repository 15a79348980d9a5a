"""Each part alone against the plain function of the same part, and a toy mixer with state of its own
that is registered, built and stepped without a change to the package's files."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import replay_util as ru
from conftest import TINY, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rt(dtype=torch.float32):
    from mimirmind_b200.engine.loader import make_runtime
    return make_runtime(dtype)


def t(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a)).to(DEV).to(dtype).contiguous()


def test_norm_part():
    from mimirmind_b200.config.spec import PartSpec
    from mimirmind_b200.parts.base import WeightView
    from mimirmind_b200.parts.norm import RMSNorm
    rng = np.random.RandomState(0)
    w = rng.randn(100)
    spec = PartSpec("rmsnorm", {"width": 100, "eps": 1e-3, "weight": "n.weight"})
    assert [s.name for s in RMSNorm.tensor_specs(spec, "p.")] == ["p.n.weight"]
    part = RMSNorm(spec, WeightView({"p.n.weight": t(w)}, "p."), rt())
    x, d = rng.randn(4, 100), rng.randn(4, 100)
    res = t(x)
    y = part.forward(res, t(d))
    assert np.abs(y.cpu().numpy() - plain.rms_norm(x + d, w, 1e-3)).max() < 1e-5
    assert np.abs(res.cpu().numpy() - (x + d)).max() < 1e-6


def test_feed_forward_part():
    from mimirmind_b200.config.spec import PartSpec
    from mimirmind_b200.parts.base import WeightView
    from mimirmind_b200.parts.mlp import SwiGLU
    rng = np.random.RandomState(1)
    d, F = 72, 200
    Wg, Wu, Wd = rng.randn(F, d) * 0.1, rng.randn(F, d) * 0.1, rng.randn(d, F) * 0.1
    spec = PartSpec("swiglu", {"hidden": d, "intermediate": F, "gate": "g", "up": "u", "down": "d"})
    part = SwiGLU(spec, WeightView({"g": t(Wg), "u": t(Wu), "d": t(Wd)}), rt())
    x = rng.randn(9, d)
    y = part.forward(t(x), None)
    ref = plain.swiglu(x, Wg, Wu, Wd)
    assert np.abs(y.cpu().numpy() - ref).max() < 1e-5 * max(1, np.abs(ref).max())


def test_embedding_and_head_parts():
    from mimirmind_b200.config.spec import PartSpec
    from mimirmind_b200.parts.base import WeightView
    from mimirmind_b200.parts.embedding import LMHead, TokenEmbedding
    rng = np.random.RandomState(2)
    E = rng.randn(50, 24)
    weights = {"emb": t(E)}
    emb = TokenEmbedding(PartSpec("token_embedding", {"vocab": 50, "width": 24, "scale": 2.0, "weight": "emb"}), WeightView(weights), rt())
    ids = torch.tensor([3, 49, 0], dtype=torch.int32, device=DEV)
    assert np.allclose(emb.forward(ids).cpu().numpy(), 2.0 * E[[3, 49, 0]], atol=1e-6)
    tied = LMHead(PartSpec("lm_head", {"vocab": 50, "width": 24, "weight": "head", "tied_to": "emb"}), WeightView(weights), rt())
    x = rng.randn(2, 24)
    assert np.abs(tied.forward(t(x)).cpu().numpy() - x @ E.T).max() < 1e-4
    with pytest.raises(KeyError, match="head"):
        LMHead(PartSpec("lm_head", {"vocab": 50, "width": 24, "weight": "head", "tied_to": None}), WeightView(weights), rt())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_alone(dtype):
    """The mixer with its own cache view: two portions of one sequence against plain attention."""
    from mimirmind_b200.config.spec import PartSpec
    from mimirmind_b200.parts.attention import GQAAttention
    from mimirmind_b200.parts.base import LayerCache, StepContext, WeightView
    rng = np.random.RandomState(3)
    d, H, G, hd, ps, theta, W = 96, 6, 2, 64, 16, 5000.0, 40
    names = {"q": "q", "k": "k", "v": "v", "o": "o"}
    spec = PartSpec("gqa_attention", dict(hidden=d, num_heads=H, num_kv_heads=G, head_dim=hd, window=W, scale=None,
                                          qkv_bias=True, position=PartSpec("rotary_half", {"theta": theta, "rotary_dim": hd}), **names))
    w = {"q.weight": rng.randn(H * hd, d) * 0.1, "k.weight": rng.randn(G * hd, d) * 0.1, "v.weight": rng.randn(G * hd, d) * 0.1,
         "o.weight": rng.randn(d, H * hd) * 0.1, "q.bias": rng.randn(H * hd) * 0.1, "k.bias": rng.randn(G * hd) * 0.1,
         "v.bias": rng.randn(G * hd) * 0.1}
    if dtype == torch.bfloat16:
        w = {k: torch.as_tensor(v, dtype=torch.float32).to(torch.bfloat16).double().numpy() for k, v in w.items()}
    part = GQAAttention(spec, WeightView({k: t(v, dtype) for k, v in w.items()}), rt(dtype))
    assert part.kv_cache_spec().window == W and part.state_spec() is None
    T = 150
    x = rng.randn(T, d)
    if dtype == torch.bfloat16:
        x = torch.as_tensor(x, dtype=torch.float32).to(torch.bfloat16).double().numpy()
    pos = np.arange(T)
    q = plain.rope(plain.linear(x, w["q.weight"], w["q.bias"]).reshape(T, H, hd), pos, theta)
    k = plain.rope(plain.linear(x, w["k.weight"], w["k.bias"]).reshape(T, G, hd), pos, theta)
    v = plain.linear(x, w["v.weight"], w["v.bias"]).reshape(T, G, hd)
    ref = plain.linear(plain.attention(q, k, v, W).reshape(T, H * hd), w["o.weight"])
    pages = 12
    kp = torch.zeros((pages, G, ps, hd), dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    table = torch.tensor([[7, 2, 9, 0, 11, 4, 1, 8, 3, 10]], dtype=torch.int32, device=DEV)
    outs = []
    for lo, hi in ((0, 100), (100, 103), (103, 150)):
        n = hi - lo
        ctx = StepContext(n_tokens=n, n_requests=1, token_ids=None, positions=t(np.arange(lo, hi), torch.int32),
                          token_req=torch.zeros(n, dtype=torch.int32, device=DEV), q_start=[0], q_len=[n], kv_len=[hi],
                          req_meta=None, state_slots=None, block_tables={}, logit_rows=None, n_logit_rows=0, page_size=ps,
                          runtime=part.rt, max_kv_len=hi, max_q_len=n)
        cache = LayerCache(k_pages=kp, v_pages=vp, block_table=table, page_size=ps)
        outs.append(part.forward(t(x[lo:hi], dtype), ctx, cache).float().cpu().numpy())
    got = np.concatenate(outs)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert np.abs(got - ref).max() <= tol * np.abs(ref).max()


# ---- a toy mixer with state of its own ---------------------------------------------------------------

def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    """A running-mean mixer: out_t = W · mean(x_0..x_t).  Its per-request state (sum, count) lives in the
    cache manager's state slots.  Only registry calls are used; no file of the package changes."""
    from mimirmind_b200 import registry
    from mimirmind_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
    from mimirmind_b200.engine.loader import make_runtime
    from mimirmind_b200.engine.model import Model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    from mimirmind_b200.parts.base import Mixer, StateSpec
    from mimirmind_b200.weights.store import expected_tensors, random_tensors
    registry._ensure_builtin()

    @registry.MIXERS.register("toy_running_mean", replace=True)
    class RunningMean(Mixer):
        @classmethod
        def tensor_specs(cls, spec, prefix):
            return [TensorSpec(prefix + "mix.weight", (spec["hidden"], spec["hidden"]))]

        def __init__(self, spec, weights, rt):
            super().__init__(spec, weights, rt)
            self.d = spec["hidden"]
            self.w = weights.get("mix.weight")

        def state_spec(self):
            return StateSpec((self.d + 1,), torch.float32)          # running sum and count

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            for r in range(ctx.n_requests):                         # a request's tokens in order
                s, n = ctx.q_start[r], ctx.q_len[r]
                slot = int(ctx.state_slots[r])
                st = cache.state[slot]
                xs = x[s:s + n].float()
                csum = st[:self.d] + torch.cumsum(xs, dim=0)
                cnt = st[self.d] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                out[s:s + n] = ((csum / cnt[:, None]) @ self.w.float().t()).to(x.dtype)
                st[:self.d] = csum[-1]
                st[self.d] = cnt[-1]
            return out

    def toy_spec(cfg):
        d = cfg["hidden_size"]
        norm = lambda name: PartSpec("rmsnorm", {"width": d, "eps": 1e-5, "weight": name})
        attn = PartSpec("gqa_attention", dict(hidden=d, num_heads=2, num_kv_heads=1, head_dim=16, window=0, scale=None, qkv_bias=False,
                                              position=PartSpec("rotary_half", {"theta": 100.0, "rotary_dim": 8}),
                                              q="q", k="k", v="v", o="o"))
        ffn = PartSpec("swiglu", {"hidden": d, "intermediate": 40, "gate": "g.weight", "up": "u.weight", "down": "d.weight"})
        layers = (
            LayerSpec("l0.", PartSpec("pre_norm"), PartSpec("toy_running_mean", {"hidden": d}), ffn, norm("n1"), norm("n2")),
            LayerSpec("l1.", PartSpec("pre_norm"), attn, ffn, norm("n1"), norm("n2")),
        )
        # layer 0 runs twice (second time with state of its own), layer 1 once
        return ModelSpec("ToyForTest", d, cfg["vocab_size"], 512, PartSpec("token_embedding", {"vocab": cfg["vocab_size"], "width": d, "scale": 1.0, "weight": "emb"}),
                         layers, (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)), norm("nf"),
                         PartSpec("lm_head", {"vocab": cfg["vocab_size"], "width": d, "weight": "head", "tied_to": "emb"}))

    registry.register_architecture("ToyForTest", lambda obj, where="": obj, toy_spec, replace=True)
    try:
        entry = registry.get_architecture("ToyForTest")
        spec = entry.build_spec(entry.parse_config({"hidden_size": 32, "vocab_size": 90}))
        assert "l0.mix.weight" in expected_tensors(spec)
        rt_ = make_runtime("float32")
        model = Model(spec, random_tensors(spec, 5, torch.float32, rt_.device), rt_)
        assert sorted(model.state_specs()) == [0, 2] and len(model.cache_groups()) == 1
        assert model.cache_groups()[0].entries == (1,)

        def run(cuts, rid, runner):
            runner.add_request(rid)
            outs, p = [], 0
            for c in cuts:
                outs.append(runner.step([StepEntry(rid, toks[p:p + c], list(range(c)))]).cpu().numpy())
                p += c
            return np.concatenate(outs)

        toks = random_tokens(90, 60, 1)
        runner = ModelRunner(model, 16, 16, 4)
        whole = run([60], "a", runner)
        parts = run([7, 1, 1, 30, 2, 19], "b", runner)             # state carries over between portions
        assert np.abs(whole - parts).max() < 1e-5
        runner.release("a")
        again = run([60], "c", runner)                              # takes a's slot: it must start from zero
        assert runner.manager.slot("c") == 0
        assert np.abs(whole - again).max() < 1e-6
        # two requests in one batch keep separate state
        runner.add_request("d"); runner.add_request("e")
        other = random_tokens(90, 60, 2)
        both = runner.step([StepEntry("d", toks, [59]), StepEntry("e", other, [59])]).cpu().numpy()
        assert np.abs(both[0] - whole[59]).max() < 1e-5
        assert np.abs(both[1] - whole[59]).max() > 1e-3
    finally:
        registry.MIXERS.unregister("toy_running_mean")
        registry.ARCHITECTURES.unregister("ToyForTest")


# ---- a block with more than four parts, and a mixer that caches something else than keys and values ---------------

def test_toy_block_with_post_norms_and_a_mixer_that_caches_one_latent_per_token():
    """Two things an architecture may need that this one does not: a block arrangement with further parts (here a norm
    after each branch, named in ``LayerSpec.extras``), and a mixer whose paged cache holds one latent vector per
    token instead of keys and values (``KVCacheSpec.arrays``).  Both are registered from here, built from random
    weights by name, stepped whole and in portions over a small pool, and compared with a numpy restatement of the
    whole model; no file of the package changes."""
    import plain_qwen2 as plain
    from mimirmind_b200 import registry
    from mimirmind_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
    from mimirmind_b200.engine.loader import make_runtime
    from mimirmind_b200.engine.model import Model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    from mimirmind_b200.parts.base import Block, CacheArray, KVCacheSpec, Mixer
    from mimirmind_b200.weights.store import expected_tensors, random_tensors
    registry._ensure_builtin()
    R = 12                                                     # width of the cached latent

    @registry.MIXERS.register("toy_latent_attention", replace=True)
    class LatentAttention(Mixer):
        """c_t = x_t Wc^T is cached; out_t = Wo . sum_s softmax_s((x_t Wq^T) . c_s / sqrt(R)) c_s over s <= t."""

        @classmethod
        def tensor_specs(cls, spec, prefix):
            d = spec["hidden"]
            return [TensorSpec(prefix + "lat.c", (R, d)), TensorSpec(prefix + "lat.q", (R, d)), TensorSpec(prefix + "lat.o", (d, R))]

        def __init__(self, spec, weights, rt):
            super().__init__(spec, weights, rt)
            self.wc, self.wq, self.wo = (weights.get(n).float() for n in ("lat.c", "lat.q", "lat.o"))

        def kv_cache_spec(self):
            return KVCacheSpec(window=0, arrays=(CacheArray("latent", (R,), torch.float32),))

        def forward(self, x, ctx, cache):
            pool, ps = cache.arrays["latent"], cache.page_size             # [pages, page_size, R]
            assert pool.shape[1:] == (ps, R) and pool.dtype == torch.float32 and cache.k_pages is None
            out = torch.empty_like(x)
            for r in range(ctx.n_requests):
                s, n, kv = ctx.q_start[r], ctx.q_len[r], ctx.kv_len[r]
                xs = x[s:s + n].float()
                pos = torch.arange(kv - n, kv, device=x.device)
                table = cache.block_table[r].long()
                pool[table[pos // ps], pos % ps] = xs @ self.wc.t()         # this step's latents into their pages
                every = torch.arange(kv, device=x.device)
                c = pool[table[every // ps], every % ps]                    # [kv, R], gathered page by page
                score = (xs @ self.wq.t()) @ c.t() / np.sqrt(R)
                score = score.masked_fill(every[None, :] > pos[:, None], float("-inf"))
                out[s:s + n] = ((torch.softmax(score, dim=-1) @ c) @ self.wo.t()).to(x.dtype)
            return out

    @registry.BLOCKS.register("toy_sandwich", replace=True)
    class Sandwich(Block):
        """x += post1(mixer(pre1(x))); x += post2(ffn(pre2(x))): the two post-norms are the layer's extra parts."""

        def forward(self, residual, pending, ctx, cache, successor=None):
            h = self.mixer_norm.forward(residual, pending)
            branch = self.mixer.forward(h, ctx, cache)
            branch = self.extras["post_mixer_norm"].forward(branch.float().contiguous(), None)
            h = self.ffn_norm.forward(residual, branch)
            out = self.feed_forward.forward(h, ctx)
            return self.extras["post_ffn_norm"].forward(out.float().contiguous(), None)

    d, V = 32, 70

    def toy_spec(cfg):
        norm = lambda name: PartSpec("rmsnorm", {"width": d, "eps": 1e-5, "weight": name}, category="norm")
        attn = PartSpec("gqa_attention", dict(hidden=d, num_heads=2, num_kv_heads=1, head_dim=16, window=0, scale=None, qkv_bias=False,
                                              position=PartSpec("rotary_half", {"theta": 100.0, "rotary_dim": 16}),
                                              q="q", k="k", v="v", o="o"))
        ffn = PartSpec("swiglu", {"hidden": d, "intermediate": 40, "gate": "g.weight", "up": "u.weight", "down": "d.weight"})
        layers = (
            LayerSpec("l0.", PartSpec("toy_sandwich"), PartSpec("toy_latent_attention", {"hidden": d}), ffn, norm("n1"), norm("n2"),
                      extras={"post_mixer_norm": norm("p1"), "post_ffn_norm": norm("p2")}),
            LayerSpec("l1.", PartSpec("pre_norm"), attn, ffn, norm("n1"), norm("n2")),
        )
        return ModelSpec("ToySandwich", d, V, 512, PartSpec("token_embedding", {"vocab": V, "width": d, "scale": 1.0, "weight": "emb"}),
                         layers, (ScheduleEntry(0), ScheduleEntry(1)), norm("nf"),
                         PartSpec("lm_head", {"vocab": V, "width": d, "weight": "head", "tied_to": None}))

    registry.register_architecture("ToySandwich", lambda obj, where="": obj, toy_spec, replace=True)
    try:
        entry = registry.get_architecture("ToySandwich")
        spec = entry.build_spec(entry.parse_config({}))
        names = expected_tensors(spec)
        assert {"l0.p1", "l0.p2", "l0.lat.c", "l0.lat.q", "l0.lat.o"} <= set(names)       # the extras' and the mixer's tensors by name
        rt_ = make_runtime("float32")
        tensors = random_tensors(spec, 9, torch.float32, rt_.device)
        w = {k: v.double().cpu().numpy() for k, v in tensors.items()}
        model = Model(spec, tensors, rt_)
        groups = {g.name: g for g in model.cache_groups()}
        assert len(groups) == 2 and any(g.arrays == (("latent", (R,), "float32"),) for g in groups.values())
        runner = ModelRunner(model, 8, 24, 4)                          # pages of 8 tokens, 24 of them per group
        assert runner.native is None                                   # parts without native classes: the Python path
        lat_pool = [p for p in runner.storage.pools.values() if "latent" in p][0]["latent"]
        assert lat_pool.shape == (1, 24, 8, R) and lat_pool.dtype == torch.float32

        def restated(toks):
            T = len(toks)
            x = w["emb"][toks]
            # layer 0: the sandwich around the latent mixer
            h = plain.rms_norm(x, w["l0.n1"], 1e-5)
            c, q = h @ w["l0.lat.c"].T, h @ w["l0.lat.q"].T
            sc = q @ c.T / np.sqrt(R)
            sc = np.where(np.arange(T)[None, :] <= np.arange(T)[:, None], sc, -np.inf)
            pr = np.exp(sc - sc.max(axis=-1, keepdims=True))
            branch = ((pr / pr.sum(axis=-1, keepdims=True)) @ c) @ w["l0.lat.o"].T
            x = x + plain.rms_norm(branch, w["l0.p1"], 1e-5)
            f = plain.swiglu(plain.rms_norm(x, w["l0.n2"], 1e-5), w["l0.g.weight"], w["l0.u.weight"], w["l0.d.weight"])
            x = x + plain.rms_norm(f, w["l0.p2"], 1e-5)
            # layer 1: the ordinary pre-norm block
            h = plain.rms_norm(x, w["l1.n1"], 1e-5)
            pos = np.arange(T)
            qh = plain.rope((h @ w["l1.q.weight"].T).reshape(T, 2, 16), pos, 100.0)
            kh = plain.rope((h @ w["l1.k.weight"].T).reshape(T, 1, 16), pos, 100.0)
            vh = (h @ w["l1.v.weight"].T).reshape(T, 1, 16)
            x = x + plain.attention(qh, kh, vh, 0).reshape(T, 32) @ w["l1.o.weight"].T
            x = x + plain.swiglu(plain.rms_norm(x, w["l1.n2"], 1e-5), w["l1.g.weight"], w["l1.u.weight"], w["l1.d.weight"])
            return plain.rms_norm(x, w["nf"], 1e-5) @ w["head"].T

        def run(cuts, rid, toks):
            runner.add_request(rid)
            outs, p = [], 0
            for c in cuts:
                outs.append(runner.step([StepEntry(rid, toks[p:p + c], list(range(c)))]).cpu().numpy())
                p += c
            return np.concatenate(outs)

        a, b = random_tokens(V, 61, 1), random_tokens(V, 50, 2)
        ref_a, ref_b = restated(a), restated(b)
        whole = run([61], "a", a)
        assert np.abs(whole - ref_a).max() <= 2e-5 * np.abs(ref_a).max()
        parts = run([7, 1, 9, 2, 30, 12], "b", a)                       # portions that end inside pages, at their edges and beyond
        assert np.abs(parts - ref_a).max() <= 2e-5 * np.abs(ref_a).max()
        runner.release("a")
        runner.release("b")
        # two requests side by side in pages that were used before
        runner.add_request("c"); runner.add_request("e")
        both = runner.step([StepEntry("c", b, list(range(50))), StepEntry("e", a[:33], [32])]).cpu().numpy()
        assert runner.manager.reuses() > 0
        assert np.abs(both[:50] - ref_b).max() <= 2e-5 * np.abs(ref_b).max()
        assert np.abs(both[50] - ref_a[32]).max() <= 2e-5 * np.abs(ref_a).max()
        runner.manager.check()
    finally:
        registry.MIXERS.unregister("toy_latent_attention")
        registry.BLOCKS.unregister("toy_sandwich")
        registry.ARCHITECTURES.unregister("ToySandwich")


def test_fused_handover_beside_a_mixer_that_does_not_fuse():
    """bfloat16, sizes the fused small-step path takes: a toy mixer that knows nothing of FactoredRows or sinks sits
    between layers whose attention and feed-forward fuse.  Its neighbours must fall back to the plain hand-over on
    its side and still fuse on the other; every way of cutting gives the same logits within bfloat16 rounding, and
    they agree with the same model run in float32."""
    from mimirmind_b200 import registry
    from mimirmind_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
    from mimirmind_b200.engine.loader import make_runtime
    from mimirmind_b200.engine.model import Model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    from mimirmind_b200.parts.base import Mixer
    from mimirmind_b200.weights.store import random_tensors
    registry._ensure_builtin()
    calls = {"plain": 0}

    @registry.MIXERS.register("toy_scaled_copy", replace=True)
    class ScaledCopy(Mixer):
        """out = x @ W^T, stateless; takes tensors only."""

        @classmethod
        def tensor_specs(cls, spec, prefix):
            return [TensorSpec(prefix + "mix.weight", (spec["hidden"], spec["hidden"]))]

        def __init__(self, spec, weights, rt):
            super().__init__(spec, weights, rt)
            self.w = weights.get("mix.weight")

        def forward(self, x, ctx, cache):
            assert isinstance(x, torch.Tensor)                  # never FactoredRows: the part does not say it fuses
            calls["plain"] += 1
            return (x.float() @ self.w.float().t()).to(x.dtype)

    def toy_spec(cfg):
        d = cfg["hidden_size"]
        norm = lambda name: PartSpec("rmsnorm", {"width": d, "eps": 1e-5, "weight": name})
        attn = PartSpec("gqa_attention", dict(hidden=d, num_heads=4, num_kv_heads=2, head_dim=64, window=0, scale=None, qkv_bias=True,
                                              position=PartSpec("rotary_half", {"theta": 100.0, "rotary_dim": 64}),
                                              q="q", k="k", v="v", o="o"))
        ffn = PartSpec("swiglu", {"hidden": d, "intermediate": 320, "gate": "g.weight", "up": "u.weight", "down": "d.weight"})
        layers = (
            LayerSpec("l0.", PartSpec("pre_norm"), PartSpec("toy_scaled_copy", {"hidden": d}), ffn, norm("n1"), norm("n2")),
            LayerSpec("l1.", PartSpec("pre_norm"), attn, ffn, norm("n1"), norm("n2")),
        )
        return ModelSpec("ToyFusedForTest", d, cfg["vocab_size"], 512,
                         PartSpec("token_embedding", {"vocab": cfg["vocab_size"], "width": d, "scale": 1.0, "weight": "emb"}),
                         layers, (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(0)), norm("nf"),
                         PartSpec("lm_head", {"vocab": cfg["vocab_size"], "width": d, "weight": "head", "tied_to": "emb"}))

    registry.register_architecture("ToyFusedForTest", lambda obj, where="": obj, toy_spec, replace=True)
    try:
        entry = registry.get_architecture("ToyFusedForTest")
        spec = entry.build_spec(entry.parse_config({"hidden_size": 256, "vocab_size": 90}))
        rt16, rt32 = make_runtime("bfloat16"), make_runtime("float32")
        tensors = random_tensors(spec, 11, torch.bfloat16, rt16.device)
        model16 = Model(spec, {k: v.clone() for k, v in tensors.items()}, rt16)
        model32 = Model(spec, {k: v.float() for k, v in tensors.items()}, rt32)
        blocks = model16.layers
        assert blocks[1].mixer.fuses(5) and blocks[1].mixer.fuses(40) and not blocks[1].mixer.fuses(200)
        assert blocks[0].feed_forward.fuses(5) and not blocks[0].mixer.fuses(5)
        assert blocks[1].entry_norm(5) is not None and blocks[0].entry_norm(5) is None
        toks = random_tokens(90, 70, 4)

        def run(model, cuts, rid):
            runner = ModelRunner(model, 16, 16, 4)
            runner.add_request(rid)
            outs, p = [], 0
            for c in cuts:
                outs.append(runner.step([StepEntry(rid, toks[p:p + c], list(range(c)))]).cpu().numpy())
                p += c
            return np.concatenate(outs)

        exact = run(model32, [70], "x")
        scale = np.abs(exact).max()
        whole = run(model16, [70], "a")                             # one step above 64 tokens: nothing fuses
        assert np.abs(whole - exact).max() <= 4e-2 * scale
        for cuts in ([40, 30], [7, 1, 1, 30, 2, 13, 16], [64, 6], [1] * 10 + [60]):
            before = calls["plain"]
            got = run(model16, cuts, ("b", len(cuts)))
            assert calls["plain"] == before + 2 * len(cuts)          # the toy mixer ran in both of its schedule entries
            assert np.abs(got - exact).max() <= 4e-2 * scale, cuts
            assert np.abs(got - whole).max() <= 4e-2 * scale, cuts
        from mimirmind_b200.kernels import ops
        ops.check_tcgen05_errors(rt16.device)
    finally:
        registry.MIXERS.unregister("toy_scaled_copy")
        registry.ARCHITECTURES.unregister("ToyFusedForTest")


# ---- another position encoding and a feed-forward with routing, defined here ---------------------------------

def test_toy_position_encoding_and_routed_feed_forward(tmp_path):
    """A position encoding the fused kernel does not know (each head's q and k are scaled by a factor that depends
    on the position) and a feed-forward that routes every token to one of two experts by fp32 router logits are
    registered from outside the package and run through the engine: whole and in portions, against a plain
    computation put together from the plain implementation's own part functions."""
    from mimirmind_b200 import registry
    from mimirmind_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
    from mimirmind_b200.engine.loader import make_runtime
    from mimirmind_b200.engine.model import Model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    from mimirmind_b200.kernels import ops as kops
    from mimirmind_b200.parts.base import FeedForward, PositionEncoding
    from mimirmind_b200.weights.store import random_tensors
    registry._ensure_builtin()

    @registry.POSITION_ENCODINGS.register("toy_position_scale", replace=True)
    class PositionScale(PositionEncoding):
        def __init__(self, spec, weights, rt):
            super().__init__(spec, weights, rt)
            self.rate = float(spec["rate"])

        def apply(self, q, k, positions):
            f = (1.0 + self.rate * positions.float()).view(-1, 1, 1)
            q.mul_(torch.cos(f * 0.1).to(q.dtype))
            k.mul_(f.to(k.dtype))

    @registry.FEED_FORWARDS.register("toy_two_experts", replace=True)
    class TwoExperts(FeedForward):
        @classmethod
        def tensor_specs(cls, spec, prefix):
            d = spec["hidden"]
            return [TensorSpec(prefix + "router.weight", (2, d)), TensorSpec(prefix + "experts.weight", (2, d, d))]

        def __init__(self, spec, weights, rt):
            super().__init__(spec, weights, rt)
            self.router = weights.get("router.weight")
            self.experts = weights.get("experts.weight")

        def forward(self, x, ctx):
            logits = torch.empty((x.shape[0], 2), dtype=torch.float32, device=x.device)
            kops.gemm_simt(x, self.router, None, logits)                   # router logits in fp32, per token
            choice = logits.argmax(-1)
            out = torch.empty_like(x)
            for e in range(2):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    y = torch.empty((rows.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
                    kops.gemm_simt(x[rows].contiguous(), self.experts[e].contiguous(), None, y)
                    out[rows] = y
            return out

    d, H, G, hd, V = 48, 3, 1, 16, 70
    norm = lambda name: PartSpec("rmsnorm", {"width": d, "eps": 1e-5, "weight": name})
    attn = PartSpec("gqa_attention", dict(hidden=d, num_heads=H, num_kv_heads=G, head_dim=hd, window=0, scale=None, qkv_bias=True,
                                          position=PartSpec("toy_position_scale", {"rate": 0.03}), q="q", k="k", v="v", o="o"))
    layer = LayerSpec("l0.", PartSpec("pre_norm"), attn, PartSpec("toy_two_experts", {"hidden": d}), norm("n1"), norm("n2"))
    spec = ModelSpec("ToyRouted", d, V, 256, PartSpec("token_embedding", {"vocab": V, "width": d, "scale": 1.0, "weight": "emb"}),
                     (layer,), (ScheduleEntry(0),), norm("nf"), PartSpec("lm_head", {"vocab": V, "width": d, "weight": "head", "tied_to": "emb"}))
    try:
        rt_ = make_runtime("float32")
        tensors = random_tensors(spec, 3, torch.float32, rt_.device)
        w = {k: v.double().cpu().numpy() for k, v in tensors.items()}
        model = Model(spec, tensors, rt_)
        toks = random_tokens(V, 50, 4)

        def run(cuts, rid, runner):
            runner.add_request(rid)
            outs, p = [], 0
            for c in cuts:
                outs.append(runner.step([StepEntry(rid, toks[p:p + c], list(range(c)))]).cpu().numpy())
                p += c
            return np.concatenate(outs)

        runner = ModelRunner(model, 16, 16, 4)
        whole = run([50], "a", runner)
        parts = run([9, 2, 1, 30, 8], "b", runner)
        assert np.abs(whole - parts).max() < 1e-5
        # plain computation from the plain implementation's part functions
        T = len(toks)
        pos = np.arange(T)
        x = plain.embedding(w["emb"], toks)
        n = plain.rms_norm(x, w["l0.n1"], 1e-5)
        q = plain.linear(n, w["l0.q.weight"], w["l0.q.bias"]).reshape(T, H, hd)
        k = plain.linear(n, w["l0.k.weight"], w["l0.k.bias"]).reshape(T, G, hd)
        v = plain.linear(n, w["l0.v.weight"], w["l0.v.bias"]).reshape(T, G, hd)
        f = (1.0 + 0.03 * pos).reshape(T, 1, 1)
        q, k = q * np.cos(f * 0.1), k * f
        x = x + plain.linear(plain.attention(q, k, v, 0).reshape(T, H * hd), w["l0.o.weight"])
        n = plain.rms_norm(x, w["l0.n2"], 1e-5)
        choice = (n @ w["l0.router.weight"].T).argmax(-1)
        y = np.stack([n[t] @ w["l0.experts.weight"][choice[t]].T for t in range(T)])
        x = x + y
        ref = plain.linear(plain.rms_norm(x, w["nf"], 1e-5), w["emb"])
        assert len(set(choice.tolist())) == 2                      # both experts were used
        assert np.abs(whole - ref).max() < 2e-5 * max(1.0, np.abs(ref).max())
    finally:
        registry.POSITION_ENCODINGS.unregister("toy_position_scale")
        registry.FEED_FORWARDS.unregister("toy_two_experts")


# ---- the order of layers is data: a layer named twice, an entry that reads another entry's cache ------------------

def _plain_scheduled(w, cfg, schedule, windows, tokens):
    """Whole-sequence forward of a model whose schedule names layers more than once and lets entries attend over the
    keys and values that an earlier entry made (plain parts; one function per part from plain_qwen2)."""
    T, H, G, hd = len(tokens), cfg["H"], cfg["G"], cfg["hd"]
    pos = np.arange(T)
    x = plain.embedding(w["emb"], tokens)
    kept = {}
    for idx, (layer, cache_from) in enumerate(schedule):
        p = f"l{layer}."
        n = plain.rms_norm(x, w[p + "n1"], cfg["eps"])
        q = plain.rope(plain.linear(n, w[p + "q.weight"], w[p + "q.bias"]).reshape(T, H, hd), pos, cfg["theta"])
        if cache_from is None:
            k = plain.rope(plain.linear(n, w[p + "k.weight"], w[p + "k.bias"]).reshape(T, G, hd), pos, cfg["theta"])
            v = plain.linear(n, w[p + "v.weight"], w[p + "v.bias"]).reshape(T, G, hd)
            kept[idx] = (k, v)
        else:
            k, v = kept[cache_from]
        o = plain.attention(q, k, v, windows[layer]).reshape(T, H * hd)
        x = x + plain.linear(o, w[p + "o.weight"])
        n = plain.rms_norm(x, w[p + "n2"], cfg["eps"])
        x = x + plain.swiglu(n, w[p + "g.weight"], w[p + "u.weight"], w[p + "d.weight"])
    return plain.linear(plain.rms_norm(x, w["nf"], cfg["eps"]), w["emb"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("use_native", [True, False])
@pytest.mark.parametrize("sizes", [(176, 83, 5, 1, 48, 208), (256, 131, 4, 2, 64, 320)])   # generic kernels; tensor-core and fused ones
def test_a_layer_named_twice_and_an_entry_that_reads_another_entrys_cache(sizes, dtype, use_native, monkeypatch):
    """Three layers of the built-in parts, five schedule entries: layer 0, layer 1 (a window), layer 2 attending over
    what entry 0 kept (with a window of its own), layer 0 a second time with a cache of its own, layer 2 over entry 0
    again.  Whole, in portions and token by token, through the library's executor and through the Python parts,
    against the plain composition; few pages, so that the window's group gives pages back."""
    from mimirmind_b200 import registry
    from mimirmind_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from mimirmind_b200.engine import native
    from mimirmind_b200.engine.loader import make_runtime
    from mimirmind_b200.engine.model import Model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    from mimirmind_b200.weights.store import random_tensors
    registry._ensure_builtin()
    monkeypatch.setattr(native, "ENABLED", use_native)
    d, V, H, G, hd, F = sizes
    cfg = dict(H=H, G=G, hd=hd, eps=3e-6, theta=5000.0)
    windows = [0, 20, 28]
    schedule = [(0, None), (1, None), (2, 0), (0, None), (2, 0)]
    norm = lambda name: PartSpec("rmsnorm", {"width": d, "eps": cfg["eps"], "weight": name})

    def attn(window):
        return PartSpec("gqa_attention", dict(hidden=d, num_heads=H, num_kv_heads=G, head_dim=hd, window=window, scale=None, qkv_bias=True,
                                              position=PartSpec("rotary_half", {"theta": cfg["theta"], "rotary_dim": hd}),
                                              q="q", k="k", v="v", o="o"))
    ffn = PartSpec("swiglu", {"hidden": d, "intermediate": F, "gate": "g.weight", "up": "u.weight", "down": "d.weight"})
    layers = tuple(LayerSpec(f"l{i}.", PartSpec("pre_norm"), attn(windows[i]), ffn, norm("n1"), norm("n2")) for i in range(3))
    spec = ModelSpec("ScheduledForTest", d, V, 512, PartSpec("token_embedding", {"vocab": V, "width": d, "scale": 1.0, "weight": "emb"}),
                     layers, tuple(ScheduleEntry(l, c) for l, c in schedule), norm("nf"),
                     PartSpec("lm_head", {"vocab": V, "width": d, "weight": "head", "tied_to": "emb"}))
    rt_ = make_runtime(dtype)
    tensors = random_tensors(spec, 5, torch.bfloat16, rt_.device)
    model = Model(spec, {k: (v.float() if dtype == "float32" and v.dtype == torch.bfloat16 else v.clone()) for k, v in tensors.items()}, rt_)
    groups = {g.name: g for g in model.cache_groups()}
    assert sorted(len(g.entries) for g in groups.values()) == [1, 2]      # entries 0 and 3 keep everything, entry 1 a window
    w = {k: v.float().cpu().numpy().astype(np.float64) for k, v in tensors.items()}
    toks = random_tokens(V, 90, 9)
    want = _plain_scheduled(w, cfg, schedule, windows, toks)
    scale = np.abs(want).max()
    tol = 2e-4 if dtype == "float32" else 4e-2

    def run(cuts, rid, runner):
        runner.add_request(rid)
        outs, p = [], 0
        for c in cuts:
            outs.append(runner.step([StepEntry(rid, toks[p:p + c], list(range(c)))]).float().cpu().numpy())
            p += c
        runner.release(rid)
        return np.concatenate(outs)

    runner = ModelRunner(model, 8, 16, 2)                               # 128 tokens of pages for 90: nothing to spare twice over
    assert (runner.native is not None) == use_native
    first = None
    for n, cuts in enumerate(([90], [58] + [1] * 32, [2, 17, 3, 40, 2, 26], [33, 31, 2, 24])):
        got = run(cuts, f"r{n}", runner)
        assert np.abs(got - want).max() <= tol * scale, (cuts, np.abs(got - want).max() / scale)
        if dtype == "float32":
            first = got if first is None else first
            assert np.array_equal(got, first), cuts                     # 32-bit: the same bits however the tokens are cut
    runner.check_errors()

    # an entry may not look further back than the entry whose cache it reads keeps
    bad = ModelSpec("ScheduledBad", d, V, 512, spec.embedding, layers, (ScheduleEntry(1), ScheduleEntry(0, 0)), spec.final_norm, spec.head)
    with pytest.raises(ValueError, match="keeps only"):
        Model(bad, {k: v.clone() for k, v in tensors.items()}, rt_)
