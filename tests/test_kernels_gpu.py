"""Each kernel alone against a plain fp32/float64 reference of the same operation, at sizes other than
the engine's tiny models (widths and vocabularies that are no power of two, head sizes in steps of
16, odd head and group counts), with inputs made so that an addressing fault shows."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from mimirmind_b200.kernels import ops as o
    return o


def t(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a)).to(DEV).to(dtype).contiguous()


def bf16_round(a):
    return torch.as_tensor(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


# ---- embedding -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,scale", [(136, 1.0), (132, 1.0), (3584, 0.5), (8200, 1.0)])
def test_embedding(dtype, d, scale):
    """Widths that are and are not a multiple of 8 (the bfloat16 table has a 16-byte-load kernel for the former)."""
    rng = np.random.RandomState(d)
    V = 1003
    table = t(rng.randn(V, d), dtype)
    ids = torch.tensor([0, V - 1, 17, V, -3, 500], dtype=torch.int32, device=DEV)
    out = torch.full((6, d), 7.0, dtype=torch.float32, device=DEV)
    ops().embedding(ids, table, out, scale)
    ref = plain.embedding(table.float().cpu().numpy().astype(np.float64), ids.cpu().tolist()) * scale
    assert np.array_equal(out.cpu().numpy(), ref.astype(np.float32))
    assert not out[3].any() and not out[4].any()          # ids outside the table give zero rows


# ---- residual add + RMSNorm -----------------------------------------------------------------
@pytest.mark.parametrize("d", [80, 3584 + 16, 13000])
@pytest.mark.parametrize("act,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)])
def test_add_rmsnorm(d, act, wdt):
    rng = np.random.RandomState(d)
    n, eps = 7, 3e-5
    res = t(rng.randn(n, d) * 3)
    delta = t(rng.randn(n, d), act)
    w = t(1 + 0.1 * rng.randn(d), wdt)
    x = res.double().cpu().numpy() + delta.double().cpu().numpy()
    ref = plain.rms_norm(x, w.double().cpu().numpy(), eps)
    out = torch.empty((n, d), dtype=act, device=DEV)
    res2 = res.clone()
    ops().add_rmsnorm(res2, delta, w, eps, out)
    assert np.abs(res2.cpu().numpy() - x).max() < 1e-6                      # the sum stays in fp32
    tol = 2e-6 if act == torch.float32 else 2 ** -8
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
    # gather form: chosen rows only, residual untouched
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out3 = torch.empty((3, d), dtype=act, device=DEV)
    res3 = res.clone()
    ops().add_rmsnorm(res3, delta, w, eps, out3, rows)
    assert torch.equal(res3, res)
    assert torch.equal(out3, out[[5, 0, 5]])
    # no delta
    out4 = torch.empty((n, d), dtype=act, device=DEV)
    ops().add_rmsnorm(res.clone(), None, w, eps, out4)
    ref4 = plain.rms_norm(res.double().cpu().numpy(), w.double().cpu().numpy(), eps)
    assert np.abs(out4.float().cpu().numpy() - ref4).max() <= tol * np.abs(ref4).max()


def test_rmsnorm_row_does_not_depend_on_the_batch():
    rng = np.random.RandomState(1)
    d = 1000
    res = t(rng.randn(9, d))
    w = t(rng.randn(d))
    a = torch.empty((9, d), device=DEV)
    b = torch.empty((1, d), device=DEV)
    ops().add_rmsnorm(res.clone(), None, w, 1e-6, a)
    ops().add_rmsnorm(res[4:5].clone(), None, w, 1e-6, b)
    assert torch.equal(a[4], b[0])


# ---- SiLU * up ---------------------------------------------------------------------------------
@pytest.mark.parametrize("F,dtype", [(176, torch.float32), (352, torch.bfloat16), (75, torch.bfloat16), (18944, torch.bfloat16)])
def test_silu_mul(F, dtype):
    rng = np.random.RandomState(F)
    n = 5
    gu = t(rng.randn(n, 2 * F) * 4, dtype)
    out = torch.empty((n, F), dtype=dtype, device=DEV)
    ops().silu_mul(gu, out)
    g, u = gu[:, :F].double().cpu().numpy(), gu[:, F:].double().cpu().numpy()
    ref = g / (1 + np.exp(-g)) * u
    tol = 1e-6 if dtype == torch.float32 else 2 ** -8
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol * max(np.abs(ref).max(), 1)


# ---- fp32 matrix product ------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 130, 67), (65, 64, 16), (2, 1003, 352), (130, 200, 129)])
def test_gemm_simt_fp32(M, N, K):
    rng = np.random.RandomState(M * N + K)
    a, w, b = t(rng.randn(M, K)), t(rng.randn(N, K)), t(rng.randn(N))
    out = torch.empty((M, N), device=DEV)
    ops().gemm_simt(a, w, b, out)
    ref = a.double().cpu().numpy() @ w.double().cpu().numpy().T + b.double().cpu().numpy()
    assert np.abs(out.cpu().numpy() - ref).max() <= 2e-6 * np.abs(ref).max() * np.sqrt(K)
    # a row's result does not depend on M or on its place in the batch
    one = torch.empty((1, N), device=DEV)
    ops().gemm_simt(a[M - 1:M].contiguous(), w, b, one)
    assert torch.equal(one[0], out[M - 1])


def test_gemm_simt_mixed_dtypes():
    rng = np.random.RandomState(3)
    a, w = t(rng.randn(5, 96), torch.bfloat16), t(rng.randn(40, 96))
    out = torch.empty((5, 40), dtype=torch.bfloat16, device=DEV)
    ops().gemm_simt(a, w, None, out)
    ref = a.double().cpu().numpy() @ w.double().cpu().numpy().T
    assert np.abs(out.float().cpu().numpy() - ref).max() <= 2 ** -8 * np.abs(ref).max()


# ---- bias + rotary + paged K/V write ---------------------------------------------------------------
def paged_layout(rng, lens, page_size, extra_pages=3):
    """Shuffled page tables for requests of the given lengths."""
    need = [(n + page_size - 1) // page_size for n in lens]
    total = sum(need) + extra_pages
    perm = rng.permutation(total)
    width = max(need)
    table = np.full((len(lens), width), -1, dtype=np.int32)
    k = 0
    for r, c in enumerate(need):
        table[r, :c] = perm[k:k + c]
        k += c
    return table, total


@pytest.mark.parametrize("dtype,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("H,G,hd,rot,ps", [(4, 2, 16, 16, 16), (6, 3, 48, 48, 8), (7, 1, 128, 128, 16), (3, 1, 32, 16, 32)])
def test_qkv_rope_kvwrite(dtype, wdt, H, G, hd, rot, ps):
    rng = np.random.RandomState(H * hd)
    theta = 1e6
    lens_before, q_lens = [0, 37, 130], [5, 1, 19]
    table, pages = paged_layout(rng, [a + b for a, b in zip(lens_before, q_lens)], ps)
    n = sum(q_lens)
    pos = np.concatenate([np.arange(a, a + b) for a, b in zip(lens_before, q_lens)]).astype(np.int32)
    req = np.concatenate([np.full(b, r) for r, b in enumerate(q_lens)]).astype(np.int32)
    width = (H + 2 * G) * hd
    qkv = t(rng.randn(n, width), dtype)
    bias = t(rng.randn(width) * 0.5, wdt)
    kp = torch.full((pages, G, ps, hd), 768.0, dtype=dtype, device=DEV)
    vp = torch.full((pages, G, ps, hd), 768.0, dtype=dtype, device=DEV)
    q_out = torch.empty((n, H * hd), dtype=dtype, device=DEV)
    ops().qkv_rope_kvwrite(qkv, bias, q_out, kp, vp, t(pos, torch.int32), t(req, torch.int32), t(table, torch.int32),
                           ps, H, G, hd, rot, theta)
    x = qkv.double().cpu().numpy() + bias.double().cpu().numpy()
    q = x[:, :H * hd].reshape(n, H, hd)
    k = x[:, H * hd:(H + G) * hd].reshape(n, G, hd)
    v = x[:, (H + G) * hd:].reshape(n, G, hd)

    def rot_part(a):
        out = a.copy()
        out[..., :rot] = plain.rope(a[..., :rot], pos, theta)
        return out
    q_ref, k_ref = rot_part(q), rot_part(k)
    tol = 3e-6 * max(1.0, pos.max() / 50) if dtype == torch.float32 else 2 ** -8
    assert np.abs(q_out.float().cpu().numpy().reshape(n, H, hd) - q_ref).max() <= tol * np.abs(q_ref).max()
    kp_h, vp_h = kp.float().cpu().numpy(), vp.float().cpu().numpy()
    written = np.zeros((pages, ps), dtype=bool)
    for i in range(n):
        page, slot = table[req[i], pos[i] // ps], pos[i] % ps
        written[page, slot] = True
        assert np.abs(kp_h[page, :, slot] - k_ref[i]).max() <= tol * np.abs(k_ref).max()
        assert np.abs(vp_h[page, :, slot] - v[i]).max() <= tol * np.abs(v).max()
    # nothing else in the pool was touched
    untouched = ~written[:, None, :].repeat(G, axis=1)
    assert (kp_h[untouched] == 768.0).all() and (vp_h[untouched] == 768.0).all()


@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16, None])
@pytest.mark.parametrize("H,G,hd,ps,interleave", [(4, 2, 16, 16, False), (6, 3, 48, 8, True), (7, 1, 128, 16, True),
                                                   (5, 5, 80, 32, False), (40, 8, 128, 16, True)])
def test_qkv_rope_with_step_tables(wdt, H, G, hd, ps, interleave):
    """The variant that reads rotation factors and cache places from the step's tables: against the plain rotation,
    and bit-equal to the kernel that works them out itself."""
    rng = np.random.RandomState(H * hd + ps)
    theta = 1e4
    lens_before, q_lens = [0, 37, 130], [21, 1, 67]
    table, pages = paged_layout(rng, [a + b for a, b in zip(lens_before, q_lens)], ps)
    n = sum(q_lens)
    pos = np.concatenate([np.arange(a, a + b) for a, b in zip(lens_before, q_lens)]).astype(np.int32)
    req = np.concatenate([np.full(b, r) for r, b in enumerate(q_lens)]).astype(np.int32)
    width = (H + 2 * G) * hd
    qkv = t(rng.randn(n, width), torch.bfloat16)
    bias = t(rng.randn(width) * 0.5, wdt) if wdt is not None else None
    d_pos, d_req, d_table = t(pos, torch.int32), t(req, torch.int32), t(table, torch.int32)
    rope = ops().rope_table(d_pos, hd, theta)
    slots = ops().slot_mapping(d_pos, d_req, d_table, ps)
    outs = []
    for which in ("tables", "positions"):
        kp = torch.full((pages, G, ps, hd), 768.0, dtype=torch.bfloat16, device=DEV)
        vp = torch.full((pages, G, ps, hd), 768.0, dtype=torch.bfloat16, device=DEV)
        q_out = torch.empty((n, H * hd), dtype=torch.bfloat16, device=DEV)
        src, b = qkv, bias
        if interleave:
            src = ops().interleave_halves(qkv.t().contiguous(), H + G, hd).t().contiguous()
            b = ops().interleave_halves(bias, H + G, hd) if bias is not None else None
        if which == "tables":
            ops().qkv_rope_tables(src, b, q_out, kp, vp, rope, slots, ps, H, G, hd, interleave=interleave)
        else:
            ops().qkv_rope_kvwrite(src, b, q_out, kp, vp, d_pos, d_req, d_table, ps, H, G, hd, hd, theta, interleave=interleave)
        outs.append((q_out, kp, vp))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    x = qkv.double().cpu().numpy() + (bias.double().cpu().numpy() if bias is not None else 0.0)
    q_ref = plain.rope(x[:, :H * hd].reshape(n, H, hd), pos, theta)
    k_ref = plain.rope(x[:, H * hd:(H + G) * hd].reshape(n, G, hd), pos, theta)
    v_ref = x[:, (H + G) * hd:].reshape(n, G, hd)
    q_out, kp, vp = outs[0]
    tol = 2 ** -8
    assert np.abs(q_out.float().cpu().numpy().reshape(n, H, hd) - q_ref).max() <= tol * np.abs(q_ref).max()
    kp_h, vp_h = kp.float().cpu().numpy(), vp.float().cpu().numpy()
    written = np.zeros((pages, ps), dtype=bool)
    for i in range(n):
        page, slot = table[req[i], pos[i] // ps], pos[i] % ps
        written[page, slot] = True
        assert np.abs(kp_h[page, :, slot] - k_ref[i]).max() <= tol * np.abs(k_ref).max()
        assert np.abs(vp_h[page, :, slot] - v_ref[i]).max() <= tol * np.abs(v_ref).max()
    untouched = ~written[:, None, :].repeat(G, axis=1)
    assert (kp_h[untouched] == 768.0).all() and (vp_h[untouched] == 768.0).all()
    # without pages only q is written
    q2 = torch.empty_like(q_out)
    src = ops().interleave_halves(qkv.t().contiguous(), H + G, hd).t().contiguous() if interleave else qkv
    b = ops().interleave_halves(bias, H + G, hd) if (interleave and bias is not None) else bias
    ops().qkv_rope_tables(src, b, q2, None, None, rope, None, ps, H, G, hd, interleave=interleave)
    assert torch.equal(q2, q_out)


# ---- attention -------------------------------------------------------------------------------------
def make_attention_case(rng, H, G, hd, ps, ctx_lens, q_lens, dtype, spike=None):
    """Requests with ``ctx_lens[r]`` cached tokens of which the last ``q_lens[r]`` are this step's queries.
    ``spike = (request, query offset, key position, head)`` makes one far key dominate one query."""
    table, pages = paged_layout(rng, ctx_lens, ps)
    K = [rng.randn(n, G, hd) for n in ctx_lens]
    V = [rng.randn(n, G, hd) for n in ctx_lens]
    Q = [rng.randn(qn, H, hd) for qn in q_lens]
    if spike is not None:
        r, qo, kpos, h = spike
        u = rng.randn(hd)
        u /= np.linalg.norm(u)
        Q[r][qo, h] = 12.0 * np.sqrt(np.sqrt(hd)) * u
        K[r][kpos, (h * G) // H] = 12.0 * np.sqrt(np.sqrt(hd)) * u
        V[r][kpos, (h * G) // H] = 50.0 + np.arange(hd)             # a value no other position has
    rnd = bf16_round if dtype == torch.bfloat16 else (lambda a: np.asarray(a, dtype=np.float32).astype(np.float64))
    K, V, Q = [rnd(a) for a in K], [rnd(a) for a in V], [rnd(a) for a in Q]
    kp = np.zeros((pages, G, ps, hd)); vp = np.zeros((pages, G, ps, hd))
    for r, n in enumerate(ctx_lens):
        for p in range(n):
            kp[table[r, p // ps], :, p % ps] = K[r][p]
            vp[table[r, p // ps], :, p % ps] = V[r][p]
    pos = np.concatenate([np.arange(n - qn, n) for n, qn in zip(ctx_lens, q_lens)]).astype(np.int32)
    req = np.concatenate([np.full(qn, r) for r, qn in enumerate(q_lens)]).astype(np.int32)
    return dict(Q=Q, K=K, V=V, q=t(np.concatenate(Q).reshape(len(pos), H * hd), dtype), kp=t(kp, dtype), vp=t(vp, dtype),
                pos=t(pos, torch.int32), req=t(req, torch.int32), table=t(table, torch.int32), ctx_lens=ctx_lens,
                q_lens=q_lens)


def attention_reference(case, window):
    outs = []
    for r, (n, qn) in enumerate(zip(case["ctx_lens"], case["q_lens"])):
        H, hd = case["Q"][r].shape[1:]
        qfull = np.zeros((n, H, hd))
        qfull[n - qn:] = case["Q"][r]
        outs.append(plain.attention(qfull, case["K"][r], case["V"][r], window)[n - qn:])
    return np.concatenate(outs)


ATT_SHAPES = [(4, 2, 16, 16), (6, 1, 32, 8), (6, 3, 48, 16), (5, 5, 80, 16), (7, 1, 128, 16), (8, 2, 64, 32), (3, 1, 256, 16)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,ps", ATT_SHAPES)
@pytest.mark.parametrize("window", [0, 50])
def test_attention_generic(dtype, H, G, hd, ps, window):
    rng = np.random.RandomState(H + hd + window)
    case = make_attention_case(rng, H, G, hd, ps, [300, 1, 77, 129], [40, 1, 77, 2], dtype, spike=(0, 39, 3 if not window else 255, H - 1))
    out = torch.empty_like(case["q"])
    ops().attention_generic(case["q"], case["kp"], case["vp"], out, case["pos"], case["req"], case["table"], ps, H, G, hd,
                            window, 1.0 / np.sqrt(hd))
    ref = attention_reference(case, window)
    tol = 3e-6 if dtype == torch.float32 else 2 ** -8
    got = out.float().cpu().numpy().reshape(ref.shape)
    assert np.abs(got - ref).max() <= tol * np.abs(ref).max()
    # the spiked query really found its far key
    assert abs(ref[39, H - 1, 0] - 50.0) < 1.0


def run_bf16_attention(case, H, G, hd, ps, window, prefill_min=None, split=None, target=None, tc=True, tma=True):
    """Through the engine's own plan builder, with a hand-made step context."""
    from mimirmind_b200.kernels import attention_bf16 as ab
    from mimirmind_b200.parts.base import LayerCache, Runtime, StepContext
    q_lens, ctx_lens = case["q_lens"], case["ctx_lens"]
    q_start = list(np.cumsum([0] + q_lens[:-1]))
    n = sum(q_lens)
    ctx = StepContext(n_tokens=n, n_requests=len(q_lens), token_ids=case["pos"], positions=case["pos"], token_req=case["req"],
                      q_start=q_start, q_len=q_lens, kv_len=ctx_lens, req_meta=None, state_slots=None, block_tables={},
                      logit_rows=None, n_logit_rows=0, page_size=ps, runtime=Runtime(torch.bfloat16, torch.device(DEV)),
                      max_kv_len=max(ctx_lens), max_q_len=max(q_lens))
    cache = LayerCache(k_pages=case["kp"], v_pages=case["vp"], block_table=case["table"], page_size=ps)
    old = (ab.PREFILL_MIN, ab.FIXED_SPLIT, ab.TARGET_CTAS, ab.USE_TCGEN05_PREFILL, ab.USE_TMA_DECODE)
    try:
        ab.USE_TCGEN05_PREFILL = tc
        ab.USE_TMA_DECODE = tma
        if prefill_min is not None:
            ab.PREFILL_MIN = prefill_min
        if split is not None:
            ab.FIXED_SPLIT = split                             # cut by absolute position: many splits per token
        if target is not None:
            ab.TARGET_CTAS = target
        out = torch.zeros_like(case["q"])
        ab.run(case["q"], cache, out, ctx, H, G, hd, window, 1.0 / np.sqrt(hd))
        plan = ctx.plans[("attention_bf16", H, G, hd)]
    finally:
        ab.PREFILL_MIN, ab.FIXED_SPLIT, ab.TARGET_CTAS, ab.USE_TCGEN05_PREFILL, ab.USE_TMA_DECODE = old
        ops().check_tcgen05_errors(case["q"].device)
    return out, plan


@pytest.mark.parametrize("H,G,hd,ps", [(7, 1, 128, 16), (8, 2, 64, 32), (28, 4, 128, 16), (16, 1, 64, 8), (3, 3, 128, 64), (40, 8, 128, 16)])
@pytest.mark.parametrize("window", [0, 100])
def test_attention_tensor_core_kernels(H, G, hd, ps, window):
    rng = np.random.RandomState(H * 3 + hd + window)
    ctx_lens, q_lens = [700, 64, 333, 1, 130, 900], [200, 64, 1, 1, 2, 17]
    # the dominant key sits far back (or at the window's far edge) and at a page's last slot
    far = 15 if not window else 700 - 1 - 99
    case = make_attention_case(rng, H, G, hd, ps, ctx_lens, q_lens, torch.bfloat16, spike=(0, 199, far, H - 1))
    ref = attention_reference(case, window)
    assert abs(ref[199, H - 1, 0] - 50.0) < 1.0
    for kwargs in (dict(), dict(prefill_min=10 ** 6, split=128), dict(prefill_min=10 ** 6, split=128, tma=False), dict(prefill_min=10 ** 6, target=10 ** 6),
                   dict(prefill_min=10 ** 6, target=10 ** 6, tma=False),
                   dict(prefill_min=10 ** 6, target=1), dict(prefill_min=1, tc=False), dict(prefill_min=1)):
        out, plan = run_bf16_attention(case, H, G, hd, ps, window, **kwargs)
        got = out.float().cpu().numpy().reshape(ref.shape)
        err = np.abs(got - ref)
        assert err.max() <= 2.5 * 2 ** -8 * np.abs(ref).max(), (kwargs, np.unravel_index(err.argmax(), err.shape))
    assert plan.n_tiles > 0 and plan.n_items == 0                  # the last run was all tiles


@pytest.mark.parametrize("H,G,hd,ps,n,size", [(28, 4, 128, 16, 8, 8), (28, 4, 128, 16, 16, 4), (28, 4, 128, 16, 30, 2), (8, 2, 64, 32, 16, 8), (6, 2, 64, 8, 32, 4),
                                              (40, 8, 128, 16, 8, 4)])
@pytest.mark.parametrize("window", [0, 100])
def test_attention_decode_cluster_merge(H, G, hd, ps, n, size, window):
    """Single tokens of n requests: the splits of a token are a thread-block cluster that merges its partial results
    through shared memory.  Contexts from one key (most CTAs of the cluster have no keys) to many tiles per split."""
    rng = np.random.RandomState(n * 7 + hd + window)
    base = [1, 63, 64, 65, 300, 1000, 129, 2, 511, 512, 513, 17]
    ctx_lens = [base[i % len(base)] + (i // len(base)) * 37 for i in range(n)]
    far = 3 if not window else 1000 - 1 - 99
    case = make_attention_case(rng, H, G, hd, ps, ctx_lens, [1] * n, torch.bfloat16, spike=(5, 0, far, H - 1))
    ref = attention_reference(case, window)
    assert abs(ref[5, H - 1, 0] - 50.0) < 1.0
    out, plan = run_bf16_attention(case, H, G, hd, ps, window)
    assert plan.cluster and plan.max_splits == size and plan.part_o is None
    err = np.abs(out.float().cpu().numpy().reshape(ref.shape) - ref)
    assert err.max() <= 2.5 * 2 ** -8 * np.abs(ref).max(), np.unravel_index(err.argmax(), err.shape)
    # the same through scratch memory and the merge kernel
    from mimirmind_b200.kernels import attention_bf16 as ab
    old = ab.USE_CLUSTER_MERGE
    try:
        ab.USE_CLUSTER_MERGE = False
        out2, plan2 = run_bf16_attention(case, H, G, hd, ps, window)
    finally:
        ab.USE_CLUSTER_MERGE = old
    assert not plan2.cluster and plan2.part_o is not None
    assert np.abs(out2.float().cpu().numpy() - out.float().cpu().numpy()).max() <= 2 ** -7 * np.abs(ref).max()


@pytest.mark.parametrize("n_keys", [4096, 8192])
@pytest.mark.parametrize("far", ["first tile", "page edge"])
def test_attention_over_thousands_of_keys(n_keys, far):
    """One KV head with five query heads (the group of the 14B- and 32B-shaped models), head size 128, thousands of
    cached keys: the tcgen05 prefill kernel over 32 and 64 key tiles (every slot of its rings many times, both softmax
    groups, the lazy rescale when the dominant key comes late in the loop) and the split-key decode kernel as a cluster
    of 8 and as 32 and more splits with the merge kernel.  The dominant key sits in the first tile, or at the last slot
    of a page in the middle of the context."""
    H, G, hd, ps = 5, 1, 128, 16
    rng = np.random.RandomState(n_keys // 1000 + len(far))
    kpos = 5 if far == "first tile" else (n_keys // 2 // ps) * ps + ps - 1
    # a portion of 300 queries at the end of the context (three tiles of the prefill kernel); the last query is spiked
    case = make_attention_case(rng, H, G, hd, ps, [n_keys], [300], torch.bfloat16, spike=(0, 299, kpos, H - 1))
    ref = attention_reference(case, 0)
    assert abs(ref[299, H - 1, 0] - 50.0) < 1.0
    out, plan = run_bf16_attention(case, H, G, hd, ps, 0, prefill_min=1)
    assert plan.n_tiles == 3 and plan.tile_rows == 128
    err = np.abs(out.float().cpu().numpy().reshape(ref.shape) - ref)
    assert err.max() <= 2.5 * 2 ** -8 * np.abs(ref).max(), np.unravel_index(err.argmax(), err.shape)
    # the last 16 of these queries token by token through the decode kernel: the splits of a token as a cluster of 8,
    # and through scratch memory and the merge kernel with 32 splits and more
    dec = dict(case, q=case["q"][-16:].contiguous(), pos=case["pos"][-16:].contiguous(), req=case["req"][-16:].contiguous(), q_lens=[16])
    for kwargs, cluster in ((dict(prefill_min=10 ** 6, target=8 * 16), True), (dict(prefill_min=10 ** 6, target=64 * 16), False),
                            (dict(prefill_min=10 ** 6, split=128), False)):
        out, plan = run_bf16_attention(dec, H, G, hd, ps, 0, **kwargs)
        assert plan.n_items == 16 and plan.cluster == cluster and (plan.max_splits == 8 if cluster else plan.max_splits >= 32)
        err = np.abs(out.float().cpu().numpy().reshape(16, H, hd) - ref[-16:])
        assert err.max() <= 2.5 * 2 ** -8 * np.abs(ref).max(), (kwargs, np.unravel_index(err.argmax(), err.shape))
    # one token alone over the whole context: the schedule of a decode step at batch 1
    single = make_attention_case(rng, H, G, hd, ps, [n_keys], [1], torch.bfloat16, spike=(0, 0, kpos, 2))
    ref1 = attention_reference(single, 0)
    out, plan = run_bf16_attention(single, H, G, hd, ps, 0)
    assert plan.max_splits >= 64 and not plan.cluster
    assert np.abs(out.float().cpu().numpy().reshape(ref1.shape) - ref1).max() <= 2.5 * 2 ** -8 * np.abs(ref1).max()


def test_attention_window_edge_is_exact():
    """A dominant key exactly one place outside the window must not be seen; one place inside must."""
    H, G, hd, ps, W = 4, 2, 64, 16, 48
    for inside in (True, False):
        rng = np.random.RandomState(7)
        n = 200
        kpos = n - W if inside else n - W - 1
        case = make_attention_case(rng, H, G, hd, ps, [n], [1], torch.bfloat16, spike=(0, 0, kpos, 1))
        ref = attention_reference(case, W)
        assert (abs(ref[0, 1, 0] - 50.0) < 1.0) == inside
        for kwargs in (dict(), dict(prefill_min=1)):
            out, _ = run_bf16_attention(case, H, G, hd, ps, W, **kwargs)
            assert np.abs(out.float().cpu().numpy().reshape(ref.shape) - ref).max() <= 2.5 * 2 ** -8 * np.abs(ref).max()
        out = torch.empty_like(case["q"])
        ops().attention_generic(case["q"], case["kp"], case["vp"], out, case["pos"], case["req"], case["table"], ps, H, G,
                                hd, W, 1.0 / np.sqrt(hd))
        assert np.abs(out.float().cpu().numpy().reshape(ref.shape) - ref).max() <= 2 ** -8 * np.abs(ref).max()


def test_attention_kernels_refuse_what_they_are_not_built_for():
    from mimirmind_b200.kernels import attention_bf16 as ab
    from mimirmind_b200.kernels.lib import KernelError
    assert not ab.supports(48, 6, 3) and not ab.supports(128, 34, 2) and ab.supports(128, 28, 4)
    q = torch.zeros((1, 3 * 528), device=DEV)
    kp = torch.zeros((1, 3, 16, 528), device=DEV)
    i32 = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="512"):
        ops().attention_generic(q, kp, kp, torch.empty_like(q), i32, i32, i32.view(1, 1), 16, 3, 3, 528, 0, 1.0)


# ---- sampling ----------------------------------------------------------------------------------------
def test_argmax_lowest_index_on_ties():
    V = 152064 + 3
    logits = torch.randn((5, V), device=DEV)
    logits[0, 777] = logits[0, 99999] = 50.0
    logits[1, V - 1] = 60.0
    logits[2, 0] = 60.0
    got = ops().argmax_rows(logits).cpu().tolist()
    assert got[:3] == [777, V - 1, 0]
    assert got[3:] == logits[3:].argmax(-1).cpu().tolist()


@pytest.mark.parametrize("V,R", [(1003, 64), (152064, 6), (50000, 40), (9001, 150)])
def test_sample_matches_the_plain_sampler(V, R):
    """One CTA per row for narrow rows; clusters of 2, 4 or 8 CTAs per row, with or without the slice kept in shared
    memory, for wide ones.  Ties at the top, among the kept candidates and across the slices of a cluster."""
    rng = np.random.RandomState(V % 1000)
    logits = (rng.randn(R, V) * 3).astype(np.float32)
    logits[5, 10] = logits[5, 20] = logits[5].max() + 1        # a tie at the top
    logits[4, V - 3] = logits[4, 7] = logits[4, V // 2] = np.sort(logits[4])[-3]   # equal logits far apart among the best
    logits[3, :] = np.round(logits[3, :])                      # many ties everywhere
    temps = rng.choice([0.0, 0.7, 1.0, 1.5], size=R).astype(np.float32)
    ks = rng.choice([0, 1, 5, 50], size=R).astype(np.int32)
    ps_ = rng.choice([1.0, 0.9, 0.5, 0.1], size=R).astype(np.float32)
    temps[3:6], ks[3:6], ps_[3:6] = [1.0, 0.7, 1.5], [0, 50, 5], [0.9, 1.0, 0.5]
    seeds = rng.randint(1, 2 ** 31, size=R).astype(np.int64)
    counters = rng.randint(0, 1000, size=R).astype(np.int64)
    got = ops().sample_rows(t(logits), t(temps), t(ks, torch.int32), t(ps_), t(seeds, torch.int64), t(counters, torch.int64)).cpu().tolist()
    for r in range(R):
        u = plain.uniform_from(int(seeds[r]), int(counters[r]))
        assert abs(u - ops().uniform_from(int(seeds[r]), int(counters[r]))) == 0
        want = plain.sample(logits[r].astype(np.float64), float(temps[r]), int(ks[r]), float(ps_[r]), u)
        assert got[r] == want, (r, temps[r], ks[r], ps_[r])


def test_sample_distribution_and_batch_independence():
    V = 37
    logits = np.linspace(-2, 2, V).astype(np.float32)
    R = 4096
    rows = t(np.tile(logits, (R, 1)))
    one = lambda v, dt: torch.full((R,), v, dtype=dt, device=DEV)
    cnt = torch.arange(R, dtype=torch.int64, device=DEV)
    got = ops().sample_rows(rows, one(1.0, torch.float32), one(0, torch.int32), one(1.0, torch.float32), one(99, torch.int64), cnt).cpu().numpy()
    p = np.exp(logits - logits.max()); p /= p.sum()
    freq = np.bincount(got, minlength=V) / R
    assert np.abs(freq - p).max() < 0.02
    # the same (seed, counter) gives the same token whatever else is in the batch
    alone = ops().sample_rows(rows[100:101].contiguous(), one(1.0, torch.float32)[:1], one(0, torch.int32)[:1],
                              one(1.0, torch.float32)[:1], one(99, torch.int64)[:1], cnt[100:101].contiguous()).item()
    assert alone == got[100]


def test_penalties_and_softcap():
    V = 50
    base = np.linspace(-3, 3, V).astype(np.float32)
    logits = t(np.tile(base, (2, 1)))
    recent = torch.tensor([[49, 49, 3, -1], [-1, -1, -1, -1]], dtype=torch.int32, device=DEV)
    f = lambda a: torch.tensor(a, dtype=torch.float32, device=DEV)
    ops().apply_penalties(logits, recent, f([2.0, 1.0]), f([0.5, 0.0]), f([0.25, 0.0]), f([0.0, 2.0]))
    got = logits.cpu().numpy()
    want0 = base.copy()
    want0[49] = base[49] / 2.0 - 0.5 * 2 - 0.25            # positive logit: divided
    want0[3] = base[3] * 2.0 - 0.5 * 1 - 0.25              # negative logit: multiplied
    assert np.allclose(got[0], want0, atol=1e-6)
    assert np.allclose(got[1], 2.0 * np.tanh(base / 2.0), atol=1e-6)


# ---- weight-streaming products for a handful of rows ----------------------------------------------
@pytest.mark.parametrize("M", [1, 3, 8])
# weight rows that give every arrangement of the dispatcher: 1, 1, 1, 1, 4, 2 and 8 row tiles per CTA
@pytest.mark.parametrize("N,K", [(4608, 3584), (3584, 18944), (160, 256), (1008, 96 * 32), (152064 // 8, 3584), (7168, 512), (37888, 256)])
def test_gemv_bf16(M, N, K):
    rng = np.random.RandomState(M + N + K)
    x, w, b = t(rng.randn(M, K), torch.bfloat16), t(rng.randn(N, K) * 0.05, torch.bfloat16), t(rng.randn(N), torch.bfloat16)
    ref = x.double().cpu().numpy() @ w.double().cpu().numpy().T + b.double().cpu().numpy()
    got32 = ops().gemv_bf16(x, w, b, torch.float32).cpu().numpy()
    assert np.abs(got32 - ref).max() <= 3e-6 * np.sqrt(K) * np.abs(ref).max() + 1e-5
    got16 = ops().gemv_bf16(x, w, b, torch.bfloat16).float().cpu().numpy()
    assert np.abs(got16 - ref).max() <= 2 ** -8 * np.abs(ref).max()
    nob = ops().gemv_bf16(x, w, None, torch.float32).cpu().numpy()
    assert np.abs(nob - (ref - b.double().cpu().numpy())).max() <= 3e-6 * np.sqrt(K) * np.abs(ref).max() + 1e-5
    # a row's result does not depend on the other rows of the batch
    alone = ops().gemv_bf16(x[M - 1:M].contiguous(), w, b, torch.float32).cpu().numpy()
    assert np.array_equal(alone[0], got32[M - 1])


@pytest.mark.parametrize("M,F,K", [(1, 18944, 3584), (8, 352, 256), (5, 1000, 512)])
def test_gemv_swiglu_epilogue_and_interleaved_silu(M, F, K):
    rng = np.random.RandomState(F)
    gate, up = rng.randn(F, K) * 0.05, rng.randn(F, K) * 0.05
    x = t(rng.randn(M, K), torch.bfloat16)
    gate_t, up_t = t(gate, torch.bfloat16), t(up, torch.bfloat16)
    w = torch.stack([gate_t.view(F // 8, 8, K), up_t.view(F // 8, 8, K)], dim=1).reshape(2 * F, K).contiguous()
    g = x.double().cpu().numpy() @ gate_t.double().cpu().numpy().T
    u = x.double().cpu().numpy() @ up_t.double().cpu().numpy().T
    ref = g / (1 + np.exp(-g)) * u
    got = ops().gemv_bf16(x, w, None, torch.bfloat16, swiglu=True).float().cpu().numpy()
    assert got.shape == (M, F)
    assert np.abs(got - ref).max() <= 2 ** -8 * np.abs(ref).max() + 1e-6
    # the unfused route over the same interleaved weight: product, then the activation kernel
    gu = ops().gemv_bf16(x, w, None, torch.bfloat16)
    act = torch.empty((M, F), dtype=torch.bfloat16, device=DEV)
    ops().silu_mul(gu, act, 8)
    assert np.abs(act.float().cpu().numpy() - ref).max() <= 3 * 2 ** -8 * np.abs(ref).max() + 1e-6


def test_gemv_refuses_unsupported_shapes():
    from mimirmind_b200.kernels.lib import KernelError
    big = ops().GEMV_MAX_ROWS + 1
    assert not ops().gemv_supported(big, 64, 256) and not ops().gemv_supported(4, 60, 256) and not ops().gemv_supported(4, 64, 100)
    assert ops().skinny_supported(big, 64, 256) and not ops().skinny_supported(ops().SKINNY_MAX_ROWS + 1, 64, 256) and not ops().skinny_supported(big, 60, 256)
    assert not ops().skinny_supported(big, 64, 100) and not ops().small_batch_supported(200, 64, 256)
    with pytest.raises(KernelError):
        ops().gemv_bf16(torch.zeros((ops().SKINNY_MAX_ROWS + 1, 256), dtype=torch.bfloat16, device=DEV), torch.zeros((64, 256), dtype=torch.bfloat16, device=DEV), None, torch.float32)
    with pytest.raises(KernelError):
        ops().gemv_bf16(torch.zeros((4, 100), dtype=torch.bfloat16, device=DEV), torch.zeros((64, 100), dtype=torch.bfloat16, device=DEV), None, torch.float32)


@pytest.mark.parametrize("M,rt,ks", [(12, 2, 4), (16, 1, 8), (7, 4, 2), (8, 8, 1)])
def test_gemv_all_layouts_of_the_kernel(M, rt, ks):
    """Row-tile / K-split arrangements and the two-tile (up to 16 rows) variant that the dispatcher
    does not pick by default."""
    from mimirmind_b200.kernels import lib
    rng = np.random.RandomState(M)
    N, K = 272, 1504
    x, w = t(rng.randn(M, K), torch.bfloat16), t(rng.randn(N, K) * 0.05, torch.bfloat16)
    out = torch.zeros((M, N), dtype=torch.float32, device=DEV)
    L = lib.load()
    rc = L.mm_gemv_bf16(w.data_ptr(), x.data_ptr(), None, 0, out.data_ptr(), 0, M, N, K, K, N, rt, ks, 0,
                        None, 0, 0, 0.0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.mm_last_error()
    ref = x.double().cpu().numpy() @ w.double().cpu().numpy().T
    assert np.abs(out.cpu().numpy() - ref).max() <= 3e-6 * np.sqrt(K) * np.abs(ref).max() + 1e-5


# ---- weight-streaming product with the decode-layer epilogues ----------------------------------------
def _row_scale(rng, M, tiles, dim, eps):
    """Partial sums of squares as a producer would leave them, and the 1/rms they stand for."""
    width = 16 if M <= ops().GEMV_MAX_ROWS else max(M, 16)     # the tcgen05 product takes any row stride >= M
    ss = np.abs(rng.randn(tiles, width)).astype(np.float32) * dim / tiles
    ss[:, M:] = np.nan                                  # rows that do not exist are never read into a result
    rstd = 1.0 / np.sqrt(ss[:, :M].astype(np.float64).sum(0) / dim + eps)
    return ops().RowScale(t(ss), dim, eps), rstd


@pytest.mark.parametrize("M,N,K", [(1, 48, 256), (5, 272, 1504), (8, 1040, 352), (13, 272, 1504), (16, 48, 256), (40, 1040, 352), (64, 4608, 3584), (50, 272, 200), (64, 400, 1504)])
def test_gemv_input_row_scale(M, N, K):
    rng = np.random.RandomState(M + N)
    x, w, b = t(rng.randn(M, K), torch.bfloat16), t(rng.randn(N, K) * 0.05, torch.bfloat16), t(rng.randn(N), torch.float32)
    scale, rstd = _row_scale(rng, M, 37, K, 1e-5)
    ref = (x.double().cpu().numpy() @ w.double().cpu().numpy().T) * rstd[:, None] + b.double().cpu().numpy()
    got = ops().gemv_bf16(x, w, b, torch.float32, scale=scale).cpu().numpy()
    assert np.abs(got - ref).max() <= 3e-6 * np.sqrt(K) * np.abs(ref).max() + 1e-5
    # the SwiGLU epilogue sees the scaled gate and up
    if N % 16 == 0 and (N // 2) % 8 == 0:
        F = N // 2
        gate, up = w[:F].float().cpu().numpy().astype(np.float64), w[F:].float().cpu().numpy().astype(np.float64)
        wi = torch.stack([w[:F].view(F // 8, 8, K), w[F:].view(F // 8, 8, K)], dim=1).reshape(N, K).contiguous()
        xs = x.double().cpu().numpy()
        g, u = (xs @ gate.T) * rstd[:, None], (xs @ up.T) * rstd[:, None]
        ref2 = g / (1.0 + np.exp(-g)) * u
        got2 = ops().gemv_bf16(x, wi, None, torch.float32, swiglu=True, scale=scale).cpu().numpy()
        assert np.abs(got2 - ref2).max() <= 1e-5 * np.sqrt(K) * np.abs(ref2).max() + 1e-5


@pytest.mark.parametrize("M,N,K,wdt", [(1, 256, 256, torch.float32), (6, 288, 1504, torch.bfloat16), (8, 1056, 352, torch.bfloat16),
                                       (13, 256, 256, torch.float32), (33, 288, 1504, torch.bfloat16), (64, 3584, 18944, torch.bfloat16),
                                       (57, 1056, 352, torch.bfloat16)])
def test_gemv_residual_epilogue(M, N, K, wdt):
    """residual += x W^T in fp32; rows of residual * norm weight; partial sums whose total is the row's sum of squares."""
    rng = np.random.RandomState(N)
    x, w = t(rng.randn(M, K), torch.bfloat16), t(rng.randn(N, K) * 0.05, torch.bfloat16)
    res0 = rng.randn(M, N).astype(np.float32) * 3
    nw = t(1.0 + 0.3 * rng.randn(N), wdt)
    scale_in, rstd_in = _row_scale(rng, M, 11, K, 1e-6)
    for sc, factor in ((None, np.ones(M)), (scale_in, rstd_in)):
        residual = t(res0)
        made = ops().gemv_bf16_residual(x, w, residual, nw, 1e-5, scale=sc)
        ref = res0.astype(np.float64) + (x.double().cpu().numpy() @ w.double().cpu().numpy().T) * factor[:, None]
        got = residual.cpu().numpy()
        assert np.abs(got - ref).max() <= 3e-6 * np.sqrt(K) * np.abs(ref).max() + 1e-5
        xw, rs = made
        assert rs.dim == N and rs.eps == 1e-5 and rs.ss.shape[0] == N // 16 and rs.ss.shape[1] >= min(M, 16)
        ref_xw = bf16_round(got.astype(np.float64) * nw.double().cpu().numpy())
        assert np.abs(xw.float().cpu().numpy() - ref_xw).max() <= 2 ** -8 * np.abs(ref_xw).max()
        ss = rs.ss.cpu().numpy()[:, :M].astype(np.float64).sum(0)
        assert np.abs(ss - (got.astype(np.float64) ** 2).sum(1)).max() <= 1e-5 * ss.max()
        # the factored rows, consumed by a product with the row scale, equal RMSNorm followed by the product
        w2 = t(rng.randn(32, N) * 0.05, torch.bfloat16)
        y = ops().gemv_bf16(xw, w2, None, torch.float32, scale=rs).cpu().numpy()
        normed = plain.rms_norm(got.astype(np.float64), nw.double().cpu().numpy(), 1e-5)
        ref_y = normed @ w2.double().cpu().numpy().T
        assert np.abs(y - ref_y).max() <= 2 ** -7 * np.abs(ref_y).max()
    # without a norm weight only the residual is written
    residual = t(res0)
    assert ops().gemv_bf16_residual(x, w, residual, None) is None
    ref = res0.astype(np.float64) + x.double().cpu().numpy() @ w.double().cpu().numpy().T
    assert np.abs(residual.cpu().numpy() - ref).max() <= 3e-6 * np.sqrt(K) * np.abs(ref).max() + 1e-5


@pytest.mark.parametrize("H,G,hd,ps,K,M", [(4, 2, 16, 16, 256, 3), (6, 3, 48, 8, 288, 8), (7, 1, 128, 16, 352, 5), (2, 2, 80, 32, 320, 1),
                                           (4, 2, 16, 16, 256, 14), (6, 3, 48, 8, 288, 40), (28, 4, 128, 16, 3584, 64), (2, 2, 80, 32, 320, 50)])
@pytest.mark.parametrize("with_scale", [False, True])
def test_gemv_qkv_rope_epilogue_and_interleaved_rope_kernel(H, G, hd, ps, K, M, with_scale):
    """The fused decode projection (interleaved weight rows, bias, rotation, cache write) against the formulas, and
    the stand-alone rotary kernel reading the same interleaved columns."""
    rng = np.random.RandomState(H * hd + M)
    theta = 1e4
    lens_before = [[0, 37, 130, 5, 64, 15, 16, 900][i % 8] + (i // 8) * 3 for i in range(M)]
    table, pages = paged_layout(rng, [a + 1 for a in lens_before], ps)
    pos = np.asarray(lens_before, dtype=np.int32)
    req = np.arange(M, dtype=np.int32)
    width = (H + 2 * G) * hd
    x = t(rng.randn(M, K), torch.bfloat16)
    w = t(rng.randn(width, K) * 0.1, torch.bfloat16)
    bias = t(rng.randn(width) * 0.5, torch.bfloat16)
    wi, bi = ops().interleave_halves(w, H + G, hd), ops().interleave_halves(bias, H + G, hd)
    assert wi.shape == w.shape and torch.equal(wi[(H + G) * hd:], w[(H + G) * hd:])
    assert torch.equal(wi[8:16], w[hd // 2:hd // 2 + 8]) and torch.equal(wi[0:8], w[0:8])
    scale, rstd = _row_scale(rng, M, 9, K, 1e-6) if with_scale else (None, np.ones(M))
    kp = torch.full((pages, G, ps, hd), 768.0, dtype=torch.bfloat16, device=DEV)
    vp = torch.full((pages, G, ps, hd), 768.0, dtype=torch.bfloat16, device=DEV)
    q_out = torch.empty((M, H * hd), dtype=torch.bfloat16, device=DEV)
    pos_d, req_d, table_d = t(pos, torch.int32), t(req, torch.int32), t(table, torch.int32)
    angles = ops().rope_table(pos_d, hd, theta)
    inv = theta ** (-np.arange(0, hd, 2, dtype=np.float64) / hd)
    ang_ref = pos[:, None].astype(np.float64) * inv[None, :]
    assert np.abs(angles.cpu().numpy() - np.concatenate([np.cos(ang_ref), np.sin(ang_ref)], axis=1)).max() <= 3e-6 * max(1.0, pos.max() / 50)
    slots = ops().slot_mapping(pos_d, req_d, table_d, ps)
    assert slots.cpu().numpy().tolist() == [int(table[req[i], pos[i] // ps]) * ps + int(pos[i]) % ps for i in range(M)]
    ops().gemv_bf16_qkv_rope(x, wi, bi, q_out, kp, vp, angles, slots, ps, H, G, hd, scale=scale)
    y = (x.double().cpu().numpy() @ w.double().cpu().numpy().T) * rstd[:, None] + bias.double().cpu().numpy()
    q_ref = plain.rope(y[:, :H * hd].reshape(M, H, hd), pos, theta)
    k_ref = plain.rope(y[:, H * hd:(H + G) * hd].reshape(M, G, hd), pos, theta)
    v_ref = y[:, (H + G) * hd:].reshape(M, G, hd)
    tol = 2 ** -8
    assert np.abs(q_out.float().cpu().numpy().reshape(M, H, hd) - q_ref).max() <= tol * np.abs(q_ref).max()
    kp_h, vp_h = kp.float().cpu().numpy(), vp.float().cpu().numpy()
    written = np.zeros((pages, ps), dtype=bool)
    for i in range(M):
        page, slot = table[req[i], pos[i] // ps], pos[i] % ps
        written[page, slot] = True
        assert np.abs(kp_h[page, :, slot] - k_ref[i]).max() <= tol * np.abs(k_ref).max()
        assert np.abs(vp_h[page, :, slot] - v_ref[i]).max() <= tol * np.abs(v_ref).max()
    untouched = ~written[:, None, :].repeat(G, axis=1)
    assert (kp_h[untouched] == 768.0).all() and (vp_h[untouched] == 768.0).all()
    # no cache to write (a layer that reads another layer's cache): q only
    q2 = torch.empty_like(q_out)
    ops().gemv_bf16_qkv_rope(x, wi, bi, q2, None, None, angles, None, ps, H, G, hd, scale=scale)
    assert torch.equal(q2, q_out)
    if not with_scale:
        # the stand-alone kernel on the interleaved product gives what it gives on the natural one
        prod = ops().gemv_bf16(x, w, None, torch.bfloat16)
        prod_i = ops().gemv_bf16(x, wi, None, torch.bfloat16)
        outs = []
        for p_, b_, il in ((prod, bias, False), (prod_i, bi, True)):
            kq = torch.zeros((pages, G, ps, hd), dtype=torch.bfloat16, device=DEV)
            vq = torch.zeros_like(kq)
            qq = torch.empty_like(q_out)
            ops().qkv_rope_kvwrite(p_, b_, qq, kq, vq, t(pos, torch.int32), t(req, torch.int32), t(table, torch.int32),
                                   ps, H, G, hd, hd, theta, interleave=il)
            outs.append((qq, kq, vq))
        for a_, b_ in zip(outs[0], outs[1]):
            assert torch.equal(a_, b_)


# ---- tcgen05 / TMA / TMEM matrix product -------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1, 8, 64), (200, 520, 192), (300, 264, 1000), (1100, 1048, 328)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("pair", [False, True])
def test_gemm_tcgen05(M, N, K, out_dtype, pair):
    """Both kernels: one CTA per 128 x 256 tile, and a pair of CTAs (cta_group::2) per 256 x 256 tile."""
    rng = np.random.RandomState(M + N + K)
    x, w, b = t(rng.randn(M, K), torch.bfloat16), t(rng.randn(N, K) * 0.05, torch.bfloat16), t(rng.randn(N), torch.float32)
    ref = x.double().cpu().numpy() @ w.double().cpu().numpy().T
    for bias in (None, b):
        want = ref + (b.double().cpu().numpy() if bias is not None else 0.0)
        got = ops().gemm_tcgen05(x, w, bias, out_dtype, pair=pair).float().cpu().numpy()
        ops().check_tcgen05_errors(x.device)
        tol = 3e-6 * np.sqrt(K) if out_dtype == torch.float32 else 2 ** -8
        assert np.abs(got - want).max() <= tol * np.abs(want).max() + 1e-5


def test_gemm_tcgen05_pair_many_tiles_per_pair():
    """More tiles than CTA pairs and more k-blocks than stages: both accumulators and every ring slot are reused,
    and the result equals the single-CTA kernel's bit for bit (same products, same order along K)."""
    rng = np.random.RandomState(5)
    M, N, K = 1300, 20 * 256 + 72, 1544
    x, w = t(rng.randn(M, K), torch.bfloat16), t(rng.randn(N, K) * 0.05, torch.bfloat16)
    one = ops().gemm_tcgen05(x, w, None, torch.float32, pair=False)
    two = ops().gemm_tcgen05(x, w, None, torch.float32, pair=True)
    ops().check_tcgen05_errors(x.device)
    assert torch.equal(one, two)
    ref = x.double().cpu().numpy() @ w.double().cpu().numpy().T
    assert np.abs(two.cpu().numpy() - ref).max() <= 3e-6 * np.sqrt(K) * np.abs(ref).max() + 1e-5


@pytest.mark.parametrize("M,F,K", [(130, 352, 256), (1030, 1000, 512), (64, 72, 64)])
@pytest.mark.parametrize("pair", [False, True])
def test_gemm_tcgen05_swiglu_epilogue(M, F, K, pair):
    rng = np.random.RandomState(F + M)
    x = t(rng.randn(M, K), torch.bfloat16)
    gate_t, up_t = t(rng.randn(F, K) * 0.05, torch.bfloat16), t(rng.randn(F, K) * 0.05, torch.bfloat16)
    w = torch.stack([gate_t.view(F // 8, 8, K), up_t.view(F // 8, 8, K)], dim=1).reshape(2 * F, K).contiguous()
    g = x.double().cpu().numpy() @ gate_t.double().cpu().numpy().T
    u = x.double().cpu().numpy() @ up_t.double().cpu().numpy().T
    ref = g / (1 + np.exp(-g)) * u
    got = ops().gemm_tcgen05(x, w, None, torch.bfloat16, swiglu=True, pair=pair).float().cpu().numpy()
    ops().check_tcgen05_errors(x.device)
    assert got.shape == (M, F)
    assert np.abs(got - ref).max() <= 2 ** -8 * np.abs(ref).max() + 1e-6


def test_gemm_tcgen05_refuses_unaligned_shapes():
    from mimirmind_b200.kernels.lib import KernelError
    z = lambda *s: torch.zeros(s, dtype=torch.bfloat16, device=DEV)
    assert not ops().gemm_tcgen05_supported(4, 64, 60) and not ops().gemm_tcgen05_supported(4, 63, 64)
    with pytest.raises(KernelError):
        ops().gemm_tcgen05(z(4, 60), z(64, 60), None, torch.bfloat16)
    with pytest.raises(KernelError, match="SwiGLU"):
        ops().gemm_tcgen05(z(4, 64), z(24, 64), None, torch.bfloat16, swiglu=True)


@pytest.mark.parametrize("M", [8, 24])
def test_gemv_builds_and_dependent_launches_give_the_same_bits(M):
    """The weight-streaming kernel exists for two and for three resident blocks per SM, and launches of the first build
    that follow each other are dependent launches: a kernel's blocks start while the one before it still runs, request
    their first weights and wait for it to finish before they read what it wrote.  A layer's four products, each reading
    the one before it, forty times over with nothing in between: the same bits from both builds, with and without
    dependent launches, eager and as a replayed graph.  The tcgen05 product of 9..64 rows launches dependently behind
    another of its kind in the same way (its residency is capped by shared memory)."""
    from mimirmind_b200.kernels import lib
    L = lib.load()
    rng = np.random.RandomState(17)
    d, F, H, G, hd, ps = 1024, 2816, 8, 2, 64, 16        # 8 rows: the register-streaming kernel; 24 rows: the tcgen05 one
    x = t(rng.randn(M, H * hd), torch.bfloat16)
    wo, wd = t(rng.randn(d, H * hd) * 0.05, torch.bfloat16), t(rng.randn(d, F) * 0.03, torch.bfloat16)
    wg, wu = t(rng.randn(F, d) * 0.05, torch.bfloat16), t(rng.randn(F, d) * 0.05, torch.bfloat16)
    wgu = torch.stack([wg.view(F // 8, 8, d), wu.view(F // 8, 8, d)], dim=1).reshape(2 * F, d).contiguous()
    wqkv = ops().interleave_halves(t(rng.randn((H + 2 * G) * hd, d) * 0.1, torch.bfloat16), H + G, hd)
    bqkv = ops().interleave_halves(t(rng.randn((H + 2 * G) * hd) * 0.5, torch.bfloat16), H + G, hd)
    nw = t(1.0 + 0.3 * rng.randn(d), torch.bfloat16)
    res0 = t(rng.randn(M, d) * 3)
    pos = t(np.arange(M) + 5, torch.int32)
    table = ops().rope_table(pos, hd, 1e4)
    slots = ops().slot_mapping(pos, t(np.arange(M), torch.int32), t(np.arange(M * 2).reshape(M, 2), torch.int32), ps)

    def layer(res, kp, vp, q):
        for _ in range(10):                                         # ten layers' worth of the same weights: every product reads the last
            xw1, rs1 = ops().gemv_bf16_residual(x, wo, res, nw, 1e-6)
            act = ops().gemv_bf16(xw1, wgu, None, torch.bfloat16, swiglu=True, scale=rs1)
            xw2, rs2 = ops().gemv_bf16_residual(act, wd, res, nw, 1e-6)
            ops().gemv_bf16_qkv_rope(xw2, wqkv, bqkv, q, kp, vp, table, slots, ps, H, G, hd, scale=rs2)
        return xw2

    def run(blocks, dependent, graph):
        old_b, old_p = L.mm_set_gemv_blocks(blocks), L.mm_get_pdl()
        L.mm_set_pdl(dependent)
        try:
            res = res0.clone()
            kp = torch.zeros((M * 2, G, ps, hd), dtype=torch.bfloat16, device=DEV)
            vp, q = torch.zeros_like(kp), torch.zeros((M, H * hd), dtype=torch.bfloat16, device=DEV)
            if not graph:
                for _ in range(4):
                    xw2 = layer(res, kp, vp, q)
            else:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    layer(res, kp, vp, q)                           # warm-up outside the capture
                    g = torch.cuda.CUDAGraph()
                    res.copy_(res0)
                    with torch.cuda.graph(g, stream=side):
                        xw2 = layer(res, kp, vp, q)
                torch.cuda.current_stream().wait_stream(side)
                res.copy_(res0)
                for _ in range(4):
                    g.replay()
            torch.cuda.synchronize()
            return res.clone(), q.clone(), kp.clone(), vp.clone(), xw2.clone()
        finally:
            L.mm_set_gemv_blocks(old_b)
            L.mm_set_pdl(old_p)

    want = run(3, 0, False)
    assert torch.isfinite(want[0]).all()
    for blocks, dependent, graph in ((2, 0, False), (2, 1, False), (0, 1, False), (2, 1, True), (0, 1, True), (3, 0, True)):
        got = run(blocks, dependent, graph)
        for a_, b_ in zip(got, want):
            assert torch.equal(a_, b_), (blocks, dependent, graph)
