"""The entry point that allocates nothing, called through its exported C symbol.

Some callers of the decode attention cannot allocate device memory (a host loop that forbids
cudaMalloc, a plugin that gets only the tensors it declared, a binding without an allocator), so they
cannot supply the scratch buffers that ``mm_attention_decode_bf16`` wants for its key splits.
``mm_attention_decode_bf16_no_alloc`` keeps that scratch inside the library.  This test calls it
through ctypes exactly as such a caller would, several times in a row on different inputs (the scratch
is shared and keeps the previous call's contents), and checks each result against the ordinary entry
point's on the same inputs, and against the plain implementation; it also checks that a request beyond
the built-in scratch is refused with a message instead of running.  It is collected last so that a run that stops at the first failure has
already run every other test.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 4 * 1024 * 1024


def make_case(seed, n_items, H, G, hd, ps, max_len):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    pages_per = (max_len + ps - 1) // ps
    pages = n_items * pages_per
    kp, vp = rnd(pages, G, ps, hd), rnd(pages, G, ps, hd)
    q = rnd(n_items, H * hd)
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).to(torch.int32)
    table = perm.view(n_items, pages_per).contiguous().cuda()
    lens = torch.randint(max_len // 2, max_len, (n_items,), generator=torch.Generator().manual_seed(seed + 1))
    positions = (lens - 1).to(torch.int32).cuda()
    token_req = torch.arange(n_items, dtype=torch.int32, device="cuda")
    return q, kp, vp, table, positions, token_req


def plain_decode_reference(q, kp, vp, table, positions, H, G, hd, ps, window):
    """The plain implementation's attention (numpy float64, whole sequences) for the last token of every item."""
    import plain_qwen2 as plain
    out = np.zeros((q.shape[0], H, hd))
    qh, kh, vh, th = (x.float().cpu().numpy().astype(np.float64) if x.is_floating_point() else x.cpu().numpy() for x in (q, kp, vp, table))
    for i, last in enumerate(positions.cpu().numpy()):
        n = int(last) + 1
        pos = np.arange(n)
        k = kh[th[i, pos // ps], :, pos % ps, :]                    # [n, G, hd]
        v = vh[th[i, pos // ps], :, pos % ps, :]
        full = np.zeros((n, H, hd))
        full[-1] = qh[i].reshape(H, hd)
        out[i] = plain.attention(full, k, v, window)[-1]
    return out.reshape(q.shape[0], H * hd)


def test_no_alloc_entry_point_matches_the_ordinary_one_call_after_call():
    """Five calls in a row through the exported symbol, on inputs of different sizes (the third needs more scratch than any
    before it, so it reads places that hold an earlier call's leftovers, or nothing yet), with and without a window, and
    one without key splits (no scratch at all): each result equals the ordinary entry point's bit for bit (same kernels,
    same order of operations; only where the scratch lives differs), and one is checked against the plain implementation."""
    from mimirmind_b200.kernels import lib as kernel_lib
    lib = kernel_lib.load()
    P, I, F = c_void_p, c_int, c_float
    ordinary = lib.mm_attention_decode_bf16
    ordinary.argtypes = [P, P, P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, I, P]
    ordinary.restype = c_int
    no_alloc = lib.mm_attention_decode_bf16_no_alloc          # the exported C symbol, nothing in between
    no_alloc.argtypes = [P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, I, P]
    no_alloc.restype = c_int
    stream = torch.cuda.current_stream().cuda_stream
    H, G, hd, ps = 28, 4, 128, 16
    #        seed, items, longest context, split length (0: no splits), window
    calls = ((1, 6, 1500, 128, 0), (2, 9, 700, 128, 0), (3, 10, 1700, 128, 0), (4, 5, 900, 128, 300), (5, 7, 400, 0, 0))
    for call, (seed, n_items, max_len, split_len, window) in enumerate(calls):
        q, kp, vp, table, positions, token_req = make_case(seed, n_items, H, G, hd, ps, max_len)
        max_splits = (max_len + split_len - 1) // split_len if split_len else 1
        assert n_items * H * max_splits * (hd + 2) <= SCRATCH_FLOATS
        scale = 1.0 / float(np.sqrt(hd))
        want = torch.zeros_like(q)
        part_o = torch.empty((n_items, H, max_splits, hd), dtype=torch.float32, device="cuda")
        part_ml = torch.empty((n_items, H, max_splits, 2), dtype=torch.float32, device="cuda")
        rc = ordinary(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), want.data_ptr(), part_o.data_ptr(), part_ml.data_ptr(), None,
                      n_items, positions.data_ptr(), token_req.data_ptr(), table.data_ptr(), table.shape[1], ps, H, G, hd, window,
                      scale, split_len, max_splits, stream)
        assert rc == 0, lib.mm_last_error()
        got = torch.full_like(q, float("nan"))
        rc = no_alloc(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), got.data_ptr(), None, n_items, positions.data_ptr(),
                      token_req.data_ptr(), table.data_ptr(), table.shape[1], ps, H, G, hd, window, scale, split_len, max_splits, stream)
        assert rc == 0, lib.mm_last_error()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all(), f"call {call}"
        assert torch.equal(got, want), f"call {call}: differs from the ordinary entry point by {(got.float() - want.float()).abs().max().item()}"
        assert want.float().abs().max().item() > 0.01
        if call in (1, 3):
            # not only the path against itself: the plain implementation, to the tolerance of the attention tests
            ref = plain_decode_reference(q, kp, vp, table, positions, H, G, hd, ps, window)
            err = np.abs(got.float().cpu().numpy() - ref).max()
            assert err <= 2.5 * 2 ** -8 * np.abs(ref).max(), f"call {call}: {err} from the plain implementation"
    assert max(c[1] * H * ((c[2] + 127) // 128) for c in calls[:2]) < calls[2][1] * H * ((calls[2][2] + 127) // 128)   # the third was the largest


def test_no_alloc_entry_point_refuses_more_than_its_scratch_holds():
    from mimirmind_b200.kernels import lib as kernel_lib
    lib = kernel_lib.load()
    P, I, F = c_void_p, c_int, c_float
    no_alloc = lib.mm_attention_decode_bf16_no_alloc
    no_alloc.argtypes = [P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, I, P]
    no_alloc.restype = c_int
    H, hd, n_items, max_splits = 28, 128, 64, 32
    assert n_items * H * max_splits * (hd + 2) > SCRATCH_FLOATS
    dummy = torch.zeros(8, device="cuda")
    p = dummy.data_ptr()
    rc = no_alloc(p, p, p, p, None, n_items, p, p, p, 1, 16, H, 4, hd, 0, 1.0, 128, max_splits, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = lib.mm_last_error().decode()
    assert "scratch" in msg and str(SCRATCH_FLOATS) in msg
    torch.cuda.synchronize()
