"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some callers of the kernel library cannot allocate device memory when they need the
split-KV decode attention (a serving loop that may not synchronise, a process whose
memory belongs to someone else's pool, a plug-in in a host that forbids it).  For them
``vcb_attention_decode_mma_static`` merges the context splits through a fixed array
inside the library instead of scratch buffers from the caller.  This test loads the
shared object with ctypes and calls that symbol several times in a row on different
inputs: the array keeps each call's contents, which must not leak into the next, so a
small call comes first, then one that fills the array to its last row, then a small one
again.  Each result must equal the ordinary entry point's to the bit (the two run the
same kernel, and its merge adds the splits in a fixed order), and one call is also
compared with a float64 reference that shares nothing with either.  Calls beyond the
array's size and page sizes the kernel cannot copy are refused, and the note the kernel
leaves when a block table names a page that is not there can be read back.

The file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROWS_LIMIT, ERR_UNSUPPORTED, ERR_TOO_SMALL, STATUS_BAD_PAGE = 8192, 10002, 10003, 11


def _case(seed, n_req, nh, nkv, d, page, max_ctx):
    rng = np.random.default_rng(seed)
    ctx = rng.integers(1, max_ctx, size=n_req).astype(np.int32)
    ctx[0] = max_ctx - 1
    blocks = -(-max_ctx // page)
    n_pages = n_req * blocks + 2
    bt = rng.permutation(n_pages)[: n_req * blocks].reshape(n_req, blocks).astype(np.int32)
    g = torch.Generator(device="cuda").manual_seed(seed)
    cache = torch.randn((n_pages, 2, nkv, page * d), generator=g, device="cuda").to(torch.bfloat16)
    q = torch.randn((n_req, nh * d), generator=g, device="cuda").to(torch.bfloat16)
    q_start = torch.arange(n_req + 1, dtype=torch.int32, device="cuda")
    return q, cache, q_start, torch.from_numpy(ctx).cuda(), torch.from_numpy(bt).cuda()


def _float64_attention(q, cache, ctx, bt, nh, nkv, d, page, window):
    """Decode attention from the cache image itself, in float64 (rows located with helpers.kv_pos)."""
    from helpers import kv_pos
    qn = q.float().cpu().numpy().astype(np.float64).reshape(len(ctx), nh, d)
    cn, btn = cache.float().cpu().numpy().astype(np.float64), bt.cpu().numpy()
    out = np.zeros_like(qn)
    for r, c in enumerate(ctx.cpu().numpy()):
        lo = max(0, c + 1 - window) if window else 0
        for g in range(nkv):
            k = np.stack([cn[btn[r, p // page], 0, g][kv_pos(d, 2, p % page, page)] for p in range(lo, c + 1)])
            v = np.stack([cn[btn[r, p // page], 1, g][kv_pos(d, 2, p % page, page)] for p in range(lo, c + 1)])
            for h in range(g * (nh // nkv), (g + 1) * (nh // nkv)):
                s = k @ qn[r, h] / np.sqrt(np.float32(d))
                w = np.exp(s - s.max())
                out[r, h] = (w / w.sum()) @ v
    return out.reshape(len(ctx), nh * d)


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from vllm_cpp_b200.csrc import build, ops
    lib = ctypes.CDLL(build.build())
    fn = lib.vcb_attention_decode_mma_static
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, F, I, P]
    fn.restype = I
    status = lib.vcb_attention_decode_mma_static_status
    status.argtypes = [ctypes.POINTER(ctypes.c_int)]
    status.restype = I
    stream = torch.cuda.current_stream().cuda_stream

    def note():
        code = ctypes.c_int(-1)
        assert status(ctypes.byref(code)) == 0
        return code.value

    note()                                          # whatever an earlier user of the library left
    #        requests, heads, kv heads, head size, page, longest context, splits, window
    calls = [(3, 6, 2, 64, 32, 700, 4, 300),        # 72 rows of the array
             (32, 8, 2, 128, 16, 260, 32, 0),       # 32 * 8 * 32 = 8192 rows: up to the array's last row
             (5, 28, 4, 128, 16, 1500, 7, 0)]       # 980 rows, over what the large call left
    assert calls[1][0] * calls[1][1] * calls[1][6] == ROWS_LIMIT
    for seed, (n_req, nh, nkv, d, page, max_ctx, nsplit, window) in enumerate(calls):
        q, cache, q_start, ctx, bt = _case(seed, n_req, nh, nkv, d, page, max_ctx)
        scale = float(np.float32(1) / np.sqrt(np.float32(d)))
        want = torch.zeros_like(q)
        part_o = torch.empty(n_req * nh * nsplit * d, dtype=torch.float32, device="cuda")
        part_ml = torch.empty(n_req * nh * nsplit * 2, dtype=torch.float32, device="cuda")
        counters = torch.zeros(n_req * nkv, dtype=torch.int32, device="cuda")
        ops.attention_decode_mma(q, cache, want, q_start, ctx, bt, None, n_req, nsplit, part_o, part_ml, counters,
                                 num_heads=nh, num_kv_heads=nkv, head_dim=d, page_size=page, window=window,
                                 scale=scale)
        got = torch.zeros_like(q)
        rc = fn(q.data_ptr(), cache.data_ptr(), got.data_ptr(), q_start.data_ptr(), ctx.data_ptr(), bt.data_ptr(),
                bt.shape[1], None, n_req, nsplit, nh, nkv, d, page, window, scale, cache.shape[0], stream)
        assert rc == 0, f"call {seed}: return code {rc}"
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {seed}: differs from the ordinary entry point"
        assert note() == 0
        if seed == 0:
            ref = _float64_attention(q, cache, ctx, bt, nh, nkv, d, page, window)
            g = got.float().cpu().numpy()
            assert np.abs(g - ref).max() <= 1e-2 * np.abs(ref).max(), f"max |diff| {np.abs(g - ref).max():.3e}"

    # one split needs no scratch; too many rows are refused and nothing is launched
    q, cache, q_start, ctx, bt = _case(9, 2, 6, 2, 64, 16, 200)
    got = torch.zeros_like(q)
    assert fn(q.data_ptr(), cache.data_ptr(), got.data_ptr(), q_start.data_ptr(), ctx.data_ptr(), bt.data_ptr(),
              bt.shape[1], None, 2, 1, 6, 2, 64, 16, 0, 0.125, cache.shape[0], stream) == 0
    torch.cuda.synchronize()
    assert got.float().abs().sum().item() > 0
    # a page number outside the cache: read as page 0, and the kernel leaves a note
    bad = bt.clone()
    bad[1, 0] = -1
    assert fn(q.data_ptr(), cache.data_ptr(), got.data_ptr(), q_start.data_ptr(), ctx.data_ptr(), bad.data_ptr(),
              bad.shape[1], None, 2, 1, 6, 2, 64, 16, 0, 0.125, cache.shape[0], stream) == 0
    assert note() == STATUS_BAD_PAGE and note() == 0
    # pages of 4 slots cannot be copied as the kernel copies a tile: refused
    untouched = torch.zeros_like(q)
    assert fn(q.data_ptr(), cache.data_ptr(), untouched.data_ptr(), q_start.data_ptr(), ctx.data_ptr(), bt.data_ptr(),
              bt.shape[1], None, 2, 1, 6, 2, 64, 4, 0, 0.125, cache.shape[0], stream) == ERR_UNSUPPORTED
    # 44 requests x 6 heads x 32 splits = 8448 rows: more than the array holds
    q, cache, q_start, ctx, bt = _case(10, 44, 6, 2, 64, 16, 100)
    too_many = 32                                   # the most splits the kernel takes
    big = torch.zeros_like(q)
    assert fn(q.data_ptr(), cache.data_ptr(), big.data_ptr(), q_start.data_ptr(), ctx.data_ptr(), bt.data_ptr(),
              bt.shape[1], None, 44, too_many, 6, 2, 64, 16, 0, 0.125, cache.shape[0], stream) == ERR_TOO_SMALL
    torch.cuda.synchronize()
    assert not untouched.any() and not big.any()
