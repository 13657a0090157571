"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some callers of the kernel library cannot allocate device memory when they need the
split-KV decode attention (a serving loop that may not synchronise, a process whose
memory belongs to someone else's pool, a plug-in in a host that forbids it).  For them
``vcb_attention_decode_mma_static`` merges the context splits through a fixed array
inside the library instead of scratch buffers from the caller.  This test loads the
shared object with ctypes, calls that symbol twice in a row on different inputs (the
array keeps the first call's contents, which must not leak into the second), and checks
each result against the ordinary entry point within the kernel tests' bfloat16 tolerance.
It also checks that a call beyond the array's size is refused.

The file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROWS_LIMIT, ERR_TOO_SMALL = 8192, 10003


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


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from vllm_cpp_b200.csrc import build, ops
    lib = ctypes.CDLL(build.build())
    fn = lib.vcb_attention_decode_mma_static
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, F, P]
    fn.restype = I
    stream = torch.cuda.current_stream().cuda_stream

    for seed, (n_req, nh, nkv, d, page, max_ctx, nsplit, window) in enumerate(
            [(5, 28, 4, 128, 16, 1500, 7, 0), (3, 6, 2, 64, 32, 700, 4, 300)]):
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
                bt.shape[1], None, n_req, nsplit, nh, nkv, d, page, window, scale, stream)
        assert rc == 0, f"call {seed}: return code {rc}"
        torch.cuda.synchronize()
        g, w = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert np.isfinite(g).all()
        assert np.abs(g - w).max() <= 1e-2 * np.abs(w).max(), f"call {seed}: max |diff| {np.abs(g - w).max():.3e}"

    # one split needs no scratch; too many rows are refused and nothing is launched
    q, cache, q_start, ctx, bt = _case(9, 2, 6, 2, 64, 16, 200)
    got = torch.zeros_like(q)
    assert fn(q.data_ptr(), cache.data_ptr(), got.data_ptr(), q_start.data_ptr(), ctx.data_ptr(), bt.data_ptr(),
              bt.shape[1], None, 2, 1, 6, 2, 64, 16, 0, 0.125, stream) == 0
    torch.cuda.synchronize()
    assert got.float().abs().sum().item() > 0
    # 44 requests x 6 heads x 32 splits = 8448 rows: more than the array holds
    q, cache, q_start, ctx, bt = _case(10, 44, 6, 2, 64, 16, 100)
    untouched = torch.zeros_like(q)
    too_many = 32                                   # the most splits the kernel takes
    assert fn(q.data_ptr(), cache.data_ptr(), untouched.data_ptr(), q_start.data_ptr(), ctx.data_ptr(), bt.data_ptr(),
              bt.shape[1], None, 44, too_many, 6, 2, 64, 16, 0, 0.125, stream) == ERR_TOO_SMALL
    torch.cuda.synchronize()
    assert not untouched.any()
