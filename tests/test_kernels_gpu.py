"""Each kernel alone against a plain numpy reference, at sizes other than the engine's
tiny models: head sizes in steps of 16, odd head and group counts, widths and
vocabularies that are no power of two, ragged edges of every tile."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from helpers import kv_pos

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def as_stored(a, dtype):
    """float32 values as the device will hold them."""
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(DT[dtype]).float().numpy()


def close(got, want, dtype, what, scale=None):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    scale = np.abs(want).max() if scale is None else scale
    tol = 2e-6 if dtype == "float32" else 1e-2
    err = np.abs(got - want).max()
    assert err <= tol * scale, f"{what}: max |diff| {err:.3e} vs {tol} * {scale:.3e}"


@pytest.fixture(scope="module")
def ops():
    from vllm_cpp_b200.csrc import ops
    return ops


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [88, 77, 3584, 5120, 8200])
def test_embedding(ops, dtype, hidden):
    """Widths that take the 16-byte path with two and with four vectors a thread (bfloat16, a multiple of 8), and
    widths that do not."""
    rng = np.random.default_rng(0)
    table = as_stored(rng.standard_normal((301, hidden)), dtype)
    ids = rng.integers(0, 301, size=37).astype(np.int32)
    ids[0], ids[1] = 0, 300
    out = torch.full((37, hidden), float("nan"), dtype=torch.float32, device="cuda")
    ops.embedding(dev(table, DT[dtype]), dev(ids), out)
    assert np.array_equal(out.cpu().numpy(), plain.embedding(ids, table).astype(np.float32))


@pytest.mark.parametrize("dtype,hidden", [("float32", 88), ("bfloat16", 88), ("bfloat16", 77)])
def test_embedding_refuses_ids_outside_the_table(ops, dtype, hidden):
    """Ids that never passed the host (a step launched ahead feeds sampled ids on the device): one outside the
    table reads nothing, leaves a row of zeros and code 12 in the status word; the other rows are right."""
    rng = np.random.default_rng(1)
    table = as_stored(rng.standard_normal((50, hidden)), dtype)
    ids = np.array([3, -1, 49, 50, 1048575, 0], dtype=np.int32)
    out = torch.full((6, hidden), float("nan"), dtype=torch.float32, device="cuda")
    ops.check_status()
    ops.embedding(dev(table, DT[dtype]), dev(ids), out)
    with pytest.raises(ops.KernelError, match="token id outside the vocabulary"):
        ops.check_status()
    got = out.cpu().numpy()
    assert np.array_equal(got[[0, 2, 5]], table[[3, 49, 0]].astype(np.float32))
    assert not got[[1, 3, 4]].any()
    ops.check_status()                                  # cleared


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [48, 200, 3584, 5000, 16384, 20000])
def test_add_rmsnorm(ops, dtype, hidden):
    rng = np.random.default_rng(1)
    res = rng.standard_normal((9, hidden)).astype(np.float32)
    delta = as_stored(rng.standard_normal((9, hidden)), dtype)
    gain = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
    eps = 3e-5
    # with delta: residual += delta, out = norm
    r, out = dev(res), torch.empty((9, hidden), dtype=DT[dtype], device="cuda")
    ops.add_rmsnorm(r, dev(delta, DT[dtype]), dev(gain), out, eps)
    summed = res + delta
    close(r.cpu().numpy(), summed, "float32", "residual sum")
    close(out.float().cpu().numpy(), plain.rms_norm(summed.astype(np.float64), gain, eps), dtype, "norm")
    # without delta the residual is untouched
    r2 = dev(res)
    ops.add_rmsnorm(r2, None, dev(gain), out, eps)
    assert torch.equal(r2.cpu(), torch.from_numpy(res))
    close(out.float().cpu().numpy(), plain.rms_norm(res.astype(np.float64), gain, eps), dtype, "norm no delta")
    # gathered rows, one of them twice: nothing is written back
    rows = np.array([7, 0, 7, 3], dtype=np.int32)
    r3, out3 = dev(res), torch.empty((4, hidden), dtype=DT[dtype], device="cuda")
    ops.add_rmsnorm(r3, dev(delta, DT[dtype]), dev(gain), out3, eps, dev(rows))
    assert torch.equal(r3.cpu(), torch.from_numpy(res))
    close(out3.float().cpu().numpy(), plain.rms_norm(summed[rows].astype(np.float64), gain, eps), dtype, "gathered")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul_and_bias(ops, dtype):
    rng = np.random.default_rng(2)
    # a width the 16-byte kernel cannot take, one it takes (several vectors a thread, a ragged end),
    # values far out on both sides
    for tokens, inter in ((5, 333), (70, 1000), (3, 8)):
        gu = as_stored(3 * rng.standard_normal((tokens, 2 * inter)), dtype)
        gu[0, :4] = [-200.0, -30.0, 40.0, 0.0]
        out = torch.empty((tokens, inter), dtype=DT[dtype], device="cuda")
        ops.silu_mul(dev(gu, DT[dtype]), out)
        close(out.float().cpu().numpy(), plain.silu(gu[:, :inter].astype(np.float64)) * gu[:, inter:], dtype,
              f"silu_mul {tokens} x {inter}")
    x = as_stored(rng.standard_normal((4, 77)), dtype)
    b = rng.standard_normal(77).astype(np.float32)
    xd = dev(x, DT[dtype])
    ops.add_bias(xd, dev(b))
    close(xd.float().cpu().numpy(), x + b, dtype, "add_bias")


def paged_layout(rng, n_reqs, max_len, page, n_pages):
    """A random assignment of pages to requests: block tables [n_reqs, max_blocks]."""
    blocks = -(-max_len // page)
    assert n_reqs * blocks <= n_pages
    perm = rng.permutation(n_pages)[: n_reqs * blocks].reshape(n_reqs, blocks)
    return perm.astype(np.int32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,d,rot,pairing", [(4, 2, 16, 16, 0), (3, 1, 32, 32, 0), (7, 7, 48, 24, 0),
                                                   (2, 1, 128, 128, 0), (5, 5, 80, 80, 1), (6, 3, 64, 0, 0),
                                                   (28, 4, 128, 128, 0), (33, 3, 64, 64, 0), (9, 3, 16, 16, 0)])
def test_rope_cache_write(ops, dtype, nh, nkv, d, rot, pairing):
    rope_cache_write_case(ops, dtype, nh, nkv, d, rot, pairing, many=False)


@pytest.mark.parametrize("nh,nkv,d", [(28, 4, 128), (3, 1, 64), (5, 5, 16)])
def test_rope_cache_write_of_a_long_portion(ops, nh, nkv, d):
    """Hundreds of tokens in one call (the kernel then takes several tokens per CTA), a count that is no
    multiple of that number, two requests."""
    rope_cache_write_case(ops, "bfloat16", nh, nkv, d, d, 0, many=True)


def rope_cache_write_case(ops, dtype, nh, nkv, d, rot, pairing, many):
    rng = np.random.default_rng(3)
    page, n_reqs = 16, 2
    if many:
        n_pages = 48
        bt = paged_layout(rng, n_reqs, 384, page, n_pages)
        req = np.array([0] * 350 + [1] * 231, dtype=np.int32)
        pos = np.concatenate([np.arange(7, 357), np.arange(100, 331)]).astype(np.int32)
    else:
        n_pages = 12
        bt = paged_layout(rng, n_reqs, 80, page, n_pages)
        req = np.array([0] * 9 + [1] * 4, dtype=np.int32)
        pos = np.concatenate([np.arange(30, 39), np.arange(61, 65)]).astype(np.int32)     # crosses page edges
    n = len(pos)
    width = (nh + 2 * nkv) * d
    qkv = as_stored(rng.standard_normal((n, width)), dtype)
    bias = rng.standard_normal(width).astype(np.float32)
    theta = 10000.0
    denom = None
    if rot:
        j = np.arange(rot // 2, dtype=np.float32)
        denom = np.power(np.float32(theta), (np.float32(2) * j) / np.float32(rot)).astype(np.float32)
    cache = torch.zeros((n_pages, 2, nkv, page * d), dtype=DT[dtype], device="cuda")
    q_out = torch.empty((n, nh * d), dtype=DT[dtype], device="cuda")
    ops.rope_cache_write(dev(qkv, DT[dtype]), dev(bias), dev(pos), dev(req), dev(bt), None if denom is None else dev(denom),
                         q_out, cache, num_heads=nh, num_kv_heads=nkv, head_dim=d, rotary_dim=rot, pairing=pairing,
                         page_size=page, write_kv=True)
    x = (qkv.astype(np.float64) + bias).reshape(n, nh + 2 * nkv, d)

    def rotate(h):
        if not rot:
            return h
        if pairing == 0:
            return plain.rope(h, pos, theta, rot)
        ang = plain.rope_angles(pos, theta, rot).astype(np.float64)[:, None, :]
        out = h.copy()
        a, b = h[..., 0:rot:2], h[..., 1:rot:2]
        out[..., 0:rot:2] = a * np.cos(ang) - b * np.sin(ang)
        out[..., 1:rot:2] = a * np.sin(ang) + b * np.cos(ang)
        return out

    q_ref, k_ref, v_ref = rotate(x[:, :nh]), rotate(x[:, nh:nh + nkv]), x[:, nh + nkv:]
    close(q_out.float().cpu().numpy().reshape(n, nh, d), q_ref, dtype, "q")
    c = cache.float().cpu().numpy().reshape(n_pages, 2, nkv, page * d)        # blocks of page x d elements
    esize = 4 if dtype == "float32" else 2
    owned = np.zeros(c.shape, dtype=bool)
    for t in range(n):
        pg, slot = bt[req[t], pos[t] // page], pos[t] % page
        where = kv_pos(d, esize, slot, page)           # where the slot's elements lie in its block
        close(c[pg, 0][:, where], k_ref[t], dtype, f"k of token {t}", scale=np.abs(k_ref).max())
        close(c[pg, 1][:, where], v_ref[t], dtype, f"v of token {t}", scale=np.abs(v_ref).max())
        owned[pg][:, :, where] = True
    assert not c[~owned].any(), "a slot that no token owns was written"
    # write_kv off leaves the cache alone
    cache2 = torch.zeros_like(cache)
    ops.rope_cache_write(dev(qkv, DT[dtype]), dev(bias), dev(pos), dev(req), dev(bt), None if denom is None else dev(denom),
                         q_out, cache2, num_heads=nh, num_kv_heads=nkv, head_dim=d, rotary_dim=rot, pairing=pairing,
                         page_size=page, write_kv=False)
    assert not cache2.any()


def reference_attention(q, k, v, q_lens, ctx_lens, nh, nkv, window):
    """q: [n, nh, d] for all requests' new tokens; k, v: per request [len, nkv, d] (whole sequences)."""
    out = np.zeros_like(q)
    t0 = 0
    group = nh // nkv
    d = q.shape[-1]
    for r, (ql, cl) in enumerate(zip(q_lens, ctx_lens)):
        for i in range(ql):
            p = cl + i
            lo = max(0, p - window + 1) if window else 0
            for h in range(nh):
                s = (k[r][lo:p + 1, h // group] @ q[t0 + i, h]) / np.sqrt(np.float32(d))
                w = np.exp(s - s.max())
                out[t0 + i, h] = (w / w.sum()) @ v[r][lo:p + 1, h // group]
        t0 += ql
    return out


def attention_case(rng, dtype, nh, nkv, d, page, q_lens, ctx_lens, spike=True, window=0):
    """A batch for the attention kernels.  With a window, the pages that the cache manager would have given
    back by now (every key at or below ctx - window: no query of the step reads them) are gone from the
    table (-1), and what they held is overwritten with large values, as a page's next owner might leave
    it: a kernel that still reads them shows it in its output or in the status word."""
    n_reqs = len(q_lens)
    total = [c + q for c, q in zip(ctx_lens, q_lens)]
    n_pages = sum(-(-t // page) for t in total) + 3
    bt_rows = []
    perm = list(rng.permutation(n_pages))
    max_blocks = max(-(-t // page) for t in total) + 1
    bt = np.full((n_reqs, max_blocks), -1, dtype=np.int32)
    for r, t in enumerate(total):
        for b in range(-(-t // page)):
            bt[r, b] = perm.pop()
    k = [as_stored(rng.standard_normal((t, nkv, d)), dtype) for t in total]
    v = [as_stored(rng.standard_normal((t, nkv, d)), dtype) for t in total]
    n = sum(q_lens)
    q = as_stored(rng.standard_normal((n, nh, d)), dtype)
    if spike:
        # one far key per request gets a score that stands out: q of the last token points at key 1
        t0 = 0
        for r, ql in enumerate(q_lens):
            if total[r] > 3:
                k[r][1] = as_stored(k[r][1] * 3.0, dtype)
                q[t0 + ql - 1] = as_stored(np.repeat(k[r][1], nh // nkv, axis=0) * 0.7, dtype)
            t0 += ql
    cache = np.zeros((n_pages, 2, nkv, page * d), dtype=np.float32)
    esize = 4 if dtype == "float32" else 2
    for r, t in enumerate(total):
        for p in range(t):
            where = kv_pos(d, esize, p % page, page)
            cache[bt[r, p // page], 0][:, where] = k[r][p]
            cache[bt[r, p // page], 1][:, where] = v[r][p]
    if window > 0:
        for r, ctx in enumerate(ctx_lens):
            for b in range(max(0, (ctx - window + 1) // page)):
                cache[bt[r, b]] = 3.0e4
                bt[r, b] = -1
    q_start = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    pos = np.concatenate([np.arange(c, c + ql) for c, ql in zip(ctx_lens, q_lens)]).astype(np.int32)
    req = np.concatenate([np.full(ql, r) for r, ql in enumerate(q_lens)]).astype(np.int32)
    return dict(q=q, k=k, v=v, cache=cache, bt=bt, q_start=q_start, pos=pos, req=req, n=n)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,d,page,window", [(4, 2, 16, 16, 0), (3, 1, 32, 32, 0), (5, 5, 48, 16, 20),
                                                   (14, 2, 64, 16, 0), (2, 2, 256, 16, 0), (6, 3, 112, 48, 37)])
def test_attention_simt(ops, dtype, nh, nkv, d, page, window):
    rng = np.random.default_rng(4)
    q_lens, ctx_lens = [1, 33, 2, 1], [300, 17, 0, 63]
    c = attention_case(rng, dtype, nh, nkv, d, page, q_lens, ctx_lens, window=window)
    out = torch.empty((c["n"], nh * d), dtype=DT[dtype], device="cuda")
    ops.attention_simt(dev(c["q"].reshape(c["n"], -1), DT[dtype]), dev(c["cache"], DT[dtype]), out, dev(c["pos"]),
                       dev(c["req"]), dev(c["bt"]), num_heads=nh, num_kv_heads=nkv, head_dim=d, page_size=page,
                       window=window, scale=float(np.float32(1) / np.sqrt(np.float32(d))))
    ops.check_status()
    want = reference_attention(c["q"].astype(np.float64), c["k"], c["v"], q_lens, ctx_lens, nh, nkv, window)
    close(out.float().cpu().numpy().reshape(c["n"], nh, d), want, dtype, "attention_simt")


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("nh,nkv,page,window", [(28, 4, 16, 0), (8, 1, 16, 100), (40, 2, 64, 0), (3, 3, 32, 40), (16, 2, 16, 300)])
def test_attention_prefill_tc(ops, nh, nkv, page, window, d):
    """The tcgen05 prefill attention (head sizes 128 and 64) against the float64 reference: portions that
    start and end inside tiles and pages, contexts before them, one far key that must dominate, windows."""
    rng = np.random.default_rng(6)
    q_lens, ctx_lens = [70, 1, 2, 300, 5], [0, 500, 63, 64, 1000]
    c = attention_case(rng, "bfloat16", nh, nkv, d, page, q_lens, ctx_lens, window=window)
    group = nh // nkv
    rows = ops.TC_ATTENTION_TILE_ROWS
    tiles = [(r, k * rows) for r, ql in enumerate(q_lens) for k in range(-(-ql * group // rows))]
    out = torch.full((c["n"], nh * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    for _ in range(2):
        ops.attention_prefill_tc(dev(c["q"].reshape(c["n"], -1), torch.bfloat16), dev(c["cache"], torch.bfloat16), out,
                                 dev(c["q_start"]), dev(np.array(ctx_lens, dtype=np.int32)), dev(c["bt"]),
                                 dev(np.array([t[0] for t in tiles], dtype=np.int32)),
                                 dev(np.array([t[1] for t in tiles], dtype=np.int32)),
                                 num_heads=nh, num_kv_heads=nkv, head_dim=d, page_size=page, window=window,
                                 scale=float(np.float32(1) / np.sqrt(np.float32(d))))
    torch.cuda.synchronize()
    ops.check_status()
    want = reference_attention(c["q"].astype(np.float64), c["k"], c["v"], q_lens, ctx_lens, nh, nkv, window)
    close(out.float().cpu().numpy().reshape(c["n"], nh, d), want, "bfloat16", "attention_prefill_tc")


@pytest.mark.parametrize("d,window", [(128, 0), (64, 0), (128, 500)])
def test_attention_prefill_tc_long(ops, d, window):
    """Long portions: CTAs that walk dozens of key tiles, more CTAs than the device holds at once, the
    warps of a CTA drifting apart.  (Two hazards between the kernel's barriers showed only at this size.)"""
    rng = np.random.default_rng(16)
    nh, nkv, page = 28, 4, 16
    q_lens, ctx_lens = [1700, 300], [0, 1100]
    if window:
        q_lens, ctx_lens = [1700, 300], [0, 2400]      # 150 pages before the second portion, most of them given back
    c = attention_case(rng, "bfloat16", nh, nkv, d, page, q_lens, ctx_lens, window=window)
    group = nh // nkv
    rows = ops.TC_ATTENTION_TILE_ROWS
    tiles = [(r, k * rows) for r, ql in enumerate(q_lens) for k in range(-(-ql * group // rows))]
    tiles.sort(key=lambda t: -(ctx_lens[t[0]] + t[1] // group))
    out = torch.full((c["n"], nh * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    args = (dev(c["q"].reshape(c["n"], -1), torch.bfloat16), dev(c["cache"], torch.bfloat16), out, dev(c["q_start"]),
            dev(np.array(ctx_lens, dtype=np.int32)), dev(c["bt"]), dev(np.array([t[0] for t in tiles], dtype=np.int32)),
            dev(np.array([t[1] for t in tiles], dtype=np.int32)))
    for _ in range(5):
        ops.attention_prefill_tc(*args, num_heads=nh, num_kv_heads=nkv, head_dim=d, page_size=page, window=window,
                                 scale=float(np.float32(1) / np.sqrt(np.float32(d))))
    torch.cuda.synchronize()
    ops.check_status()
    want = reference_attention(c["q"].astype(np.float64), c["k"], c["v"], q_lens, ctx_lens, nh, nkv, window)
    close(out.float().cpu().numpy().reshape(c["n"], nh, d), want, "bfloat16", "attention_prefill_tc, long")


@pytest.mark.parametrize("nsplit", [1, 3, 8])
@pytest.mark.parametrize("nh,nkv,d,page,window", [(28, 4, 128, 16, 0), (6, 2, 64, 32, 0), (3, 3, 64, 16, 40),
                                                   (40, 2, 128, 16, 0), (16, 1, 128, 16, 200), (8, 2, 128, 8, 0)])
def test_attention_decode_mma(ops, nsplit, nh, nkv, d, page, window):
    rng = np.random.default_rng(6)
    ctx_lens = [0, 1, 63, 64, 65, 777, 2000]
    if window:
        ctx_lens = [0, 1, 63, 64, 65, 777, 3000]       # 188 pages of 16, of which a window of 200 keeps 13
    q_lens = [1] * len(ctx_lens)
    c = attention_case(rng, "bfloat16", nh, nkv, d, page, q_lens, ctx_lens, window=window)
    n = c["n"]
    out = torch.zeros((n, nh * d), dtype=torch.bfloat16, device="cuda")
    part_o = torch.empty(n * nh * nsplit * d, dtype=torch.float32, device="cuda")
    part_ml = torch.empty(n * nh * nsplit * 2, dtype=torch.float32, device="cuda")
    counters = torch.zeros(n * nkv, dtype=torch.int32, device="cuda")
    ops.attention_decode_mma(dev(c["q"].reshape(n, -1), torch.bfloat16), dev(c["cache"], torch.bfloat16), out,
                             dev(c["q_start"]), dev(np.array(ctx_lens, dtype=np.int32)), dev(c["bt"]), None, n, nsplit,
                             part_o, part_ml, counters, num_heads=nh, num_kv_heads=nkv, head_dim=d, page_size=page,
                             window=window, scale=float(np.float32(1) / np.sqrt(np.float32(d))))
    ops.check_status()
    want = reference_attention(c["q"].astype(np.float64), c["k"], c["v"], q_lens, ctx_lens, nh, nkv, window)
    close(out.float().cpu().numpy().reshape(n, nh, d), want, "bfloat16", f"attention_decode_mma nsplit={nsplit}")
    # a request list picks and reorders requests
    sel = np.array([5, 2], dtype=np.int32)
    out2 = torch.zeros_like(out)
    ops.attention_decode_mma(dev(c["q"].reshape(n, -1), torch.bfloat16), dev(c["cache"], torch.bfloat16), out2,
                             dev(c["q_start"]), dev(np.array(ctx_lens, dtype=np.int32)), dev(c["bt"]), dev(sel), 2, nsplit,
                             part_o, part_ml, counters, num_heads=nh, num_kv_heads=nkv, head_dim=d, page_size=page,
                             window=window, scale=float(np.float32(1) / np.sqrt(np.float32(d))))
    got2 = out2.float().cpu().numpy().reshape(n, nh, d)
    close(got2[[5, 2]], want[[5, 2]], "bfloat16", "decode with a request list")
    assert not got2[[0, 1, 3, 4, 6]].any()
    # splits of a fixed number of tiles: the long contexts take several grid columns, the short ones one;
    # a number that would need more columns than the grid has falls back to equal parts
    for tiles_per_split in (1, 5, 11, 1000):
        out3 = torch.zeros_like(out)
        ops.attention_decode_mma(dev(c["q"].reshape(n, -1), torch.bfloat16), dev(c["cache"], torch.bfloat16), out3,
                                 dev(c["q_start"]), dev(np.array(ctx_lens, dtype=np.int32)), dev(c["bt"]), None, n, nsplit,
                                 part_o, part_ml, counters, num_heads=nh, num_kv_heads=nkv, head_dim=d, page_size=page,
                                 window=window, scale=float(np.float32(1) / np.sqrt(np.float32(d))),
                                 split_tiles=dev(np.array([tiles_per_split], dtype=np.int32)))
        close(out3.float().cpu().numpy().reshape(n, nh, d), want, "bfloat16",
              f"attention_decode_mma nsplit={nsplit}, {tiles_per_split} tiles a split")
        assert not counters.any()


def test_attention_refuses_what_it_cannot_do(ops):
    q = torch.zeros((1, 2 * 80), dtype=torch.bfloat16, device="cuda")
    z = torch.zeros(4, dtype=torch.int32, device="cuda")
    cache = torch.zeros((2, 2, 2, 16, 80), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="head sizes"):
        ops.attention_prefill_tc(q, cache, q, z, z, z.view(1, 4), z[:1], z[:1], num_heads=2, num_kv_heads=2,
                                  head_dim=80, page_size=16, window=0, scale=1.0)
    with pytest.raises(ops.KernelError, match="256"):
        ops.attention_simt(torch.zeros((1, 272), dtype=torch.float32, device="cuda"), cache.float(), q.float(), z[:1],
                           z[:1], z.view(1, 4), num_heads=1, num_kv_heads=1, head_dim=272, page_size=16, window=0, scale=1.0)


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (7, 130, 33), (64, 64, 16), (200, 301, 96), (3, 1000, 513)])
def test_gemm_f32_is_true_32_bit(ops, m, n, k):
    rng = np.random.default_rng(7)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((n, k)).astype(np.float32)
    # values with many mantissa bits: a product in TF32 or bfloat16 would miss by about 1e-3
    out = torch.empty((m, n), dtype=torch.float32, device="cuda")
    ops.gemm_f32(dev(a), dev(w), out)
    want = a.astype(np.float64) @ w.astype(np.float64).T
    err = np.abs(out.cpu().numpy() - want).max()
    assert err <= 1e-6 * np.sqrt(k) * np.abs(want).max() + 1e-6, f"max |diff| {err:.3e}"
    # strided rows of a wider buffer
    big = torch.zeros((m, n + 5), dtype=torch.float32, device="cuda")
    ops.gemm_f32(dev(a), dev(w), big[:, 2:2 + n])
    assert torch.equal(big[:, 2:2 + n], out) and not big[:, :2].any() and not big[:, 2 + n:].any()


def test_linear_bfloat16_float_output(ops):
    rng = np.random.default_rng(8)
    a, w = as_stored(rng.standard_normal((5, 96)), "bfloat16"), as_stored(rng.standard_normal((301, 96)), "bfloat16")
    out32 = torch.empty((5, 301), dtype=torch.float32, device="cuda")
    ops.linear(dev(a, torch.bfloat16), dev(w, torch.bfloat16), out32)
    want = a.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(out32.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max()
    out16 = torch.empty((5, 301), dtype=torch.bfloat16, device="cuda")
    ops.linear(dev(a, torch.bfloat16), dev(w, torch.bfloat16), out16)
    close(out16.float().cpu().numpy(), want, "bfloat16", "linear bf16")


def test_sampling_greedy_and_temperature(ops):
    rng = np.random.default_rng(9)
    vocab, rows = 1237, 6
    logits = (3 * rng.standard_normal((rows, vocab))).astype(np.float32)
    logits[0, 77] = logits[0, 900] = logits[0].max() + 1          # a tie: the lower id wins
    logits[1, 0] = 50.0
    temps = np.array([0.0, 0.0, 0.7, 1.0, 1.3, -1.0], dtype=np.float32)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    for trial in range(20):
        u = rng.random(rows).astype(np.float32)
        ops.sample(dev(logits), dev(temps), dev(u), out)
        got = out.cpu().numpy()
        for r in range(rows):
            want = plain.sample(logits[r], float(temps[r]), 1.0, -1, 1.0, [], float(u[r]))
            if got[r] != want:                                    # rounding of the running sum at a boundary
                p = plain.softmax(logits[r] / max(temps[r], 1e-9))
                c = np.cumsum(p.astype(np.float64))
                assert abs(got[r] - want) == 1 and min(abs(c[got[r]] - u[r]), abs(c[want] - u[r])) < 1e-5, (r, got[r], want)
    assert got[0] == 77 and got[1] == 0
    # u just below 1 gives the last id with any mass; u = 0 the first
    ops.sample(dev(logits), dev(temps), dev(np.zeros(rows, dtype=np.float32)), out)
    assert out.cpu().numpy()[3] == 0


@pytest.mark.parametrize("vocab", [152064, 40003])
def test_greedy_sampling_over_a_large_vocabulary(ops, vocab):
    """The argmax pass with several loads in flight per thread: the maximum at the start, at the end, in the
    ragged tail, a tie far apart (the lower id wins), rows of a wider buffer."""
    rng = np.random.default_rng(10)
    rows = 5
    buf = rng.standard_normal((rows, vocab + 6)).astype(np.float32)
    logits = buf[:, :vocab]
    logits[0, 0] = 9.0
    logits[1, vocab - 1] = 9.0
    logits[2, vocab - 3] = 9.0
    logits[3, 4097] = logits[3, vocab - 2] = 9.0
    want = [0, vocab - 1, vocab - 3, 4097, int(np.argmax(logits[4]))]
    full = dev(buf)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.sample(full[:, :vocab], dev(np.zeros(rows, dtype=np.float32)), dev(np.zeros(rows, dtype=np.float32)), out)
    assert out.cpu().numpy().tolist() == want


@pytest.mark.parametrize("vocab", [152064, 40003, 130])
def test_temperature_sampling_over_a_large_vocabulary(ops, vocab):
    """The draw by inverse CDF in the order of the ids, every warp summing a slab of the row: rows of a wider
    buffer (so that some rows are not 16-byte aligned), flat and peaked rows, draws at both ends and in the
    middle.  The id must be the one whose interval of the cumulative sum (in float64) holds u, up to the
    rounding of a float32 sum."""
    rng = np.random.default_rng(12)
    rows = 6
    buf = (2 * rng.standard_normal((rows, vocab + 5))).astype(np.float32)
    logits = buf[:, :vocab]
    logits[1] *= 0.01                                  # nearly flat
    logits[2, vocab - 1] = 25.0                        # all mass at the end
    logits[3, vocab // 2 + 1] = 12.0                   # most mass in the middle
    temps = np.array([1.0, 0.5, 1.0, 2.0, 0.8, 1.5], dtype=np.float32)
    full = dev(buf)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    x = logits.astype(np.float64) / temps[:, None].astype(np.float64)
    p = np.exp(x - x.max(axis=1, keepdims=True))
    c = np.cumsum(p / p.sum(axis=1, keepdims=True), axis=1)
    for u in [0.0, 1e-7, 0.25, 0.5, 0.75, 0.999, 0.99999994] + rng.random(12).tolist():
        uu = np.full(rows, u, dtype=np.float32)
        ops.sample(full[:, :vocab], dev(temps), dev(uu), out)
        got = out.cpu().numpy()
        for r in range(rows):
            g = int(got[r])
            assert 0 <= g < vocab
            below = c[r, g - 1] if g > 0 else 0.0
            assert below - 2e-5 <= float(uu[r]) < c[r, g] + 2e-5, (vocab, r, u, g, below, c[r, g])
            assert p[r, g] > 0


@pytest.mark.parametrize("std", [0.05, 0.3, 2.0])
def test_top_p_and_top_k_over_a_large_flat_vocabulary(ops, std):
    """152,064 ids of similar weight: a single id's share is then a few rounding steps of the running sums, and
    the thresholds' digit-by-digit search meets prefixes under which, by rounding, no digit reaches the bound.
    Every draw must be an id of the kept set whose interval of the renormalised cumulative sum (float64, in the
    order of falling probability, ties by lower id) holds u up to the rounding of a float32 sum."""
    rng = np.random.default_rng(14)
    vocab, rows = 152064, 8
    logits = (std * rng.standard_normal((rows, vocab))).astype(np.float32)
    temps = np.array([0.8, 1.0, 0.8, 1.3, 0.8, 1.0, 0.7, 0.8], dtype=np.float32)
    top_p = np.array([0.9, 0.5, 0.99, 0.9, 1.0, 0.3, 0.9, 0.9], dtype=np.float32)
    top_k = np.array([-1, -1, -1, 5000, 100, -1, 40000, -1], dtype=np.int32)
    x = logits.astype(np.float64) / temps[:, None]
    e = np.exp(x - x.max(axis=1, keepdims=True))
    ranks, cdfs, keeps = [], [], []
    for r in range(rows):
        order = np.lexsort((np.arange(vocab), -e[r]))
        c = np.cumsum(e[r][order])
        n_keep = vocab if top_k[r] <= 0 else min(int(top_k[r]), vocab)
        if top_p[r] < 1.0 or top_k[r] > 0:
            n_keep = min(n_keep, int(np.searchsorted(c[:n_keep], top_p[r] * c[n_keep - 1], side="left")) + 1)
        rank = np.empty(vocab, dtype=np.int64)
        rank[order] = np.arange(vocab)
        ranks.append(rank); cdfs.append(c[:n_keep] / c[n_keep - 1]); keeps.append(n_keep)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    d_logits, d_t, d_p, d_k = dev(logits), dev(temps), dev(top_p), dev(top_k)
    for trial in range(150):
        u = rng.random(rows).astype(np.float32)
        if trial == 0:
            u[:] = 0.0
        if trial == 1:
            u[:] = np.float32(0.99999994)
        ops.sample(d_logits, d_t, dev(u), out)
        ops.sample_filtered(d_logits, d_t, dev(u), d_p, d_k, out)
        got = out.cpu().numpy()
        for r in range(rows):
            g = int(got[r])
            assert 0 <= g < vocab, (std, trial, r, g, float(u[r]))
            pos = int(ranks[r][g])
            # the kept set's edge may move by the ids whose weight a rounding step of the sum covers
            assert pos < keeps[r] + max(2, keeps[r] // 2000), (std, trial, r, pos, keeps[r])
            pos = min(pos, keeps[r] - 1)
            below = cdfs[r][pos - 1] if pos > 0 else 0.0
            assert below - 1e-4 <= float(u[r]) < cdfs[r][pos] + 1e-4, (std, trial, r, float(u[r]), below, cdfs[r][pos])


def test_sampling_top_k_top_p_and_penalty(ops):
    rng = np.random.default_rng(10)
    vocab, rows = 997, 8
    logits = (2.5 * rng.standard_normal((rows, vocab))).astype(np.float32)
    logits[2, 5] = logits[2, 400] = logits[2].max() + 0.5         # tie inside the kept set
    temps = np.array([1.0, 0.8, 1.0, 1.2, 1.0, 0.0, 1.0, 0.9], dtype=np.float32)
    top_k = np.array([5, -1, 2, 50, 1, 3, -1, 997], dtype=np.int32)
    top_p = np.array([1.0, 0.5, 1.0, 0.9, 1.0, 0.5, 1.0, 0.3], dtype=np.float32)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    mismatches = 0
    for trial in range(25):
        u = rng.random(rows).astype(np.float32)
        ops.sample(dev(logits), dev(temps), dev(u), out)
        ops.sample_filtered(dev(logits), dev(temps), dev(u), dev(top_p), dev(top_k), out)
        got = out.cpu().numpy()
        for r in range(rows):
            want = plain.sample(logits[r], float(temps[r]), float(top_p[r]), int(top_k[r]), 1.0, [], float(u[r]))
            if got[r] != want:
                # only a knife-edge of the running sums may differ: the two ids are neighbours in
                # the reference's order
                p = plain.softmax(logits[r] * (np.float32(1) / temps[r]) if temps[r] > 0 else logits[r])
                order = plain.order_by_probability(p, list(range(vocab)))
                assert abs(order.index(got[r]) - order.index(want)) == 1, (r, got[r], want)
                mismatches += 1
    assert mismatches <= 3
    assert got[4] == int(np.argmax(logits[4]))                    # top_k = 1 is the largest
    # repetition penalty: each generated id once, l > 0 ? l / p : l * p
    l = dev(logits.copy())
    ids = np.array([3, 9, 9 + 0, 500, 7], dtype=np.int32)          # row 0: {3, 9}, row 1: none, row 2: {500, 7}
    start = np.array([0, 2, 2, 4, 4, 4, 4, 4, 4], dtype=np.int32)
    pen = np.array([1.5, 1.0, 2.0, 1, 1, 1, 1, 1], dtype=np.float32)
    ops.repetition_penalty(l, dev(np.array([3, 9, 500, 7], dtype=np.int32)), dev(start), dev(pen))
    want = logits.copy()
    want[0] = plain.repetition_penalty(logits[0], [3, 9, 3], 1.5)
    want[2] = plain.repetition_penalty(logits[2], [500, 7], 2.0)
    assert np.allclose(l.cpu().numpy(), want, rtol=1e-6)


@pytest.mark.parametrize("m,n,k,plan,ctas", [
    (8, 256, 512, (True, 16), 148), (1, 128, 64, (True, 16), 148), (8, 4608, 3584, None, 148), (5, 300, 200, (True, 16), 3),
    (33, 1000, 1024, (True, 64), 7), (64, 3584, 18944, None, 148), (100, 384, 576, (True, 128), 148),
    (300, 520, 448, (False, 256), 148), (2048, 1024, 512, (False, 256), 5), (130, 130, 72, (False, 256), 1),
    (16, 152064, 256, None, 148), (200, 700, 1032, (False, 128), 11), (40, 640, 8192, (True, 64), 148)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_gemm_bf16_tcgen05(ops, m, n, k, plan, ctas, out_dtype):
    """The tcgen05 + TMA product against a float64 product of the same bfloat16 operands: both
    orientations, every tile width, runs of (tile, slab) units that split tiles between CTAs in
    every way, ragged edges in rows, columns and K."""
    rng = np.random.default_rng(11)
    x, w = as_stored(rng.standard_normal((m, k)), "bfloat16"), as_stored(rng.standard_normal((n, k)) * 0.1, "bfloat16")
    want = x.astype(np.float64) @ w.astype(np.float64).T
    # float accumulation over k terms; bfloat16 output adds its own rounding
    tol = 4e-7 * np.sqrt(k) + (4e-3 if out_dtype == "bfloat16" else 0.0)
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    swapped = (plan or ops.tcgen05_plan(m, n, k))[0]
    if swapped:
        ops.tile_weights(wd)
    for tiled in ([False, True] if swapped else [False]):      # weights through a tensor map, then pre-tiled
        out = torch.full((m, n), float("nan"), dtype=DT[out_dtype], device="cuda")
        for _ in range(2):                              # twice: tickets must be zero again after a launch
            ops.gemm_bf16_tcgen05(xd, wd, out, plan, ctas, use_tiled=tiled)
        torch.cuda.synchronize()
        ops.check_status()
        got = out.float().cpu().numpy()
        assert np.isfinite(got).all()
        err = np.abs(got - want).max()
        assert err <= tol * np.abs(want).max(), f"tiled={tiled}: max |diff| {err:.3e} vs scale {np.abs(want).max():.3e}"


@pytest.mark.parametrize("m,n,k,ctas", [(8, 3584, 512, 148), (1, 128, 64, 148), (5, 296, 200, 3), (33, 1000, 1024, 7),
                                        (64, 3584, 4736, 148), (100, 384, 576, 148), (128, 200, 1088, 11)])
def test_gemm_bf16_tcgen05_fused_norm(ops, m, n, k, ctas):
    """A product that ends a residual branch (residual += x w^T; out = residual * gain; sums of squares
    left in parts) followed by a product that applies the rows' factor, against the same done plainly:
    y = rmsnorm(residual + x w^T) w2^T.  Tiles split between CTAs, ragged feature counts."""
    rng = np.random.default_rng(5)
    x = as_stored(rng.standard_normal((m, k)), "bfloat16")
    w = as_stored(rng.standard_normal((n, k)) * 0.1, "bfloat16")
    n2 = 264
    w2 = as_stored(rng.standard_normal((n2, -(-n // 8) * 8)) * 0.1, "bfloat16")[:, :n]
    res = rng.standard_normal((m, n)).astype(np.float32) * 2
    gain = (1 + 0.3 * rng.standard_normal(n)).astype(np.float32)
    eps = 1e-5
    new_res = res.astype(np.float64) + x.astype(np.float64) @ w.astype(np.float64).T
    rstd = 1.0 / np.sqrt((new_res ** 2).mean(axis=1, keepdims=True) + eps)
    scaled = new_res * gain
    assert n % 8 == 0, "the second product needs K a multiple of 8"
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    w2d = dev(np.ascontiguousarray(w2), torch.bfloat16)
    ops.tile_weights(wd)
    for rep in range(2):
        rd, gd = dev(res), dev(gain)
        parts = ops.sumsq_parts(n)
        ss = torch.full((parts + 1, m + 3), float("nan"), device="cuda")
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        fuse = ops.ResidualNorm(rd, gd, ss, eps)
        ops.gemm_bf16_tcgen05(xd, wd, out, None, ctas, fuse=fuse)
        y = torch.full((m, n2), float("nan"), dtype=torch.float32, device="cuda")
        ops.gemm_bf16_tcgen05(out, w2d, y, None, ctas, x_scale=fuse.scale())
        torch.cuda.synchronize()
        ops.check_status()
        got_res = rd.cpu().numpy()
        assert np.abs(got_res - new_res).max() <= 1e-5 * np.abs(new_res).max() + 4e-7 * np.sqrt(k) * np.abs(new_res).max()
        got_ss = ss[:parts, :m].cpu().numpy().astype(np.float64).sum(axis=0)
        assert np.allclose(got_ss, (new_res ** 2).sum(axis=1), rtol=1e-5)
        assert torch.isnan(ss[parts]).all() and torch.isnan(ss[:, m:]).all()       # nothing written outside
        got_out = out.float().cpu().numpy()
        assert np.abs(got_out - scaled).max() <= 4e-3 * np.abs(scaled).max() + 1e-6
        # second product: on the bfloat16 values the first one stored
        want_y = (got_out.astype(np.float64) * rstd) @ w2.astype(np.float64).T
        got_y = y.cpu().numpy()
        assert np.isfinite(got_y).all()
        assert np.abs(got_y - want_y).max() <= (4e-7 * np.sqrt(n) + 2e-6) * np.abs(want_y).max()


@pytest.mark.parametrize("m,inter,k,ctas", [(8, 18944 // 4, 512, 148), (1, 64, 64, 148), (5, 200, 200, 3), (33, 176, 1024, 7),
                                            (16, 1000, 576, 148), (100, 224, 96, 11), (128, 128, 64, 148),
                                            # whole tiles of 32 and 64 columns: the epilogue that works in rounds of 32
                                            (40, 200, 256, 148), (64, 192, 128, 2), (17, 100, 64, 148), (49, 328, 512, 6)])
@pytest.mark.parametrize("scaled", [False, True])
def test_gemm_bf16_tcgen05_gated(ops, m, inter, k, ctas, scaled):
    """The gate-and-up product with the activation in its epilogue against silu(x g^T) * (x u^T) done
    plainly; feature counts that are no multiple of 64, tiles split between CTAs, with and without
    the rows' factor of a norm."""
    rng = np.random.default_rng(9)
    x = as_stored(rng.standard_normal((m, k)), "bfloat16")
    w = as_stored(rng.standard_normal((2 * inter, k)) * 0.1, "bfloat16")
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    ops.tile_weights(wd, inter)
    factor = np.ones((m, 1))
    scale = None
    if scaled:
        parts = 5
        ss = rng.random((parts, m)).astype(np.float32) * 40
        scale = ops.RowScale(dev(ss), parts, 96, 1e-5)
        factor = 1.0 / np.sqrt(ss.astype(np.float64).sum(axis=0) / 96 + 1e-5)[:, None]
    gu = (x.astype(np.float64) @ w.astype(np.float64).T) * factor
    g, u = gu[:, :inter], gu[:, inter:]
    want = g / (1 + np.exp(-g)) * u
    full = torch.full((m, inter + 8), float("nan"), dtype=torch.bfloat16, device="cuda")
    out = full[:, :inter]
    for _ in range(2):
        ops.gemm_bf16_tcgen05(xd, wd, out, None, ctas, x_scale=scale, gated=True)
    torch.cuda.synchronize()
    ops.check_status()
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    # bfloat16 output; float accumulation errors of gate and up multiply each other's values
    assert np.abs(got - want).max() <= (4e-3 + 4e-6 * np.sqrt(k)) * np.abs(want).max()
    assert torch.isnan(full[:, inter:]).all()                   # nothing written beyond the gate features


def test_device_sampler_on_the_reference_samplers_golden_rows(ops):
    """The device sampler on the rows for which tests/golden holds the reference sampler's answers."""
    import json
    import os
    with open(os.path.join(os.path.dirname(__file__), "golden", "sampler_golden.json")) as f:
        cases = json.load(f)["cases"]
    logits = np.array([c["logits"] for c in cases], dtype=np.float32)
    temps = np.array([c["temperature"] for c in cases], dtype=np.float32)
    u = np.array([c["u"] for c in cases], dtype=np.float32)
    top_p = np.array([c["top_p"] for c in cases], dtype=np.float32)
    top_k = np.array([c["top_k"] for c in cases], dtype=np.int32)
    out = torch.empty(len(cases), dtype=torch.int32, device="cuda")
    ops.sample(dev(logits), dev(temps), dev(u), out)
    ops.sample_filtered(dev(logits), dev(temps), dev(u), dev(top_p), dev(top_k), out)
    got = out.cpu().numpy()
    wrong = [i for i, c in enumerate(cases) if got[i] != c["token"]]
    for i in wrong:                                   # only a knife-edge of a running sum may differ
        p = plain.softmax(logits[i] * (np.float32(1) / temps[i]) if temps[i] > 0 else logits[i])
        order = plain.order_by_probability(p, list(range(logits.shape[1])))
        assert abs(order.index(int(got[i])) - order.index(cases[i]["token"])) == 1 or \
            abs(int(got[i]) - cases[i]["token"]) == 1, (i, got[i], cases[i]["token"])
    assert len(wrong) <= 2


def test_a_page_that_is_not_there_is_reported_not_followed(ops):
    """A block table with an entry that names no page of the cache (what the cache manager stores for a
    page it took back is -1): the cache write leaves every byte alone (rows beside the cache tensor
    included), the attention kernels read page 0 in its place, and all of them leave a note that
    ops.check_status() raises on.  Nothing traps."""
    rng = np.random.default_rng(8)
    nh, nkv, d, page, n_pages = 4, 2, 128, 16, 6
    ops.check_status()
    whole = torch.full((n_pages + 2, 2, nkv, page * d), 7.0, dtype=torch.bfloat16, device="cuda")
    cache = whole[1:-1]                                   # canary pages before and after the cache
    bt = np.array([[2, -1, 3], [4, 77, 5]], dtype=np.int32)
    pos = np.array([15, 16, 17, 20], dtype=np.int32)      # request 0: slot 15 of page 2, then its missing second page
    req = np.array([0, 0, 0, 1], dtype=np.int32)          # request 1: its second entry lies beyond the cache
    qkv = rng.standard_normal((4, (nh + 2 * nkv) * d)).astype(np.float32)
    denom = np.power(np.float32(1e4), np.arange(d // 2, dtype=np.float32) * 2 / d).astype(np.float32)
    for dtype in (torch.bfloat16, torch.float32):
        w = whole.to(dtype)
        c = w[1:-1]
        q_out = torch.empty((4, nh * d), dtype=dtype, device="cuda")
        ops.rope_cache_write(dev(qkv, dtype), None, dev(pos), dev(req), dev(bt), dev(denom), q_out, c, num_heads=nh,
                             num_kv_heads=nkv, head_dim=d, rotary_dim=d, pairing=0, page_size=page, write_kv=True)
        with pytest.raises(ops.KernelError, match="names a page|named a page"):
            ops.check_status()
        changed = (w != 7.0).flatten(1).any(dim=1).cpu().numpy()
        assert changed.tolist() == [False, False, False, True, False, False, False, False], changed   # page 2 only
        ops.check_status()                                # the note was cleared
    # the readers: a decode step and a portion whose visible pages include the missing one
    q = dev(rng.standard_normal((2, nh * d)), torch.bfloat16)
    q_start, ctx = dev(np.array([0, 1, 2], dtype=np.int32)), dev(np.array([20, 20], dtype=np.int32))
    out = torch.zeros_like(q)
    scale = float(1 / np.sqrt(np.float32(d)))
    ops.attention_decode_mma(q, cache, out, q_start, ctx, dev(bt), None, 2, 1, None, None, None, num_heads=nh,
                             num_kv_heads=nkv, head_dim=d, page_size=page, window=0, scale=scale)
    with pytest.raises(ops.KernelError, match="named a page"):
        ops.check_status()
    ops.attention_prefill_tc(q, cache, out, q_start, ctx, dev(bt), dev(np.array([0, 1], dtype=np.int32)),
                             dev(np.array([0, 0], dtype=np.int32)), num_heads=nh, num_kv_heads=nkv, head_dim=d,
                             page_size=page, window=0, scale=scale)
    with pytest.raises(ops.KernelError, match="named a page"):
        ops.check_status()
    ops.attention_simt(q, cache, out, dev(np.array([20, 20], dtype=np.int32)), dev(np.array([0, 1], dtype=np.int32)), dev(bt),
                       num_heads=nh, num_kv_heads=nkv, head_dim=d, page_size=page, window=0, scale=scale)
    with pytest.raises(ops.KernelError, match="named a page"):
        ops.check_status()
    assert torch.isfinite(out.float()).all()


def test_decode_attention_refuses_pages_it_cannot_copy(ops):
    """Pages of fewer than 8 slots (or no multiple of 8) cannot be copied as the kernel copies a tile: refused,
    nothing launched."""
    q = torch.zeros((1, 2 * 64), dtype=torch.bfloat16, device="cuda")
    out = torch.full_like(q, 5.0)
    cache = torch.zeros((4, 2, 2, 4 * 64), dtype=torch.bfloat16, device="cuda")
    z = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        ops.attention_decode_mma(q, cache, out, z[:2], z[:1], z.view(1, 4), None, 1, 1, None, None, None, num_heads=2,
                                 num_kv_heads=2, head_dim=64, page_size=4, window=0, scale=0.125)
    rc = ops.lib().vcb_attention_decode_mma(q.data_ptr(), cache.data_ptr(), out.data_ptr(), z.data_ptr(), z.data_ptr(),
                                            z.data_ptr(), 4, None, 1, 1, None, None, None, None, 2, 2, 64, 4, 0, 0.125, 4,
                                            None, None)
    assert rc == 10002
    torch.cuda.synchronize()
    assert (out == 5.0).all()
