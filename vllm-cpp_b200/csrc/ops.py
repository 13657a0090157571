"""Python face of the CUDA kernels: argument checks, then one launch each.

Tensors are ``torch`` CUDA tensors used as typed device buffers; the launchers
get their pointers and the current stream.  Every function refuses what the
kernel behind it cannot do with a :class:`KernelError` that says why.  Nothing
here runs on the CPU.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build as _build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


_lib = None
_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float

_SIGNATURES = {
    "vcb_embedding": [_P, _P, _P, _I, _I, _I, _P],
    "vcb_add_rmsnorm": [_P, _P, _P, _P, _P, _I, _I, _F, _I, _P],
    "vcb_silu_mul": [_P, _P, _I, _I, _I, _P],
    "vcb_add_bias": [_P, _P, _I, _I, _I, _P],
    "vcb_rope_cache_write": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P],
    "vcb_attention_simt": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P, _I, _P],
    "vcb_gemm_f32": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "vcb_attention_decode_mma": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "vcb_attention_prefill_tc": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "vcb_gemm_bf16_tcgen05": [_P, _I, _I, _P, _P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _P, _P, _I, _P, _P],
    "vcb_gemm_bf16_tcgen05_fused": [_P, _I, _I, _P, _P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _P, _P, _I, _P,
                                    _P, _I, _I, _I, _F, _P, _I, _P, _P, _I, _I, _P],
    "vcb_tile_weights": [_P, _I, _I, _I, _I, _P, _P],
    "vcb_repetition_penalty": [_P, _I, _P, _P, _P, _I, _I, _P],
    "vcb_sample": [_P, _I, _I, _P, _P, _P, _I, _P],
    "vcb_sample_filtered": [_P, _I, _I, _P, _P, _P, _P, _P, _P, _I, _P],
    "vcb_random_normal": [_P, ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_ulonglong, _F, _F, _I, _P],
}


_pdl = True


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch of this library's kernels on or off (see common.cuh)."""
    global _pdl
    _pdl = bool(on)
    if _lib is not None:
        _lib.vcb_set_pdl(1 if _pdl else 0)


def lib():
    """The kernel library; built and loaded on first use."""
    global _lib
    if _lib is None:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine runs on an sm_100a GPU only and has no CPU path")
        l = _build.load()
        for name, sig in _SIGNATURES.items():
            fn = getattr(l, name, None)
            if fn is None:
                raise KernelError(f"kernel library lacks {name}; rebuild it (delete csrc/_build)")
            fn.argtypes = sig
            fn.restype = _I
        l.vcb_set_pdl.argtypes = [_I]
        l.vcb_set_pdl.restype = None
        l.vcb_set_pdl(1 if _pdl else 0)
        _lib = l
    return _lib


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = None


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch (a caller may have switched streams, as a
    graph capture does), so through torch's raw query where it has one: torch.cuda.current_stream() builds a
    Stream object each time, a quarter of the host's time in a step that is launched kernel by kernel."""
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


_launches = 0


def launch_count() -> int:
    """Launches of this library's own kernels so far (library products are not counted)."""
    return _launches


def add_launches(n: int) -> None:
    """Account for kernels that ran inside a replayed CUDA graph."""
    global _launches
    _launches += n


def _check(code: int, what: str) -> None:
    global _launches
    if code == 0:
        _launches += 1
        return
    if code == 10001:
        raise KernelError(f"{what}: the kernel refused its arguments")
    if code == 10002:
        raise KernelError(f"{what}: size not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {code}")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"storage type {dt} is not supported (float32 or bfloat16)")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _dev(t: torch.Tensor, name: str, dtype=None) -> int:
    _need(t.is_cuda, f"{name} must live on the GPU")
    _need(t.is_contiguous(), f"{name} must be contiguous")
    if dtype is not None:
        _need(t.dtype == dtype, f"{name} must be {dtype}, is {t.dtype}")
    return t.data_ptr()


# --------------------------------------------------------------------- ops
def embedding(table: torch.Tensor, ids: torch.Tensor, residual: torch.Tensor) -> None:
    """residual[t] = float(table[ids[t]]); ids int32 [n], residual float32 [n, hidden].  An id outside the
    table leaves a row of zeros and code 12 in the status word."""
    n, hidden = residual.shape
    _need(table.dim() == 2 and table.shape[1] == hidden, "embedding table width differs from the residual's")
    _need(ids.numel() == n, "one id per residual row")
    _check(lib().vcb_embedding(_dev(table, "table"), _dev(ids, "ids", torch.int32),
                               _dev(residual, "residual", torch.float32), n, hidden, table.shape[0],
                               status_tensor(table.device).data_ptr(), dtype_code(table.dtype), _stream()), "embedding")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor,
                out: torch.Tensor, eps: float, row_index: Optional[torch.Tensor] = None) -> None:
    """out = rmsnorm(residual (+ delta)) * gain; the sum is written back to residual unless rows are gathered."""
    hidden = residual.shape[1]
    n_rows = out.shape[0]
    _need(out.shape[1] == hidden and gain.numel() == hidden, "add_rmsnorm: widths differ")
    if delta is not None:
        _need(delta.shape == residual.shape and delta.dtype == out.dtype, "add_rmsnorm: delta shape or type differs")
    if row_index is None:
        _need(n_rows == residual.shape[0], "add_rmsnorm: one output row per residual row")
    else:
        _need(row_index.numel() == n_rows, "add_rmsnorm: one row index per output row")
    _check(lib().vcb_add_rmsnorm(_dev(residual, "residual", torch.float32),
                                 None if delta is None else _dev(delta, "delta"),
                                 _dev(gain, "gain", torch.float32), _dev(out, "out"),
                                 None if row_index is None else _dev(row_index, "row_index", torch.int32),
                                 n_rows, hidden, float(eps), dtype_code(out.dtype), _stream()), "add_rmsnorm")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, inter + i]."""
    n, inter = out.shape
    _need(gate_up.shape == (n, 2 * inter) and gate_up.dtype == out.dtype, "silu_mul: gate_up must be [n, 2*inter]")
    _check(lib().vcb_silu_mul(_dev(gate_up, "gate_up"), _dev(out, "out"), n, inter,
                              dtype_code(out.dtype), _stream()), "silu_mul")


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    """x[t, c] += bias[c] in place."""
    rows, cols = x.shape
    _need(bias.numel() == cols, "add_bias: one bias value per column")
    _check(lib().vcb_add_bias(_dev(x, "x"), _dev(bias, "bias", torch.float32), rows, cols,
                              dtype_code(x.dtype), _stream()), "add_bias")


def rope_cache_write(qkv, bias, positions, req_of_token, block_table, denom, q_out, cache, *,
                     num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int, pairing: int,
                     page_size: int, write_kv: bool) -> None:
    """Bias, rotation and cache write in one pass over the q/k/v product (see elementwise.cu)."""
    n = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    _need(qkv.shape == (n, width), f"qkv must be [n, {width}], is {tuple(qkv.shape)}")
    _need(q_out.shape == (n, num_heads * head_dim) and q_out.dtype == qkv.dtype, "q_out shape or type")
    _need(head_dim % 2 == 0 and rotary_dim % 2 == 0 and 0 <= rotary_dim <= head_dim, "rotary_dim must be even and <= head_dim")
    _need(cache.dtype == qkv.dtype, "cache and activations must share a storage type")
    if rotary_dim:
        _need(denom is not None and denom.numel() == rotary_dim // 2, "denom must hold rotary_dim/2 values")
    if bias is not None:
        _need(bias.numel() == width, "bias width")
    _check(lib().vcb_rope_cache_write(
        _dev(qkv, "qkv"), None if bias is None else _dev(bias, "bias", torch.float32),
        _dev(positions, "positions", torch.int32), _dev(req_of_token, "req_of_token", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1],
        None if denom is None else _dev(denom, "denom", torch.float32), _dev(q_out, "q_out"),
        _dev(cache, "cache"), n, num_heads, num_kv_heads, head_dim, rotary_dim, pairing, page_size,
        1 if write_kv else 0, cache.shape[0], status_tensor(qkv.device).data_ptr(), dtype_code(qkv.dtype), _stream()),
        "rope_cache_write")


def attention_simt(q, cache, out, positions, req_of_token, block_table, *, num_heads: int,
                   num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float) -> None:
    n = q.shape[0]
    _need(head_dim <= 256, f"head_dim {head_dim} exceeds 256, the largest this attention kernel takes")
    _need(q.shape == (n, num_heads * head_dim) and out.shape == q.shape and out.dtype == q.dtype, "q/out shape")
    _need(num_heads % num_kv_heads == 0, "num_heads must be a multiple of num_kv_heads")
    _need(cache.dtype == q.dtype, "cache and q must share a storage type")
    _check(lib().vcb_attention_simt(
        _dev(q, "q"), _dev(cache, "cache"), _dev(out, "out"), _dev(positions, "positions", torch.int32),
        _dev(req_of_token, "req_of_token", torch.int32), _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], n, num_heads, num_kv_heads, head_dim, page_size, window, float(scale),
        cache.shape[0], status_tensor(q.device).data_ptr(), dtype_code(q.dtype), _stream()), "attention_simt")


MMA_HEAD_DIMS = (64, 128)
DECODE_KEY_TILE = 64          # keys per tile of the decode kernel
DECODE_MAX_SPLITS = 32


def attention_decode_mma(q, cache, out, q_start, ctx_lens, block_table, req_list, n_list: int, nsplit: int,
                         part_o, part_ml, counters, *, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                         window: int, scale: float, split_tiles=None) -> None:
    """Split-KV tensor-core attention for requests that bring one token each (bfloat16).  The grid has
    ``nsplit`` columns; without ``split_tiles`` every request's keys are cut into that many equal parts,
    with it (int32 [1] on the device: tiles of DECODE_KEY_TILE keys per split) a request takes as many
    columns as its context needs, so that requests of different lengths keep all CTAs equally busy."""
    _need(q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attention_decode_mma is a bfloat16 kernel")
    _need(head_dim in MMA_HEAD_DIMS and page_size % 8 == 0,
          f"attention_decode_mma takes head sizes {MMA_HEAD_DIMS} and pages of a multiple of 8 slots, got {head_dim} and {page_size}")
    if nsplit > 1:
        need = n_list * num_heads * nsplit
        _need(part_o is not None and part_o.numel() >= need * head_dim and part_ml.numel() >= need * 2
              and counters is not None and counters.numel() >= n_list * num_kv_heads,
              "attention_decode_mma: scratch for the split merge is too small")
    _check(lib().vcb_attention_decode_mma(
        _dev(q, "q"), _dev(cache, "cache"), _dev(out, "out"), _dev(q_start, "q_start", torch.int32),
        _dev(ctx_lens, "ctx_lens", torch.int32), _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], None if req_list is None else _dev(req_list, "req_list", torch.int32),
        n_list, nsplit, None if part_o is None else _dev(part_o, "part_o", torch.float32),
        None if part_ml is None else _dev(part_ml, "part_ml", torch.float32),
        None if counters is None else _dev(counters, "counters", torch.int32),
        None if split_tiles is None else _dev(split_tiles, "split_tiles", torch.int32),
        num_heads, num_kv_heads, head_dim, page_size, window, float(scale), cache.shape[0],
        status_tensor(q.device).data_ptr(), _stream()), "attention_decode_mma")


TC_ATTENTION_HEAD_DIMS = (64, 128)      # head sizes of the tcgen05 prefill attention kernel
TC_ATTENTION_TILE_ROWS = 128     # packed rows per tile of its work list


def attention_prefill_tc(q, cache, out, q_start, ctx_lens, block_table, tile_req, tile_row0, *,
                         num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int,
                         scale: float) -> None:
    """Attention for portions of any length on tcgen05 tensor cores (scores and output tiles in tensor
    memory); head sizes 64 and 128, bfloat16, pages of a multiple of 8 slots, tiles of 128 packed rows."""
    _need(q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attention_prefill_tc is a bfloat16 kernel")
    _need(head_dim in TC_ATTENTION_HEAD_DIMS and page_size % 8 == 0,
          f"attention_prefill_tc takes head sizes {TC_ATTENTION_HEAD_DIMS} and pages of a multiple of 8 slots")
    n_tiles = tile_req.numel()
    _need(tile_row0.numel() == n_tiles, "one first row per tile")
    _check(lib().vcb_attention_prefill_tc(
        _dev(q, "q"), _dev(cache, "cache"), _dev(out, "out"), _dev(q_start, "q_start", torch.int32),
        _dev(ctx_lens, "ctx_lens", torch.int32), _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], _dev(tile_req, "tile_req", torch.int32), _dev(tile_row0, "tile_row0", torch.int32),
        n_tiles, num_heads, num_kv_heads, head_dim, page_size, window, float(scale), cache.shape[0],
        status_tensor(q.device).data_ptr(), _stream()), "attention_prefill_tc")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T in true 32-bit arithmetic; rows may be strided."""
    m, k = a.shape
    n = w.shape[0]
    _need(w.shape[1] == k and out.shape == (m, n), "gemm_f32: shapes do not agree")
    for t, name in ((a, "a"), (w, "w"), (out, "out")):
        _need(t.is_cuda and t.dtype == torch.float32 and t.stride(1) == 1, f"gemm_f32: {name} must be float32 with unit inner stride")
    _check(lib().vcb_gemm_f32(a.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k,
                              a.stride(0), w.stride(0), out.stride(0), _stream()), "gemm_f32")


_sm_count: Optional[int] = None


def sm_count() -> int:
    """Streaming multiprocessors of the device the engine runs on, asked once (148 on a B200): the
    most CTAs of a persistent kernel, and what the parts size their work lists by."""
    global _sm_count
    if _sm_count is None:
        _need(torch.cuda.is_available(), "no CUDA device")
        _sm_count = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
    return _sm_count


_status: Optional[torch.Tensor] = None
STATUS_MEANING = {1: "the TMA producer waited too long for a free stage", 2: "the MMA issuer waited too long for a loaded stage",
                  3: "the epilogue waited too long for the accumulator", 4: "the MMA issuer waited too long for a free accumulator",
                  5: "decode attention waited too long for a cache tile", 6: "prefill attention waited too long for a cache tile",
                  8: "a product's merge waited too long for the tile's other segments",
                  9: "tcgen05 prefill attention waited too long on one of its barriers",
                  10: "tcgen05 prefill attention found its shared memory not aligned to 1024 bytes",
                  12: "a token id outside the vocabulary reached the embedding on the device (a sampled id of the step "
                      "before, which the host had not yet seen); its row was left zero",
                  11: "a block table named a page that the cache does not have (a released or missing entry); "
                      "nothing was written through it and attention read page 0 in its place"}


def status_tensor(device) -> torch.Tensor:
    """The device word in which kernels with bounded waits record a wait that ran out."""
    global _status
    if _status is None or _status.device != torch.device(device):
        _status = torch.zeros(1, dtype=torch.int32, device=device)
    return _status


def check_status() -> None:
    """Raise if a kernel noted something in the status word since the last check: a bounded wait that ran
    out, a page or a token id that does not exist (synchronises)."""
    if _status is None:
        return
    code = int(_status.item())
    if code:
        _status.zero_()
        raise KernelError(f"a kernel left status {code}: {STATUS_MEANING.get(code, code)}")


def tcgen05_plan(tokens: int, features: int, k: int):
    """(swapped, bn) for out[tokens, features] = x[tokens, k] @ w[features, k]^T: few tokens put the
    weights on the 128-row side of the tensor-core tile."""
    if tokens <= 128:
        return True, (16 if tokens <= 16 else 32 if tokens <= 32 else 64 if tokens <= 64 else 128)
    return False, 256


GEMM_MAX_TICKETS = 16384


def tile_weights(w: torch.Tensor, gated: int = 0) -> torch.Tensor:
    """The pre-tiled image of a weight matrix for decode products (see gemm_tcgen05.cu): made once,
    kept on the tensor object itself (so it lives and dies with the matrix), and used by ``linear``
    whenever the weights sit on the 128-row side.  The matrix must not change afterwards.
    ``gated`` > 0: w is the [2 * gated, k] gate-and-up matrix of a gated feed-forward and the image
    pairs gate and up rows in every tile, for ``linear_gated``."""
    attr = "_vcb_tiled_gated" if gated else "_vcb_tiled"
    t = getattr(w, attr, None)
    if t is None:
        _need(w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1, "tile_weights: a bfloat16 matrix")
        rows, k = w.shape
        _need(gated == 0 or rows == 2 * gated, "tile_weights: a gated matrix has 2 * gated rows")
        tiles = -(-gated // 64) if gated else -(-rows // 128)
        t = torch.empty(tiles * -(-k // 64) * 16384, dtype=torch.uint8, device=w.device)
        _check(lib().vcb_tile_weights(w.data_ptr(), rows, k, w.stride(0), gated, t.data_ptr(), _stream()), "tile_weights")
        setattr(w, attr, t)
    return t


def drop_tiled_weights(w: torch.Tensor) -> None:
    for attr in ("_vcb_tiled", "_vcb_tiled_gated"):
        if getattr(w, attr, None) is not None:
            setattr(w, attr, None)


def tiled_weights_of(w: torch.Tensor, gated: bool = False) -> Optional[torch.Tensor]:
    return getattr(w, "_vcb_tiled_gated" if gated else "_vcb_tiled", None)


class RowScale:
    """Says that the rows of a product's input still lack the factor of an RMSNorm:
    row t is to be multiplied by rsqrt(sum(sumsq[:parts, t]) / width + eps).  ``sumsq`` holds
    partial sums of squares of the un-normalised row, [parts, tokens] float32."""
    __slots__ = ("sumsq", "parts", "width", "eps")

    def __init__(self, sumsq: torch.Tensor, parts: int, width: int, eps: float):
        self.sumsq, self.parts, self.width, self.eps = sumsq, parts, width, float(eps)


class ResidualNorm:
    """Asks a product to end a residual branch itself: residual (float32 [tokens, features]) += result;
    out = bfloat16(residual * gain), the un-normalised input of the norm that follows; sumsq
    ([sumsq_parts(features), tokens] float32) = partial sums of squares of the new residual rows.
    ``scale()`` is the RowScale the next product needs."""
    __slots__ = ("residual", "gain", "sumsq", "eps")

    def __init__(self, residual: torch.Tensor, gain: torch.Tensor, sumsq: torch.Tensor, eps: float):
        self.residual, self.gain, self.sumsq, self.eps = residual, gain, sumsq, float(eps)

    def scale(self) -> RowScale:
        return RowScale(self.sumsq, sumsq_parts(self.residual.shape[1]), self.residual.shape[1], self.eps)


def sumsq_parts(features: int) -> int:
    """Partial sums a ResidualNorm product leaves per token: one per epilogue warp of every 128-row tile."""
    return 4 * (-(-features // 128))


def gemm_bf16_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, plan=None, max_ctas: Optional[int] = None,
                      use_tiled: bool = True, x_scale: Optional[RowScale] = None,
                      fuse: Optional[ResidualNorm] = None, gated: bool = False) -> None:
    """out = x @ w^T on tcgen05 tensor cores fed by TMA (see gemm_tcgen05.cu); out bfloat16 or float32.
    When the weights are the 128-row operand and tile_weights(w) has been made, the image is used
    (``use_tiled`` False forces the tensor-map path).  ``x_scale`` and ``fuse`` (up to 128 tokens):
    see RowScale and ResidualNorm.  ``gated``: w is a gate-and-up matrix [2 * inter, k] with a gated
    image (tile_weights(w, inter)) and out [tokens, inter] = silu(x gate^T) * (x up^T)."""
    m, k = x.shape
    n = w.shape[0]
    _need(w.shape[1] == k and out.shape == (m, n // 2 if gated else n), "gemm_bf16_tcgen05: shapes do not agree")
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_bf16_tcgen05: operands must be bfloat16")
    _need(out.dtype in (torch.bfloat16, torch.float32) and out.stride(1) == 1 and x.stride(1) == 1 and w.stride(1) == 1,
          "gemm_bf16_tcgen05: unit inner strides, out bfloat16 or float32")
    _need(k % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0,
          "gemm_bf16_tcgen05: TMA needs K and the row strides to be multiples of 8 and 16-byte aligned bases")
    swapped, bn = plan or tcgen05_plan(m, n, k)
    sc = (None, 0, 0, 1, 0.0)
    if x_scale is not None:
        _need(swapped and m <= bn <= 128, "gemm_bf16_tcgen05: a row scale needs the few-token form")
        _need(x_scale.sumsq.dtype == torch.float32 and x_scale.sumsq.dim() == 2 and x_scale.sumsq.stride(1) == 1
              and x_scale.sumsq.shape[0] >= x_scale.parts and x_scale.sumsq.shape[1] >= m,
              "gemm_bf16_tcgen05: sums of squares must be float32 [parts, tokens]")
        sc = (x_scale.sumsq.data_ptr(), x_scale.parts, x_scale.sumsq.stride(0), x_scale.width, x_scale.eps)
    fu = (None, 0, None, None, 0)
    if fuse is not None:
        _need(swapped and m <= bn <= 128 and out.dtype == torch.bfloat16,
              "gemm_bf16_tcgen05: a fused residual needs the few-token form and a bfloat16 result")
        r, g, ss = fuse.residual, fuse.gain, fuse.sumsq
        _need(r.dtype == torch.float32 and r.shape == (m, n) and r.stride(1) == 1 and g.dtype == torch.float32
              and g.shape == (n,) and g.is_contiguous(), "gemm_bf16_tcgen05: residual float32 [tokens, features], gain float32 [features]")
        _need(ss.dtype == torch.float32 and ss.dim() == 2 and ss.stride(1) == 1 and ss.shape[0] >= sumsq_parts(n)
              and ss.shape[1] >= m, "gemm_bf16_tcgen05: sums of squares must be float32 [sumsq_parts(features), tokens]")
        fu = (r.data_ptr(), r.stride(0), g.data_ptr(), ss.data_ptr(), ss.stride(0))
    p, q = (w, x) if swapped else (x, w)
    tiled = tiled_weights_of(w, gated) if (swapped and use_tiled) else None
    if gated:
        _need(swapped and m <= bn <= 128 and tiled is not None and out.dtype == torch.bfloat16 and fuse is None,
              "gemm_bf16_tcgen05: the gated form needs few tokens, a gated tile image and a bfloat16 result")
    sms = sm_count()
    if max_ctas is None:
        # What the measurement at load chose for this shape (choose_ctas), else: tiles of 32 and 64 columns
        # run two CTAs of the product on every SM (its ring is then four or five stages deep each).  A stage
        # carries the tokens' operand beside the weights', half as much again at 64 tokens, and one CTA's ring
        # does not hold enough bytes in flight for the memory's rate (measured at 64 tokens, 7B sizes:
        # gate-and-up 49.9 -> 44.6 us, qkv 14.8 -> 12.8; at 128 it is slower).
        max_ctas = _cta_choice.get((n, k, bn, bool(gated), fuse is not None), 2 * sms if bn in (32, 64) else sms)
    partial = scratch("gemm_partial", sms * 2 * 256 * 128, out.device)
    tickets = zeroed_ints("gemm_tickets", GEMM_MAX_TICKETS, out.device)
    _check(lib().vcb_gemm_bf16_tcgen05_fused(p.data_ptr(), p.shape[0], p.stride(0),
                                             None if tiled is None else tiled.data_ptr(),
                                             q.data_ptr(), q.shape[0], q.stride(0), k,
                                             out.data_ptr(), out.stride(0), 1 if out.dtype == torch.float32 else 0,
                                             1 if swapped else 0, bn, min(max_ctas, 2 * sms), partial.data_ptr(),
                                             tickets.data_ptr(), GEMM_MAX_TICKETS, status_tensor(out.device).data_ptr(),
                                             *sc, *fu, n // 2 if gated else 0, _stream()), "gemm_bf16_tcgen05")


TCGEN05_MAX_TOKENS = 128      # up to here the engine's own tcgen05 product may run; above, the library's
_tcgen05_linear = True
# (features, k, token bucket) -> True if the tcgen05 kernel was measured faster than cuBLAS here
_linear_choice = {}


def set_tcgen05_linear(on: bool) -> None:
    """Allow this library's tcgen05 product for bfloat16 products with few tokens (default), or cuBLAS for all."""
    global _tcgen05_linear
    _tcgen05_linear = bool(on)


_linear_tuning = True


def set_linear_tuning(on: bool) -> None:
    """With tuning off nothing is measured at load, so every product with few tokens runs this
    library's tcgen05 kernel (tests use it to pin the path)."""
    global _linear_tuning
    _linear_tuning = bool(on)


def token_bucket(m: int) -> int:
    return 16 if m <= 16 else 32 if m <= 32 else 64 if m <= 64 else 128


def _tcgen05_ok(x, w, out) -> bool:
    m, k = x.shape
    return (m <= TCGEN05_MAX_TOKENS and k % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.stride(1) == 1 and x.stride(1) == 1
            and w.stride(1) == 1 and -(-w.shape[0] // 128) <= GEMM_MAX_TICKETS)


def _library_mm(x, w, out) -> None:
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    else:
        _need(out.dtype == torch.float32, "linear: out must be bfloat16 or float32")
        try:
            torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
        except (TypeError, RuntimeError):
            out.copy_(torch.mm(x, w.t(), out_dtype=torch.float32))


TOKEN_BUCKETS = ((16, 8), (32, 32), (64, 64), (128, 128))      # (bucket, token count it is measured at)


def time_in_graph(fn, reps: int = 8) -> float:
    """Microseconds per call of ``fn(i)``: ``reps`` calls are captured into a CUDA graph and the graph
    is replayed, so that the host's launch cost stays out of the figure."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(2):
            fn(i)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(reps):
                fn(i)
        graph.replay()
        side.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        graph.replay()
        e1.record()
        side.synchronize()
    torch.cuda.current_stream().wait_stream(side)
    return e0.elapsed_time(e1) * 1e3 / (2 * reps)


def measure_linear(weights, out_dtype=torch.bfloat16, gated: int = 0):
    """{bucket: (microseconds of this library's tcgen05 product, of the library's)} for one shape of
    weight matrix.  ``weights``: matrices of the same shape (the same projection of several layers),
    used in rotation so that the L2 cache cannot serve them; their tiled images must exist.
    ``gated`` > 0: the matrices are gate-and-up matrices with gated images; this library's side is
    ``linear_gated``, the library's side the product followed by the activation kernel.
    Buckets the tcgen05 kernel cannot take are left out."""
    n, k = weights[0].shape
    dev_ = weights[0].device
    out_times = {}
    for bucket, m in TOKEN_BUCKETS:
        x = torch.randn(m, k, device=dev_).to(torch.bfloat16)
        out = torch.empty(m, n, dtype=out_dtype, device=dev_)
        if not _tcgen05_ok(x, weights[0], out):
            continue
        if gated:
            act = torch.empty(m, gated, dtype=out_dtype, device=dev_)

            def theirs(i):
                _library_mm(x, weights[i % len(weights)], out)
                silu_mul(out, act)
            out_times[bucket] = (time_in_graph(lambda i: gemm_bf16_tcgen05(x, weights[i % len(weights)], act, gated=True)),
                                 time_in_graph(theirs))
        else:
            out_times[bucket] = (time_in_graph(lambda i: gemm_bf16_tcgen05(x, weights[i % len(weights)], out)),
                                 time_in_graph(lambda i: _library_mm(x, weights[i % len(weights)], out)))
    check_status()
    return out_times


def measure_layer(products, hidden: int, fusable_norms: int, dtype=torch.bfloat16) -> dict:
    """{bucket: (microseconds of a layer's products as this library runs them, as the library would)}.
    ``products``: for every product of a layer, in the order they run, (matrices of that product
    across layers, gated, reads a norm's output, ends a residual branch) with tiled images made.  This
    library's side is its tcgen05 product for each, linked as the blocks link them: the rows' factor
    applied by a product that reads a norm's output (RowScale), the addition into the residual stream,
    the next norm's gain and the sums of squares in the epilogue of one that ends a branch
    (ResidualNorm), the activation inside the gated ones.  The library's side is a product each, the
    activation kernel after a gated one and ``fusable_norms`` norm kernels, which the other side does
    not need."""
    dev_ = products[0][0][0].device
    times = {}
    for bucket, m in TOKEN_BUCKETS:
        xs, outs, acts = {}, [], []
        ok = True
        for mats, gated, _, _ in products:
            n, k = mats[0].shape
            if k not in xs:
                xs[k] = torch.randn(m, k, device=dev_).to(dtype)
            outs.append(torch.empty(m, n, dtype=dtype, device=dev_))
            acts.append(torch.empty(m, gated, dtype=dtype, device=dev_) if gated else None)
            ok = ok and _tcgen05_ok(xs[k], mats[0], outs[-1])
        if not ok:
            continue
        res = torch.zeros(m, hidden, device=dev_)
        delta = torch.zeros(m, hidden, dtype=dtype, device=dev_)
        normed = torch.empty(m, hidden, dtype=dtype, device=dev_)
        gain = torch.ones(hidden, device=dev_)
        sumsq = torch.ones(sumsq_parts(hidden), m, device=dev_)
        scale = RowScale(sumsq, sumsq_parts(hidden), hidden, 1e-6)
        ends = ResidualNorm(res, gain, torch.empty(sumsq_parts(hidden), m, device=dev_), 1e-6)

        def ours(i):
            for j, (mats, gated, reads_norm, ends_branch) in enumerate(products):
                w = mats[i % len(mats)]
                gemm_bf16_tcgen05(xs[w.shape[1]], w, acts[j] if gated else outs[j],
                                  x_scale=scale if reads_norm and w.shape[1] == hidden else None,
                                  fuse=ends if ends_branch and w.shape[0] == hidden and not gated else None, gated=bool(gated))

        def theirs(i):
            for j, (mats, gated, _, _) in enumerate(products):
                w = mats[i % len(mats)]
                _library_mm(xs[w.shape[1]], w, outs[j])
                if gated:
                    silu_mul(outs[j], acts[j])
            for _ in range(fusable_norms):
                add_rmsnorm(res, delta, gain, normed, 1e-6)

        times[bucket] = (time_in_graph(ours), time_in_graph(theirs))
    check_status()
    return times


# (features, k, tile columns, gated, ends a residual branch) -> persistent CTAs of the tcgen05 product, where a
# measurement chose them
_cta_choice = {}


def cta_candidates(features: int, k: int, gated: int = 0):
    """Grid sizes worth measuring for a few-token product: one CTA per SM (the next kernel's CTAs then sit
    beside this one's and prefetch), two per SM, and in between the counts that cut every 128-row tile into
    the same number of whole runs of k slabs (no CTA then holds pieces of two tiles, and a count equal to the
    number of tiles needs no merge at all)."""
    sms = sm_count()
    tiles = -(-gated // 64) if gated else -(-features // 128)
    slabs = -(-k // 64)
    out = {sms, 2 * sms}
    for per_tile in range(1, slabs // 4 + 1):
        if slabs % per_tile == 0 and sms * 3 // 4 <= tiles * per_tile <= 2 * sms:
            out.add(tiles * per_tile)
    return sorted(out)


def choose_ctas(weights, bucket: int, tokens: int, gated: int = 0, out_dtype=torch.bfloat16, residual: bool = False) -> int:
    """Measure the tcgen05 product on ``weights`` (matrices of one shape, used in rotation) at every candidate
    grid size, record the fastest for this shape and bucket, and return it.  ``residual``: the product as it
    ends a residual branch (ResidualNorm), whose merge does more than the plain one's."""
    n, k = weights[0].shape
    dev_ = weights[0].device
    x = torch.randn(tokens, k, device=dev_).to(torch.bfloat16)
    out = torch.empty(tokens, gated or n, dtype=out_dtype, device=dev_)
    fuse = ResidualNorm(torch.zeros(tokens, n, device=dev_), torch.ones(n, device=dev_),
                        torch.empty(sumsq_parts(n), tokens, device=dev_), 1e-6) if residual else None
    best, best_t = None, None
    for ctas in cta_candidates(n, k, gated):
        t = time_in_graph(lambda i: gemm_bf16_tcgen05(x, weights[i % len(weights)], out, max_ctas=ctas, gated=bool(gated), fuse=fuse))
        if best_t is None or t < best_t * 0.98:           # a larger grid must win by more than the noise
            best, best_t = ctas, t
    _cta_choice[(n, k, tcgen05_plan(tokens, n, k)[1], bool(gated), residual)] = best
    return best


def choose_linear(features: int, k: int, bucket: int, out_dtype, tcgen05: bool) -> None:
    """Record which product ``linear`` runs for this shape and bucket of token counts."""
    _linear_choice[(features, k, bucket, out_dtype)] = bool(tcgen05)


def forget_choices(features: int, k: int) -> None:
    """Drop what was measured for products of this shape (kernel per bucket, grid per tile width): the defaults
    apply again."""
    for key in [key for key in _linear_choice if key[0] == features and key[1] == k]:
        del _linear_choice[key]
    for key in [key for key in _cta_choice if key[0] == features and key[1] == k]:
        del _cta_choice[key]


def linear_tuning() -> bool:
    return _linear_tuning


_norm_fusion = True


def set_norm_fusion(on: bool) -> None:
    """Allow products to take over the norms around them (default), or run every norm as a kernel."""
    global _norm_fusion
    _norm_fusion = bool(on)


def linear_fuses_norm(tokens: int, w: torch.Tensor, out_dtype=torch.bfloat16) -> bool:
    """True if ``linear`` will run this library's tcgen05 product for ``tokens`` rows against ``w``
    (taken contiguous and 16-byte aligned, as workspace buffers and loaded weights are): only then can
    it apply a RowScale or a ResidualNorm."""
    return (_norm_fusion and _tcgen05_linear and w.dtype == torch.bfloat16 and 0 < tokens <= TCGEN05_MAX_TOKENS
            and w.shape[1] % 8 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0
            and -(-w.shape[0] // 128) <= GEMM_MAX_TICKETS
            and _linear_choice.get((w.shape[0], w.shape[1], token_bucket(tokens), out_dtype), True))


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, x_scale: Optional[RowScale] = None,
           fuse: Optional[ResidualNorm] = None) -> None:
    """out = x @ w^T.  float32: the engine's own FMA kernel.  bfloat16 with up to TCGEN05_MAX_TOKENS
    rows (decode steps, short portions): the engine's tcgen05 + TMA kernel with the weights on the
    128-row side of the tile, where the measurement at load found it faster than the library (and always
    when nothing was measured); otherwise the library product (cuBLAS through torch.mm, float
    accumulation).  out is bfloat16 or float32.  ``x_scale`` / ``fuse`` may be given only where
    ``linear_fuses_norm`` said yes."""
    if x.dtype == torch.float32:
        _need(x_scale is None and fuse is None, "linear: the float32 product fuses no norm")
        gemm_f32(x, w, out)
        return
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear: operands must both be bfloat16")
    if _tcgen05_linear and _tcgen05_ok(x, w, out) and \
            _linear_choice.get((w.shape[0], w.shape[1], token_bucket(x.shape[0]), out.dtype), True):
        gemm_bf16_tcgen05(x, w, out, x_scale=x_scale, fuse=fuse)
        return
    _need(x_scale is None and fuse is None, "linear: the library product fuses no norm; ask linear_fuses_norm first")
    _library_mm(x, w, out)


def linear_gated_fuses(tokens: int, w: torch.Tensor) -> bool:
    """True if ``linear_gated`` will run as one kernel (this library's tcgen05 product on a gated tile image)."""
    return tiled_weights_of(w, gated=True) is not None and _tcgen05_linear and 0 < tokens <= TCGEN05_MAX_TOKENS \
        and _linear_choice.get((w.shape[0], w.shape[1], token_bucket(tokens), torch.bfloat16), True)


def linear_gated(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, x_scale: Optional[RowScale] = None) -> None:
    """out [tokens, inter] = silu(x gate^T) * (x up^T) for w = [gate; up] ([2 * inter, k]) in one kernel;
    only where ``linear_gated_fuses`` said yes."""
    _need(linear_gated_fuses(x.shape[0], w), "linear_gated: ask linear_gated_fuses first")
    gemm_bf16_tcgen05(x, w, out, x_scale=x_scale, gated=True)


def random_normal(out: torch.Tensor, key: int, mean: float, std: float, first: int = 0) -> None:
    """out.flatten()[i] = mean + std * normal(key, first + i), rounded to out's type: the counter-based
    generator of the random-weights mode (csrc/random_init.cu; weights/random_init.py has it in numpy)."""
    _check(lib().vcb_random_normal(_dev(out, "out"), out.numel(), int(first), int(key) & ((1 << 64) - 1),
                                   float(mean), float(std), dtype_code(out.dtype), _stream()), "random_normal")


def repetition_penalty(logits, ids, row_start, penalty) -> None:
    n, vocab = logits.shape
    _check(lib().vcb_repetition_penalty(_dev(logits, "logits", torch.float32), logits.stride(0),
                                        _dev(ids, "ids", torch.int32), _dev(row_start, "row_start", torch.int32),
                                        _dev(penalty, "penalty", torch.float32), n, vocab, _stream()),
           "repetition_penalty")


def sample(logits, temperature, uniform, out) -> None:
    """out[r] = argmax (temperature <= 0) or an inverse-CDF draw with uniform[r] in id order."""
    n, vocab = logits.shape
    _need(logits.is_cuda and logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 rows")
    _check(lib().vcb_sample(logits.data_ptr(), logits.stride(0), vocab, _dev(temperature, "temperature", torch.float32),
                            _dev(uniform, "uniform", torch.float32), _dev(out, "out", torch.int32), n, _stream()),
           "sample")


_filter_scratch: Optional[torch.Tensor] = None


def sample_filtered(logits, temperature, uniform, top_p, top_k, out, scratch: Optional[torch.Tensor] = None) -> None:
    """Redraws, in place in ``out``, the rows that have top-k or top-p set (see sampling.cu).
    ``scratch``: float32, at least rows * vocab elements; one is kept and grown here if not given."""
    global _filter_scratch
    n, vocab = logits.shape
    _need(logits.is_cuda and logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 rows")
    _need(vocab <= 1 << 20, f"top-k/top-p sampling takes vocabularies up to {1 << 20}, got {vocab}")
    if scratch is None:
        if _filter_scratch is None or _filter_scratch.numel() < n * vocab or _filter_scratch.device != logits.device:
            _filter_scratch = torch.empty(n * vocab, dtype=torch.float32, device=logits.device)
        scratch = _filter_scratch
    _need(scratch.numel() >= n * vocab, "sample_filtered: scratch too small")
    _check(lib().vcb_sample_filtered(logits.data_ptr(), logits.stride(0), vocab,
                                     _dev(temperature, "temperature", torch.float32),
                                     _dev(uniform, "uniform", torch.float32), _dev(top_p, "top_p", torch.float32),
                                     _dev(top_k, "top_k", torch.int32), _dev(scratch, "scratch", torch.float32),
                                     _dev(out, "out", torch.int32), n, _stream()), "sample_filtered")


_scratch = {}
_scratch_epoch = 0


def scratch_epoch() -> int:
    """Changes whenever a scratch buffer moves; captured CUDA graphs that used one are stale then."""
    return _scratch_epoch


def zeroed_ints(name: str, numel: int, device) -> torch.Tensor:
    """An int32 device buffer of at least ``numel`` zeros, kept under ``name``.  Kernels that
    count tickets in it leave it zero again."""
    t = _scratch.get(name)
    if t is None or t.numel() < numel or t.device != torch.device(device):
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"scratch buffer {name!r} must be sized before a CUDA graph is captured")
        t = torch.zeros(max(numel, 1024), dtype=torch.int32, device=device)
        _scratch[name] = t
        global _scratch_epoch
        _scratch_epoch += 1
    return t


def scratch(name: str, numel: int, device) -> torch.Tensor:
    """A float32 device buffer of at least ``numel`` elements, kept under ``name`` and grown
    when needed.  Kernels that merge partial results through global memory use it."""
    t = _scratch.get(name)
    if t is None or t.numel() < numel or t.device != torch.device(device):
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"scratch buffer {name!r} must be sized before a CUDA graph is captured")
        t = torch.empty(max(numel, 1024), dtype=torch.float32, device=device)
        _scratch[name] = t
        global _scratch_epoch
        _scratch_epoch += 1
    return t
