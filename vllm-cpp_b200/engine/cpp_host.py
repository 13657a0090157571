"""The C++ host runtime (src/, include/vllm/vllm.hpp) driven from Python through its C face.

``CppEngine`` has the calls of ``vllm::Engine``: ``add_request``, ``step``, ``run``-like ``generate``,
``abort_request``, and ``step_tokens`` for explicit batches.  It exists so that the two hosts can be set side by
side (tests run one workload through both and compare the token ids) and so that a Python program can use the
C++ scheduler, cache manager and forward pass without a compiler at hand.  The library is built on first use
beside the kernel library (csrc/build.py).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np

from ..csrc import build as _build

_lib = None


class CppEngineError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        _build.load()                                   # the kernels first: the engine links against them
        l = ctypes.CDLL(_build.build_engine()["lib"])
        P, I, F, L, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_ulonglong
        C = ctypes.c_char_p
        l.vcbe_last_error.restype = C
        l.vcbe_create.argtypes, l.vcbe_create.restype = [C, C, C, I, I, I, I, I, I, U, I, I, I, C], P
        l.vcbe_destroy.argtypes = [P]
        l.vcbe_add_request.argtypes, l.vcbe_add_request.restype = [P, P, I, I, F, F, I, F, I, U, I, P, I], L
        l.vcbe_step.argtypes, l.vcbe_step.restype = [P, P, P, P, I], I
        l.vcbe_has_pending_work.argtypes, l.vcbe_has_pending_work.restype = [P], I
        l.vcbe_abort_request.argtypes = [P, L]
        l.vcbe_step_tokens.argtypes, l.vcbe_step_tokens.restype = [P, I, P, P, P, P, P, P, L], I
        l.vcbe_release.argtypes = [P, L]
        for name in ("vcbe_num_free_blocks", "vcbe_num_total_blocks", "vcbe_num_preemptions", "vcbe_pool_total_bytes",
                     "vcbe_pool_used_bytes"):
            getattr(l, name).argtypes, getattr(l, name).restype = [P], L
        l.vcbe_vocab_size.argtypes, l.vcbe_vocab_size.restype = [P], I
        _lib = l
    return _lib


def _ints(values) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(list(values), dtype=np.int32))


class CppEngine:
    def __init__(self, model_path: str, dtype: str = "bfloat16", model_arch: str = "", block_size: int = 16,
                 num_gpu_blocks: int = 0, max_num_seqs: int = 64, max_model_len: int = 8192,
                 max_num_batched_tokens: int = 16384, max_tokens_per_step: int = 512, seed: int = 0,
                 gpu_memory_utilization: int = 90, preempted_to_front: bool = False, fused_decode_tokens: int = 64,
                 load_format: str = "safetensors"):
        """``load_format``: "random" fills the weights from ``seed`` (the tensors ``write_random_model`` would
        store for it); ``model_path`` then needs config.json only."""
        self._l = lib()
        self._h = self._l.vcbe_create(model_path.encode(), model_arch.encode(), dtype.encode(), block_size, num_gpu_blocks,
                                      max_num_seqs, max_model_len, max_num_batched_tokens, max_tokens_per_step, seed,
                                      gpu_memory_utilization, 1 if preempted_to_front else 0, fused_decode_tokens,
                                      load_format.encode())
        if not self._h:
            raise CppEngineError(self._l.vcbe_last_error().decode())
        self.max_num_seqs = max_num_seqs
        self.vocab = self._l.vcbe_vocab_size(self._h)

    def close(self):
        if self._h:
            self._l.vcbe_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def _fail(self):
        raise CppEngineError(self._l.vcbe_last_error().decode())

    def add_request(self, prompt: Sequence[int], max_tokens: int = 64, temperature: float = -1.0, top_p: float = -1.0,
                    top_k: int = 0, repetition_penalty: float = -1.0, seed: Optional[int] = None, ignore_eos: bool = False,
                    stop_token_ids: Optional[Sequence[int]] = None) -> int:
        ids = _ints(prompt)
        stops = _ints(stop_token_ids or [])
        rid = self._l.vcbe_add_request(self._h, ids.ctypes.data, len(ids), max_tokens, temperature, top_p, top_k,
                                       repetition_penalty, 0 if seed is None else 1, seed or 0, 1 if ignore_eos else 0,
                                       stops.ctypes.data, -1 if stop_token_ids is None else len(stops))
        if rid < 0:
            self._fail()
        return rid

    def step(self) -> List[Tuple[int, int, Optional[str]]]:
        """[(request, new token, None or 'stop' or 'length')]."""
        cap = self.max_num_seqs
        ids, toks, fin = (np.empty(cap, dtype=np.int64), np.empty(cap, dtype=np.int32), np.empty(cap, dtype=np.int32))
        n = self._l.vcbe_step(self._h, ids.ctypes.data, toks.ctypes.data, fin.ctypes.data, cap)
        if n < 0:
            self._fail()
        return [(int(ids[i]), int(toks[i]), (None, "stop", "length")[fin[i]]) for i in range(n)]

    def has_pending_work(self) -> bool:
        return bool(self._l.vcbe_has_pending_work(self._h))

    def abort_request(self, rid: int) -> None:
        self._l.vcbe_abort_request(self._h, rid)

    def generate(self, prompts, **params) -> List[List[int]]:
        """All prompts at once under the scheduler; ``params`` as add_request's, or a list of dicts, one per prompt."""
        per = params.pop("per_request", None)
        rids = [self.add_request(p, **(per[i] if per else params)) for i, p in enumerate(prompts)]
        out = {r: [] for r in rids}
        while self.has_pending_work():
            for rid, tok, _ in self.step():
                out[rid].append(tok)
        return [out[r] for r in rids]

    def step_tokens(self, entries) -> np.ndarray:
        """entries: [(request id >= 0, tokens, wanted places)] -> float32 logits [wanted, vocab]."""
        req = np.ascontiguousarray([e[0] for e in entries], dtype=np.int64)
        counts, wcounts = _ints(len(e[1]) for e in entries), _ints(len(e[2]) for e in entries)
        toks, want = _ints(t for e in entries for t in e[1]), _ints(w for e in entries for w in e[2])
        out = np.empty((max(1, int(wcounts.sum())), self.vocab), dtype=np.float32)
        rows = self._l.vcbe_step_tokens(self._h, len(entries), req.ctypes.data, counts.ctypes.data, toks.ctypes.data,
                                        wcounts.ctypes.data, want.ctypes.data, out.ctypes.data, out.size)
        if rows < 0:
            self._fail()
        return out[:rows]

    def release(self, rid: int) -> None:
        self._l.vcbe_release(self._h, rid)

    num_free_blocks = property(lambda self: self._l.vcbe_num_free_blocks(self._h))
    num_total_blocks = property(lambda self: self._l.vcbe_num_total_blocks(self._h))
    num_preemptions = property(lambda self: self._l.vcbe_num_preemptions(self._h))
    pool_total_bytes = property(lambda self: self._l.vcbe_pool_total_bytes(self._h))
    pool_used_bytes = property(lambda self: self._l.vcbe_pool_used_bytes(self._h))
