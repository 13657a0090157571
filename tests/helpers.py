"""Shared by the tests: the tiny configurations, model folders, traces and comparisons.

The tiny configurations differ in every size and option: head counts and groups,
head size, widths that are no power of two, depth, vocabulary (one of them odd),
rope_theta, the norms' eps, tying, the window, the page size.
"""
from __future__ import annotations

import os
import tempfile

import numpy as np

import plain_qwen2 as plain

TINY_A = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 64,
          "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2,
          "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
          "tie_word_embeddings": True, "use_sliding_window": False, "max_position_embeddings": 256,
          "hidden_act": "silu"}
TINY_B = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 96,
          "num_hidden_layers": 3, "num_attention_heads": 3, "num_key_value_heads": 1,
          "intermediate_size": 224, "vocab_size": 384, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
          "tie_word_embeddings": False, "use_sliding_window": False, "max_position_embeddings": 512,
          "hidden_act": "silu"}
# windowed upper layers, full multi-head attention, widths with odd factors, an odd vocabulary
TINY_C = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 80,
          "num_hidden_layers": 4, "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 16,
          "intermediate_size": 176, "vocab_size": 301, "rope_theta": 500000.0, "rms_norm_eps": 3e-6,
          "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 24,
          "max_window_layers": 2, "max_position_embeddings": 384, "hidden_act": "silu"}
# head size given apart from the width (heads * head_dim != hidden_size), head size 64
TINY_D = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 72,
          "num_hidden_layers": 2, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64,
          "intermediate_size": 200, "vocab_size": 272, "rope_theta": 20000.0, "rms_norm_eps": 1e-5,
          "tie_word_embeddings": True, "use_sliding_window": False, "max_position_embeddings": 320,
          "hidden_act": "silu"}

# head size 128 (the tcgen05 prefill attention and the widest decode tiles), one query group of two
# heads, the second layer windowed
TINY_E = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 88,
          "num_hidden_layers": 2, "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 128,
          "intermediate_size": 136, "vocab_size": 264, "rope_theta": 50000.0, "rms_norm_eps": 2e-6,
          "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 70,
          "max_window_layers": 1, "max_position_embeddings": 400, "hidden_act": "silu"}

# The models whose logits the reference itself can anchor (tests/golden/make_reference_logits.py): tied
# embeddings and eps 1e-6 only.  The second has the sizes of B: three heads on one kv head, widths that are
# no power of two, another theta.
GOLDEN_CONFIGS = {"A": TINY_A, "B_tied": dict(TINY_B, tie_word_embeddings=True, rms_norm_eps=1e-6)}
GOLDEN_PROMPTS = (5, 17, 33)

CONFIGS = {"A": (TINY_A, 16), "B": (TINY_B, 32), "C": (TINY_C, 16), "D": (TINY_D, 32), "E": (TINY_E, 16)}   # name -> (config, page size)

def random_config(rng):
    """A Qwen2 configuration drawn at random: head sizes in steps of 16, any number of heads and groups, widths
    and vocabularies with odd factors, a head size given apart from the width or not, windows on some layers."""
    d = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128]))
    heads = int(rng.integers(1, 9))
    kv = int(rng.choice([k for k in range(1, heads + 1) if heads % k == 0]))
    layers = int(rng.integers(1, 5))
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": layers,
           "num_attention_heads": heads, "num_key_value_heads": kv,
           "intermediate_size": int(rng.integers(40, 300)), "vocab_size": int(rng.integers(60, 2000)),
           "rope_theta": float(rng.choice([1e4, 1e6, 5e5, 123456.0])), "rms_norm_eps": float(rng.choice([1e-5, 1e-6, 3e-6])),
           "tie_word_embeddings": bool(rng.integers(0, 2)), "max_position_embeddings": int(rng.integers(256, 600)),
           "hidden_act": "silu"}
    if rng.random() < 0.4:
        cfg["hidden_size"] = heads * d
        if rng.random() < 0.5:
            cfg["head_dim"] = d
    else:
        cfg["hidden_size"] = int(rng.integers(24, 220))
        cfg["head_dim"] = d
    if rng.random() < 0.5:
        cfg.update(use_sliding_window=True, sliding_window=int(rng.integers(8, 100)),
                   max_window_layers=int(rng.integers(0, layers + 1)))
    else:
        cfg["use_sliding_window"] = False
    return cfg


# |engine - plain| <= TOL * max|plain| over the compared rows
TOL = {"float32": 1e-4, "bfloat16": 3e-2}
MEAN_TOL = {"float32": 2e-5, "bfloat16": 6e-3}


def make_weights(cfg, seed, dtype, sharp=None):
    """Weights as the plain implementation will use them (bfloat16 runs: rounded to bfloat16)."""
    if sharp is None:
        # q and k scaled up so that attention is peaked and one wrong key shows;
        # less so in bfloat16, where rounding of large scores is itself visible
        # The scores' standard deviation is (std * sharp)^2 * hidden; aim at 5 in
        # 32-bit (a few keys carry nearly all the weight) and at 1.5 in bfloat16.
        target = 5.0 if dtype == "float32" else 1.5
        sharp = float(np.sqrt(target / cfg["hidden_size"]) / 0.08)
    w = plain.random_weights(cfg, seed, std=0.08, gain_std=0.1, sharp=sharp)
    return plain.round_to_bf16(w) if dtype == "bfloat16" else w


def model_folder(tmp_path, cfg, weights, dtype):
    d = os.path.join(str(tmp_path), f"model_{abs(hash(str(sorted(cfg.items())))) % 10**8}_{dtype}")
    plain.write_model_folder(d, cfg, weights, store="BF16" if dtype == "bfloat16" else "F32")
    return d


def token_ids(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab_size"], size=n).tolist()


def compare(got, want, dtype, what=""):
    """got, want: [rows, vocab]."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shapes {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: engine logits are not finite"
    scale = np.abs(want).max()
    err = np.abs(got - want)
    worst = np.unravel_index(err.argmax(), err.shape)
    assert err.max() <= TOL[dtype] * scale, (
        f"{what}: max |diff| {err.max():.3e} at row {worst[0]} col {worst[1]} exceeds "
        f"{TOL[dtype]:.0e} * {scale:.3e}; first bad row "
        f"{int(np.argmax(err.max(axis=1) > TOL[dtype] * scale))}")
    assert err.mean() <= MEAN_TOL[dtype] * scale, f"{what}: mean |diff| {err.mean():.3e} vs scale {scale:.3e}"


class Replayer:
    """Drives a ModelRunner like the replay tool does and collects logits by (request, position)."""

    def __init__(self, runner, cache):
        self.runner, self.cache = runner, cache
        self.fed = {}
        self.rows = {}

    def step(self, entries, end=()):
        """entries: list of (request id, tokens, want places)."""
        from vllm_cpp_b200.engine.runner import StepEntry
        batch = []
        for rid, toks, want in entries:
            if rid not in self.cache.requests:
                self.cache.add_request(rid)
                self.fed[rid] = 0
            batch.append(StepEntry(rid, list(toks), list(want)))
        logits = self.runner.step(batch).float().cpu().numpy()
        i = 0
        for rid, toks, want in entries:
            for w in want:
                self.rows[(rid, self.fed[rid] + w)] = logits[i].copy()
                i += 1
            self.fed[rid] += len(toks)
        for rid in end:
            self.cache.free_request(rid)
            del self.fed[rid]

    def logits_of(self, rid, positions):
        return np.stack([self.rows[(rid, p)] for p in positions])


def kv_pos(d, esize, slot, page):
    """Where the elements of slot ``slot`` lie inside a (page, k|v, kv head) block of page * d elements
    (the layout the engine documents in csrc/common.cuh): rows that are a multiple of 128 bytes are
    stored in planes of 128-byte pieces, [plane][slot][piece], with the 16-byte chunks of a piece
    XOR-swizzled by the slot number; other rows as they are.  block.ravel()[kv_pos(...)] = the row."""
    e = np.arange(d)
    if (d * esize) % 128:
        return slot * d + e
    per_plane, per_chunk = 128 // esize, 16 // esize
    plane, w = e // per_plane, e % per_plane
    return plane * (page * per_plane) + slot * per_plane + ((w // per_chunk) ^ (slot & 7)) * per_chunk + w % per_chunk
