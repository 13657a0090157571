"""Plain implementation of the Qwen2 decoder, the scheduler-free oracle of the tests.

Whole sequences, no cache, one function per part, numpy only.  It shares no code
with the engine: it has its own safetensors reader and writer, its own rotation
table, its own sampler.  Every function is written from the formulas of
jiamumuzhao/vllm-cpp and cites the file and lines it follows.

It is written from the formulas.  The reference's model code (src/model/qwen.cpp,
src/layers/*.cpp) calls the CUDA runtime and cuBLAS in every layer and has no CPU
forward, so it cannot run on a CPU-only machine; built on a GPU machine it gave the
logits of two tiny tied models token by token, and those are kept under tests/golden/
(reference_logits.npz, made by make_reference_logits.py) and compared with
``forward`` here in tests/test_plain.py.  Its host-only sampler helpers run anywhere;
their outputs for a few small inputs are kept there too, with the program that made
them.

Arithmetic is float64 unless ``dtype`` says otherwise, so that it judges the
engine's float32 path as well as its bfloat16 path.  One thing is kept in float32
on purpose: the rotation angle, which the reference computes as
``pos / powf(theta, 2i/d)`` in float (src/model/qwen.cpp:119-128); an angle in
float64 would differ from any float32 engine by more than rounding at large
positions.

Where the reference's code has a fault, the formula follows what it evidently
means: eps comes from the configuration (the reference passes 1e-6 whatever the
model says, src/model/qwen.cpp:303,312,322), a causal mask is applied (the
reference feeds one token per call and so needs none,
src/attention/paged_attention.cu:20-21), and an untied lm_head is a matrix of its
own (the reference copies it over the embedding table, src/model/qwen.cpp:279-281).
A window (config.json's use_sliding_window, sliding_window, max_window_layers),
which the reference does not read, lets a query at position p see keys j with
p - window < j <= p in layers at or above max_window_layers.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np


# ------------------------------------------------------------------ parts
def embedding(ids, table):
    """out[t, :] = table[ids[t], :], no scaling  (src/kernels/embedding_kernel.cu:20-28)."""
    return table[np.asarray(ids, dtype=np.int64)]


def rms_norm(x, weight, eps):
    """y_i = (x_i * rsqrt(mean_j x_j^2 + eps)) * w_i  (src/kernels/layernorm.cu:20-23,41,48)."""
    r = 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return (x * r) * weight


# The type the operands of every product are rounded through, or None.  The reference rounds both the
# weights (src/layers/linear.cpp:38-42) and the inputs (:67, launch_f32_to_fp16) to half precision and
# accumulates in float; ``forward(..., operand=np.float16)`` restates that, for the comparison with
# logits the reference itself produced (tests/golden/).
_OPERAND = None


def linear(x, weight, bias=None):
    """out[t, o] = sum_i W[o, i] x[t, i] (+ bias[o]); W is [out, in]
    (src/layers/linear.cpp:70-77 computes it through cuBLAS, :84-86 adds the bias)."""
    if _OPERAND is not None:
        x, weight = x.astype(_OPERAND).astype(x.dtype), weight.astype(_OPERAND).astype(weight.dtype)
    y = x @ weight.T
    return y if bias is None else y + bias


def rope_angles(positions, theta, rotary_dim):
    """angle[p, i] = p / powf(theta, 2i / d) in float32, i < d/2  (src/model/qwen.cpp:119-128)."""
    i = np.arange(rotary_dim // 2, dtype=np.float32)
    denom = np.power(np.float32(theta), (np.float32(2.0) * i) / np.float32(rotary_dim)).astype(np.float32)
    return np.asarray(positions, dtype=np.float32)[:, None] / denom[None, :]


def rope(x, positions, theta, rotary_dim=None):
    """Rotate-half rotation of x [T, heads, d] (src/kernels/rotary_embedding.cu:18-33):
    x'_i = x_i cos - x_{i+d/2} sin;  x'_{i+d/2} = x_i sin + x_{i+d/2} cos."""
    d = x.shape[-1]
    rd = d if rotary_dim is None else rotary_dim
    ang = rope_angles(positions, theta, rd).astype(x.dtype)
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    a, b = x[..., : rd // 2], x[..., rd // 2: rd]
    out[..., : rd // 2] = a * cos - b * sin
    out[..., rd // 2: rd] = a * sin + b * cos
    return out


def attention(q, k, v, num_heads, num_kv_heads, window=0):
    """Causal grouped-query attention over a whole sequence.
    q: [T, nh, d], k and v: [T, nkv, d].  Head h reads kv head h // (nh / nkv)
    (src/attention/paged_attention.cu:19); score = (q . k) / sqrt(d)
    (src/layers/attention.cpp:126); softmax over the visible keys
    (paged_attention.cu:48-51,75); out = sum_j w_j v_j (:76-79)."""
    t, _, d = q.shape
    group = num_heads // num_kv_heads
    scale = 1.0 / np.sqrt(np.float32(d)).astype(q.dtype)
    pos = np.arange(t)
    visible = pos[None, :] <= pos[:, None]
    if window > 0:
        visible &= pos[None, :] > pos[:, None] - window
    out = np.empty_like(q)
    for h in range(num_heads):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = np.where(visible, s, -np.inf)
        m = s.max(axis=-1, keepdims=True)
        e = np.exp(s - m)
        w = e / e.sum(axis=-1, keepdims=True)
        out[:, h, :] = w @ v[:, g, :]
    return out


def silu(z):
    """z / (1 + exp(-z))  (src/kernels/activation.cu:8-10)."""
    return z / (1.0 + np.exp(-z))


def swiglu_mlp(x, w_gate, w_up, w_down):
    """down( silu(gate(x)) * up(x) ), no biases  (src/layers/mlp.cpp:49-64, activation.cu:34-39)."""
    return linear(silu(linear(x, w_gate)) * linear(x, w_up), w_down)


def attention_block(x, positions, w, prefix, cfg, window):
    """q/k/v with bias, rotation of q and k, attention, output projection without bias
    (src/layers/attention.cpp:74-79,126-134; bias flags :19-22)."""
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // nh
    t = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"], w[prefix + "q_proj.bias"]).reshape(t, nh, d)
    k = linear(x, w[prefix + "k_proj.weight"], w[prefix + "k_proj.bias"]).reshape(t, nkv, d)
    v = linear(x, w[prefix + "v_proj.weight"], w[prefix + "v_proj.bias"]).reshape(t, nkv, d)
    q = rope(q, positions, cfg["rope_theta"])
    k = rope(k, positions, cfg["rope_theta"])
    o = attention(q, k, v, nh, nkv, window).reshape(t, nh * d)
    return linear(o, w[prefix + "o_proj.weight"])


def layer_window(cfg, layer):
    if cfg.get("use_sliding_window", False) and layer >= cfg.get("max_window_layers", 0):
        return int(cfg["sliding_window"])
    return 0


def forward(weights, cfg, ids, dtype=np.float64, operand=None, rows=None):
    """Logits [T, vocab] of a whole sequence  (src/model/qwen.cpp:291-328):
    embedding, then per layer  x += attn(norm(x));  x += mlp(norm(x)),  final norm, lm_head.
    ``operand``: see _OPERAND above (the embedding table is stored in that type too,
    src/layers/embedding.cpp:27-31).  ``rows``: positions whose logits are returned ([len(rows), vocab];
    with a vocabulary of 150,000 the output product of every position is most of the work)."""
    global _OPERAND
    _OPERAND = operand
    try:
        return _forward(weights, cfg, ids, dtype, operand, rows)
    finally:
        _OPERAND = None


def _forward(weights, cfg, ids, dtype, operand, rows=None):
    w = {k: (v if isinstance(v, np.ndarray) and v.dtype == dtype else np.asarray(v, dtype=dtype)) for k, v in weights.items()}
    if operand is not None:
        e = "model.embed_tokens.weight"
        w[e] = w[e].astype(operand).astype(dtype)
    eps = cfg.get("rms_norm_eps", 1e-6)
    positions = np.arange(len(ids))
    x = embedding(ids, w["model.embed_tokens.weight"])
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
        x = x + attention_block(h, positions, w, p + "self_attn.", cfg, layer_window(cfg, l))
        h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                           w[p + "mlp.down_proj.weight"])
    if rows is not None:
        x = x[np.asarray(rows, dtype=np.int64)]
    x = rms_norm(x, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(x, head)


# --------------------------------------------------------------- sampling
def greedy(logits):
    """First largest value  (src/sampler/sampler.cpp:11-21)."""
    best, best_val = 0, logits[0]
    for i in range(1, len(logits)):
        if logits[i] > best_val:
            best, best_val = i, logits[i]
    return best


def repetition_penalty(logits, prev_tokens, penalty):
    """Each generated id once: l > 0 ? l / p : l * p  (src/sampler/sampler.cpp:81-92)."""
    out = np.array(logits, dtype=np.float32)
    seen = set()
    for t in prev_tokens:
        if 0 <= t < len(out) and t not in seen:
            seen.add(t)
            out[t] = out[t] / np.float32(penalty) if out[t] > 0 else out[t] * np.float32(penalty)
    return out


def softmax(x):
    """exp(x - max) / sum  (src/sampler/topk_topp.cpp:37-47), float32."""
    e = np.exp((x - x.max()).astype(np.float32)).astype(np.float32)
    return e / e.sum(dtype=np.float32)


def order_by_probability(probs, indices):
    """Falling probability, ties by lower id  (src/sampler/topk_topp.cpp:10-12,21-23)."""
    return sorted(indices, key=lambda i: (-probs[i], i))


def top_k_filter(probs, indices, k):
    """The k most probable ids in order  (src/sampler/topk_topp.cpp:8-18)."""
    k = max(1, min(k, len(indices)))
    return order_by_probability(probs, indices)[:k]


def top_p_filter(probs, indices, p):
    """Shortest prefix of the ordered ids whose share of their total reaches p
    (src/sampler/topk_topp.cpp:20-35)."""
    order = order_by_probability(probs, indices)
    if p >= 1.0:
        return order
    total = np.float32(0)
    for i in order:
        total += probs[i]
    s, kept = np.float32(0), 0
    for i in order:
        s += probs[i]
        kept += 1
        if total > 0 and s / total >= np.float32(p):
            break
    return order[:kept]


def sample(logits, temperature, top_p, top_k, penalty, prev_tokens, u):
    """One token from one row  (src/sampler/sampler.cpp:23-79) with the uniform number u given."""
    x = np.array(logits, dtype=np.float32)
    if penalty != 1.0 and len(prev_tokens):
        x = repetition_penalty(x, prev_tokens, penalty)
    if temperature > 0 and temperature != 1.0:
        x = x * (np.float32(1.0) / np.float32(temperature))
    if temperature <= 0:
        return greedy(x)
    probs = softmax(x)
    idx = list(range(len(x)))
    if 0 < top_k < len(x):
        idx = top_k_filter(probs, idx, top_k)
    if top_p < 1.0 or top_k > 0:
        idx = top_p_filter(probs, idx, top_p)
    sel = np.array([probs[i] for i in idx], dtype=np.float32)
    sel = sel / sel.sum(dtype=np.float32)
    c = np.float32(0)
    for j, pj in enumerate(sel):                      # src/sampler/topk_topp.cpp:49-56
        c += pj
        if np.float32(u) < c:
            return idx[j]
    return idx[-1]


# ----------------------------------------------------- weights and files
def parameter_shapes(cfg):
    """Tensor names and shapes the reference looks up  (src/model/qwen.cpp:228-281)."""
    h, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or h // nh
    inter, v = cfg["intermediate_size"], cfg["vocab_size"]
    shapes = {"model.embed_tokens.weight": (v, h), "model.norm.weight": (h,)}
    if not cfg.get("tie_word_embeddings", False):
        shapes["lm_head.weight"] = (v, h)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        shapes.update({
            p + "self_attn.q_proj.weight": (nh * d, h), p + "self_attn.q_proj.bias": (nh * d,),
            p + "self_attn.k_proj.weight": (nkv * d, h), p + "self_attn.k_proj.bias": (nkv * d,),
            p + "self_attn.v_proj.weight": (nkv * d, h), p + "self_attn.v_proj.bias": (nkv * d,),
            p + "self_attn.o_proj.weight": (h, nh * d),
            p + "mlp.gate_proj.weight": (inter, h), p + "mlp.up_proj.weight": (inter, h),
            p + "mlp.down_proj.weight": (h, inter),
            p + "input_layernorm.weight": (h,), p + "post_attention_layernorm.weight": (h,)})
    return shapes


def random_weights(cfg, seed, std=0.02, gain_std=0.02, sharp=0.0):
    """Seeded float32 weights: N(0, std) for matrices and biases, 1 + N(0, gain_std) for gains.
    ``sharp`` > 0 multiplies the q and k projections so that attention is far from uniform
    and a single wrong key changes the result visibly."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in parameter_shapes(cfg).items():
        x = rng.standard_normal(shape).astype(np.float32)
        if name.endswith("layernorm.weight") or name == "model.norm.weight":
            out[name] = (1.0 + gain_std * x).astype(np.float32)
        else:
            out[name] = (std * x).astype(np.float32)
            if sharp and (".q_proj." in name or ".k_proj." in name):
                out[name] *= np.float32(sharp)
    return out


def to_bf16_bits(x):
    """float32 -> bfloat16 bit patterns, round to nearest even."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


def from_bf16_bits(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_to_bf16(weights):
    return {k: from_bf16_bits(to_bf16_bits(v)).reshape(v.shape) for k, v in weights.items()}


def write_model_folder(path, cfg, weights, store="F32"):
    """config.json and model.safetensors (8-byte header length, JSON header, raw data:
    the layout src/model/model_loader.cpp:41-103 parses)."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name in sorted(weights):
        a = np.ascontiguousarray(weights[name], dtype=np.float32)
        raw = a.tobytes() if store == "F32" else to_bf16_bits(a).tobytes()
        header[name] = {"dtype": store, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hb = json.dumps(header).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for raw in blobs:
            f.write(raw)


def read_model_folder(path):
    """(config dict, name -> float32 array) of a folder written by anyone."""
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        if e["dtype"] == "F32":
            a = np.frombuffer(data[b:en], dtype=np.float32)
        elif e["dtype"] == "BF16":
            a = from_bf16_bits(np.frombuffer(data[b:en], dtype=np.uint16))
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = a.reshape(e["shape"]).copy()
    return cfg, out
