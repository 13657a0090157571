"""Each part of a layer alone against its plain formula, and the generality of the parts:
a toy architecture defined in this file — a mixer with state of its own, a feed-forward that
routes tokens to experts, a position encoding the fused kernel does not know, different mixers
and feed-forwards in different layers, a layer that
runs twice, a layer that reads another layer's cache — is registered, built, loaded and
stepped through the unchanged framework, and compared with a plain model under different
ways of cutting the work."""
import types

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from helpers import TOL, compare, model_folder

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def stored(a, dtype):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(DT[dtype]).float().numpy()


def part_harness(mixer, page=16, pages=32, max_len=256, max_seqs=4):
    """A cache manager and a runner around one mixer, to get real StepContexts for it."""
    from vllm_cpp_b200.cache.manager import CacheManager
    from vllm_cpp_b200.engine.runner import ModelRunner
    cache = CacheManager([mixer.cache_spec()], page, pages, max_seqs, mixer.dtype, "cuda")
    fake = types.SimpleNamespace(vocab=1000, blocks=[types.SimpleNamespace(parts={"mixer": mixer})], final_norm=None,
                                 spec=types.SimpleNamespace(max_position_embeddings=max_len))
    return cache, ModelRunner(fake, cache, 512, max_seqs, max_len, torch.device("cuda", 0))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from vllm_cpp_b200.parts.norm import RMSNorm
    rng = np.random.default_rng(0)
    n = RMSNorm(size=120, eps=2e-5, dtype=DT[dtype], device="cuda")
    assert n.param_specs()["weight"].shape == (120,) and n.param_specs()["weight"].role == "gain"
    g = (1 + 0.2 * rng.standard_normal(120)).astype(np.float32)
    n.load_params({"weight": dev(g)})
    res = rng.standard_normal((6, 120)).astype(np.float32)
    delta = stored(rng.standard_normal((6, 120)), dtype)
    r, out = dev(res), torch.empty((6, 120), dtype=DT[dtype], device="cuda")
    n.forward(r, dev(delta, DT[dtype]), out)
    want = plain.rms_norm((res + delta).astype(np.float64), g, 2e-5)
    assert np.abs(out.float().cpu().numpy() - want).max() <= (2e-6 if dtype == "float32" else 1e-2) * np.abs(want).max()
    assert np.allclose(r.cpu().numpy(), res + delta, atol=1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_mlp_part(dtype):
    from vllm_cpp_b200.parts.base import Workspace
    from vllm_cpp_b200.parts.mlp import GatedMLP
    rng = np.random.default_rng(1)
    h, inter = 72, 200
    m = GatedMLP(hidden_size=h, intermediate_size=inter, activation="silu", dtype=DT[dtype], device="cuda")
    w = {k: stored(0.2 * rng.standard_normal(s.shape), dtype) for k, s in m.param_specs().items()}
    m.load_params({k: dev(v, DT[dtype]) for k, v in w.items()})
    x = stored(rng.standard_normal((9, h)), dtype)
    out = torch.empty((9, h), dtype=DT[dtype], device="cuda")
    m.forward(dev(x, DT[dtype]), out, None, Workspace("cuda"))
    want = plain.swiglu_mlp(x.astype(np.float64), w["gate_proj.weight"], w["up_proj.weight"], w["down_proj.weight"])
    assert np.abs(out.float().cpu().numpy() - want).max() <= (1e-5 if dtype == "float32" else 2e-2) * np.abs(want).max()
    with pytest.raises(ValueError, match="activation"):
        GatedMLP(hidden_size=8, intermediate_size=8, activation="gelu", dtype=DT[dtype], device="cuda")


def test_rope_part_arguments():
    from vllm_cpp_b200.parts.position import NoPosition, RotaryEmbedding
    r = RotaryEmbedding(theta=1e6, rotary_dim=32, pairing="half", device="cuda")
    f = r.fused()
    j = np.arange(16, dtype=np.float32)
    # theta^(2j/d) with theta and the exponent in float; the part takes the power in double and rounds it, the
    # reference's powf may differ from that in the last bit
    want = np.power(np.float32(1e6), (np.float32(2) * j) / np.float32(32)).astype(np.float32)
    got = f["denom"].cpu().numpy()
    assert f["rotary_dim"] == 32 and f["pairing"] == 0 and got.dtype == np.float32
    assert np.all(np.abs(got.astype(np.float64) - want) <= np.spacing(want))
    assert np.array_equal(got, np.power(np.float64(np.float32(1e6)), ((np.float32(2) * j) / np.float32(32)).astype(np.float64)).astype(np.float32))
    assert NoPosition().fused()["rotary_dim"] == 0
    with pytest.raises(ValueError):
        RotaryEmbedding(theta=1e4, rotary_dim=7)
    with pytest.raises(ValueError):
        RotaryEmbedding(theta=1e4, rotary_dim=8, pairing="spiral")


@pytest.mark.parametrize("dtype,nh,nkv,d,window", [("float32", 4, 2, 16, 0), ("float32", 3, 1, 48, 11),
                                                    ("bfloat16", 6, 2, 64, 0), ("bfloat16", 14, 2, 128, 50),
                                                    ("bfloat16", 5, 5, 32, 0)])
def test_attention_part_whole_and_in_portions(dtype, nh, nkv, d, window):
    """The attention mixer alone: q/k/v with bias, rotation, cache write, attention, output projection."""
    from vllm_cpp_b200.config.model_spec import PartSpec
    from vllm_cpp_b200.engine.runner import StepEntry
    from vllm_cpp_b200.parts.attention import PagedAttention
    rng = np.random.default_rng(2)
    hidden, theta = 88, 50000.0
    att = PagedAttention(hidden_size=hidden, num_heads=nh, num_kv_heads=nkv, head_dim=d, qkv_bias=True, out_bias=False,
                         window=window, position=PartSpec("rope", {"theta": theta, "rotary_dim": d, "pairing": "half"}),
                         dtype=DT[dtype], device="cuda")
    specs = att.param_specs()
    w = {k: stored((0.3 if "q_proj.w" in k or "k_proj.w" in k else 0.15) * rng.standard_normal(s.shape),
                   dtype if s.role == "matrix" else "float32") for k, s in specs.items()}
    att.load_params({k: dev(v, DT[dtype] if specs[k].role == "matrix" else torch.float32) for k, v in w.items()})
    cache, runner = part_harness(att)
    n = 150
    x = stored(rng.standard_normal((n, hidden)), dtype)
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": d, "hidden_size": hidden, "rope_theta": theta}
    pw = {"p." + k: v.astype(np.float64) for k, v in w.items()}
    want = plain.attention_block(x.astype(np.float64), np.arange(n), pw, "p.", cfg, window)

    def run(cuts, rid):
        cache.add_request(rid)
        outs = []
        for a, b in cuts:
            step = runner._prepare([StepEntry(rid, [0] * (b - a), [])])
            runner.ws.reset()
            out = torch.empty((b - a, hidden), dtype=DT[dtype], device="cuda")
            att.forward(dev(x[a:b], DT[dtype]), out, step, runner.views[0], True, runner.ws)
            cache.commit(rid, b - a)
            outs.append(out.float().cpu().numpy())
        cache.free_request(rid)
        return np.concatenate(outs)

    tol = 1e-5 if dtype == "float32" else 2e-2
    whole = run([(0, n)], "w")
    assert np.abs(whole - want).max() <= tol * np.abs(want).max()
    parts = run([(0, 70), (70, 72), (72, 129), (129, 130), (130, 131), (131, 150)], "p")
    assert np.abs(parts - want).max() <= tol * np.abs(want).max()


# --------------------------------------------------------------------------------------
# A toy architecture, defined here and nowhere in the framework.
TOY_CFG = {"architectures": ["ToyMixForCausalLM"], "hidden_size": 48, "vocab_size": 97, "heads": 3, "head_dim": 16,
           "inter": 80, "experts": 3, "expert_inter": 24, "eps": 1e-5, "max_position_embeddings": 200, "tie_word_embeddings": False}


def register_toy():
    from vllm_cpp_b200.config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
    from vllm_cpp_b200.config.registry import register_architecture
    from vllm_cpp_b200.parts.base import (Block, FeedForward, Mixer, ParamSpec, PositionEncoding, StateSpec,
                                          register_block, register_feed_forward, register_mixer, register_norm,
                                          register_position_encoding)
    from vllm_cpp_b200.parts.model import DecoderModel, register_model_class
    from vllm_cpp_b200.parts.norm import RMSNorm

    @register_mixer("toy_running_mean")
    class RunningMean(Mixer):
        """out_t = W * mean(x_0 .. x_t): its state is the running sum and the count."""

        def __init__(self, hidden_size, dtype, device):
            self.h, self.dtype = hidden_size, dtype

        def param_specs(self):
            return {"mix.weight": ParamSpec((self.h, self.h))}

        def load_params(self, tensors):
            self.w = tensors["mix.weight"]

        def cache_spec(self):
            return StateSpec((self.h + 1,), torch.float32)

        def forward(self, x, out, step, cache, writes_cache, ws):
            for r in range(step.n_reqs):
                a, b = step.h_q_start[r], step.h_q_start[r + 1]
                state = cache.slots[step.h_state_slots[r]]
                sums = state[: self.h] + torch.cumsum(x[a:b].float(), dim=0)
                counts = state[self.h] + torch.arange(1, b - a + 1, device=x.device, dtype=torch.float32)
                out[a:b] = ((sums / counts[:, None]).to(self.dtype) @ self.w.t())
                if writes_cache:
                    state[: self.h] = sums[-1]
                    state[self.h] = counts[-1]

    @register_feed_forward("toy_relu_routed")
    class ReluRouted(FeedForward):
        """out = sum_e g_e(x) down_e(relu(up_e x)) with g = relu(router x) / (1 + sum relu(router x)), router
        logits in 32-bit.  An expert runs only on the tokens that give it a weight above zero; the
        weights fall to zero continuously, so rounding cannot flip a choice into a different result."""

        def __init__(self, hidden_size, inter, experts, dtype, device):
            self.h, self.inter, self.n, self.dtype = hidden_size, inter, experts, dtype

        def param_specs(self):
            specs = {"router.weight": ParamSpec((self.n, self.h), "bias")}        # held in float32
            for e in range(self.n):
                specs[f"experts.{e}.up.weight"] = ParamSpec((self.inter, self.h))
                specs[f"experts.{e}.down.weight"] = ParamSpec((self.h, self.inter))
            return specs

        def load_params(self, tensors):
            self.router = tensors["router.weight"]
            self.up = [tensors[f"experts.{e}.up.weight"] for e in range(self.n)]
            self.down = [tensors[f"experts.{e}.down.weight"] for e in range(self.n)]
            self.tokens_per_expert = [0] * self.n

        def forward(self, x, out, step, ws):
            gate = torch.relu(x.float() @ self.router.t())
            gate = gate / (1.0 + gate.sum(dim=1, keepdim=True))
            acc = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e in range(self.n):
                rows = torch.nonzero(gate[:, e] > 0).flatten()
                self.tokens_per_expert[e] += rows.numel()
                if rows.numel() == 0:
                    continue
                hidden = torch.relu(x[rows] @ self.up[e].t())
                acc.index_add_(0, rows, (hidden @ self.down[e].t()).float() * gate[rows, e, None])
            out.copy_(acc)

    @register_position_encoding("toy_ramp")
    class Ramp(PositionEncoding):
        """Adds slope * position to the first element of every q and k head; not a rotation,
        so the mixer has to call apply() instead of using the fused kernel."""

        def __init__(self, slope, dtype=None, device=None):
            self.slope = slope

        def apply(self, q, k, positions):
            q[:, :, 0] += (self.slope * positions.float()).to(q.dtype)[:, None]
            k[:, :, 0] += (self.slope * positions.float()).to(k.dtype)[:, None]

    @register_norm("toy_first_token_norm")
    class FirstTokenNorm(RMSNorm):
        """An RMSNorm whose output row is doubled for the token at position 0 of a request.  Which rows
        those are it learns from a work list of its own, built on the host for every step."""

        def step_arrays(self):
            def first_rows(host):
                flags, t = np.zeros(sum(host.q_lens), dtype=np.int32), 0
                for q, ctx in zip(host.q_lens, host.ctx_lens):
                    flags[t] = 1 if ctx == 0 else 0
                    t += q
                return flags
            return {"toy_first_rows": first_rows}

        def forward_branch(self, x, out, step):
            """out = norm(x) for a branch's output x (not the residual stream), rows of first tokens doubled."""
            self.forward(x.float(), None, out)
            out.mul_((1 + step.extras["toy_first_rows"]).to(out.dtype)[:, None])

    @register_block("toy_sandwich")
    class Sandwich(Block):
        """x += post(mixer(norm_a(x)));  x += feed_forward(norm_b(x)): a third norm on the mixer's output."""
        SLOTS = dict(Block.SLOTS, post_mixer_norm="norm")

        def forward(self, residual, delta, pending, step, cache, writes_cache, ws, next_block=None, carry=None):
            mark = ws.mark()
            n, hidden = residual.shape
            h, mixed, normed = (ws.take((n, hidden), delta.dtype) for _ in range(3))
            self.mixer_norm.forward(residual, delta if pending else None, h)
            self.mixer.forward(h, mixed, step, cache, writes_cache, ws)
            self.post_mixer_norm.forward_branch(mixed, normed, step)
            self.feed_forward_norm.forward(residual, normed, h)
            self.feed_forward.forward(h, delta, step, ws)
            ws.release(mark)
            return True

    @register_model_class("toy_scaled")
    class ScaledModel(DecoderModel):
        """Embeddings times sqrt(hidden), logits capped smoothly at +-cap: the two hooks of the model class."""
        CAP = 3.0

        def embed_tokens(self, step, residual):
            super().embed_tokens(step, residual)
            residual.mul_(float(np.sqrt(np.float32(self.hidden))))

        def head(self, normed, out):
            super().head(normed, out)
            out.copy_(self.CAP * torch.tanh(out / self.CAP))

    @register_architecture("ToyMixForCausalLM")
    def build(cfg):
        h = cfg["hidden_size"]
        norm = lambda: PartSpec("rmsnorm", {"size": h, "eps": cfg["eps"]})
        ff = lambda: PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": cfg["inter"], "activation": "silu"})
        attn = lambda pos: PartSpec("attention", {"hidden_size": h, "num_heads": cfg["heads"], "num_kv_heads": 1,
                                                  "head_dim": cfg["head_dim"], "qkv_bias": False, "out_bias": False,
                                                  "window": 0, "position": pos})
        routed = PartSpec("toy_relu_routed", {"hidden_size": h, "inter": cfg["expert_inter"], "experts": cfg["experts"]})
        kinds = [(attn(PartSpec("rope", {"theta": 1e4, "rotary_dim": 8, "pairing": "interleaved"})), ff()),
                 (PartSpec("toy_running_mean", {"hidden_size": h}), routed),
                 (attn(PartSpec("toy_ramp", {"slope": 0.01})), ff())]
        layers = []
        for i, (mixer, feed_forward) in enumerate(kinds):
            p = f"toy.{i}."
            parts = {"mixer": mixer, "feed_forward": feed_forward, "mixer_norm": norm(), "feed_forward_norm": norm()}
            names = {"mixer": p + "mixer.", "feed_forward": p + "ff.", "mixer_norm": p + "n1.", "feed_forward_norm": p + "n2."}
            if i == 2:                      # the last layer has three norms, one of them with a work list of its own
                parts["post_mixer_norm"] = PartSpec("toy_first_token_norm", {"size": h, "eps": cfg["eps"]})
                names["post_mixer_norm"] = p + "n3."
            layers.append(LayerSpec(parts, block="toy_sandwich" if i == 2 else "prenorm", names=names))
        # layer 0, the state layer, layer 2, then layer 0's weights once more on layer 0's cache
        # (read only), then the state layer again with a cache of its own
        order = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(2, 2), LayerCall(0, 0, writes_cache=False),
                 LayerCall(1, 3)]
        spec = ModelSpec(architecture="ToyMixForCausalLM", hidden_size=h, vocab_size=cfg["vocab_size"], layers=layers,
                         run_order=order, final_norm=norm(), tie_word_embeddings=False,
                         max_position_embeddings=cfg["max_position_embeddings"], embed_name="toy.embed",
                         final_norm_prefix="toy.final.", lm_head_name="toy.head", model_class="toy_scaled")
        return cfg, spec


def toy_plain_forward(w, cfg, ids):
    """The same model with the plain parts, whole sequence, float64."""
    w = {k: v.astype(np.float64) for k, v in w.items()}
    h, nh, d, eps = cfg["hidden_size"], cfg["heads"], cfg["head_dim"], cfg["eps"]
    t = len(ids)
    pos = np.arange(t)

    def attn(x, p, kind, kv=None):
        q = plain.linear(x, w[p + "q_proj.weight"]).reshape(t, nh, d)
        k = plain.linear(x, w[p + "k_proj.weight"]).reshape(t, 1, d)
        v = plain.linear(x, w[p + "v_proj.weight"]).reshape(t, 1, d)

        def encode(z):
            z = z.copy()
            if kind == "rope":                     # interleaved pairs over the first 8 elements
                ang = plain.rope_angles(pos, 1e4, 8).astype(np.float64)[:, None, :]
                a, b = z[..., 0:8:2].copy(), z[..., 1:8:2].copy()
                z[..., 0:8:2] = a * np.cos(ang) - b * np.sin(ang)
                z[..., 1:8:2] = a * np.sin(ang) + b * np.cos(ang)
            else:
                z[..., 0] += 0.01 * pos[:, None]
            return z

        q = encode(q)
        if kv is None:
            kv = (encode(k), v)
        o = plain.attention(q, kv[0], kv[1], nh, 1).reshape(t, nh * d)
        return plain.linear(o, w[p + "o_proj.weight"]), kv

    def mean_mixer(x, p):
        run = np.cumsum(x, axis=0) / np.arange(1, t + 1)[:, None]
        return plain.linear(run, w[p + "mix.weight"])

    def ff(x, p):
        if p + "router.weight" in w:               # the routed feed-forward: every expert on every token
            gate = np.maximum(plain.linear(x, w[p + "router.weight"]), 0.0)
            gate = gate / (1.0 + gate.sum(axis=1, keepdims=True))
            y = np.zeros_like(x)
            for e in range(cfg["experts"]):
                hidden = np.maximum(plain.linear(x, w[p + f"experts.{e}.up.weight"]), 0.0)
                y += gate[:, e:e + 1] * plain.linear(hidden, w[p + f"experts.{e}.down.weight"])
            return y
        return plain.swiglu_mlp(x, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])

    x = plain.embedding(ids, w["toy.embed"]) * np.float64(np.sqrt(np.float32(h)))
    kv0 = None
    for layer, kind in [(0, "rope"), (1, "mean"), (2, "ramp"), (0, "rope-shared"), (1, "mean")]:
        p = f"toy.{layer}."
        hdn = plain.rms_norm(x, w[p + "n1.weight"], eps)
        if kind == "mean":
            x = x + mean_mixer(hdn, p + "mixer.")
        elif kind == "rope-shared":
            x = x + attn(hdn, p + "mixer.", "rope", kv0)[0]
        else:
            o, kv = attn(hdn, p + "mixer.", kind)
            if layer == 0:
                kv0 = kv
            if layer == 2:                             # the third norm, on the branch; the first token's row doubled
                o = plain.rms_norm(o, w[p + "n3.weight"], eps)
                o[0] *= 2.0
            x = x + o
        x = x + ff(plain.rms_norm(x, w[p + "n2.weight"], eps), p + "ff.")
    logits = plain.linear(plain.rms_norm(x, w["toy.final.weight"], eps), w["toy.head"])
    return 3.0 * np.tanh(logits / 3.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_state_runs_through_the_unchanged_framework(tmp_path, dtype):
    register_toy()
    from helpers import Replayer
    from vllm_cpp_b200 import EngineConfig, resolve_architecture
    from vllm_cpp_b200.engine import factory
    from vllm_cpp_b200.parts.base import PagedKVSpec, StateSpec
    from vllm_cpp_b200.parts.model import DecoderModel

    _, spec = resolve_architecture(TOY_CFG)
    from vllm_cpp_b200.parts.model import build_model
    shapes = {k: v.shape for k, v in build_model(spec, torch.float32, "meta").param_specs().items()}
    assert "toy.2.n3.weight" in shapes and type(build_model(spec, torch.float32, "meta")).__name__ == "ScaledModel"
    rng = np.random.default_rng(7)
    w = {}
    for name, shape in shapes.items():
        x = rng.standard_normal(shape).astype(np.float32)
        w[name] = (1 + 0.1 * x) if name.endswith(("n1.weight", "n2.weight", "n3.weight", "final.weight")) else 0.15 * x
        w[name] = w[name].astype(np.float32)
    if dtype == "bfloat16":
        w = plain.round_to_bf16(w)
    folder = model_folder(tmp_path, TOY_CFG, w, dtype)
    model, cache, runner = factory.build(EngineConfig(model_path=folder, dtype=dtype, block_size=16, num_gpu_blocks=24,
                                                      max_num_seqs=3, max_model_len=200, max_num_batched_tokens=256,
                                                      use_cuda_graphs=False))
    kinds = [type(s) for s in model.cache_specs()]
    assert kinds == [PagedKVSpec, StateSpec, PagedKVSpec, StateSpec]
    assert len(cache.paged) == 1 and len(cache.state) == 1 and cache.state[0].layers == [1, 3]

    ids = {r: np.random.default_rng(s).integers(0, 97, size=n).tolist() for r, s, n in
           [("a", 1, 90), ("b", 2, 61), ("c", 3, 40), ("d", 4, 75)]}
    want = {r: toy_plain_forward(w, TOY_CFG, t) for r, t in ids.items()}
    rp = Replayer(runner, cache)
    # whole
    rp.step([("a", ids["a"], range(90))], end=["a"])
    compare(rp.logits_of("a", range(90)), want["a"], dtype, "toy whole")
    # portions and single tokens, mixed with others; slots are used again (3 slots, 4 requests)
    rp.rows.clear()
    rp.step([("a", ids["a"][:33], range(33)), ("b", ids["b"][:2], range(2))])
    rp.step([("a", ids["a"][33:35], range(2)), ("b", ids["b"][2:50], range(48)), ("c", ids["c"][:17], range(17))])
    rp.step([("b", ids["b"][50:], range(11)), ("c", ids["c"][17:18], [0])], end=["b"])
    rp.step([("a", ids["a"][35:], range(55)), ("d", ids["d"][:30], range(30)), ("c", ids["c"][18:], range(22))],
            end=["a", "c"])
    for t in range(30, 75):
        rp.step([("d", ids["d"][t:t + 1], [0])])
    rp.step([("e", [1, 2, 3], [])], end=["d", "e"])
    for r in "abcd":
        compare(rp.logits_of(r, range(len(ids[r]))), want[r], dtype, f"toy mixed {r}")
    assert cache.num_free_pages() == 24 and len(cache._free_slots) == 3
    # the routed feed-forward did route: every expert got some tokens and none got all of them
    seen = model.blocks[1].feed_forward.tokens_per_expert
    assert all(0 < n < sum(seen) for n in seen), seen
