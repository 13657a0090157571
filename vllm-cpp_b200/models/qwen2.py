"""Qwen2 / Qwen2.5 dense decoder: typed configuration and its description as parts.

Reference: ``QwenModel`` (src/model/qwen.cpp).  It reads eight keys from
config.json with silent Qwen2.5-0.5B defaults (:33-47) and hard-codes the rest:
RMSNorm eps 1e-6 (:303,312,322), bias on q/k/v only
(src/layers/attention.cpp:19-22), "silu" (:191), tying inferred from the absence
of lm_head.weight (:279-285).  Here every one of these is read from config.json,
the eight keys are required, and what the engine cannot run is refused.

Tensor names are the ones the reference looks up (src/model/qwen.cpp:228-281).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from ..config.engine_config import ConfigError
from ..config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture

_REQUIRED_INT = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                 "intermediate_size", "max_position_embeddings", "vocab_size")


@dataclass
class Qwen2Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    max_position_embeddings: int
    vocab_size: int
    rope_theta: float
    head_dim: int
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    initializer_range: float = 0.02
    eos_token_ids: List[int] = field(default_factory=list)
    torch_dtype: Optional[str] = None

    @classmethod
    def from_dict(cls, cfg: dict) -> "Qwen2Config":
        problems = []

        def get_int(key, default=None, required=False):
            v = cfg.get(key, default)
            if v is None:
                if required:
                    problems.append(f"missing required key '{key}'")
                return default
            if isinstance(v, bool) or not isinstance(v, int):
                problems.append(f"'{key}' must be an integer, got {v!r}")
                return default
            return v

        vals = {k: get_int(k, required=True) for k in _REQUIRED_INT}
        theta = cfg.get("rope_theta")
        if theta is None:
            problems.append("missing required key 'rope_theta'")
        elif isinstance(theta, bool) or not isinstance(theta, (int, float)):
            problems.append(f"'rope_theta' must be a number, got {theta!r}")
            theta = None
        if problems:
            raise ConfigError("Qwen2 config.json: " + "; ".join(problems))

        for k, v in vals.items():
            if v <= 0:
                problems.append(f"'{k}' must be positive, got {v}")
        if theta is not None and theta <= 0:
            problems.append(f"'rope_theta' must be positive, got {theta}")
        if problems:
            raise ConfigError("Qwen2 config.json: " + "; ".join(problems))

        nh, nkv, hidden = vals["num_attention_heads"], vals["num_key_value_heads"], vals["hidden_size"]
        head_dim = get_int("head_dim")
        if head_dim is None:
            if hidden % nh:
                problems.append(f"hidden_size {hidden} is not a multiple of num_attention_heads {nh} "
                                "and no 'head_dim' is given")
                head_dim = 0
            else:
                head_dim = hidden // nh       # src/model/qwen.cpp:47
        if head_dim and head_dim % 2:
            problems.append(f"head_dim {head_dim} must be even (rotary pairs)")
        if nh % nkv:
            problems.append(f"num_attention_heads {nh} is not a multiple of num_key_value_heads {nkv}")

        eps = cfg.get("rms_norm_eps", 1e-6)
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not eps > 0:
            problems.append(f"'rms_norm_eps' must be a positive number, got {eps!r}")
        act = cfg.get("hidden_act", "silu")
        if act != "silu":
            problems.append(f"hidden_act {act!r} is not supported (only 'silu')")
        if cfg.get("rope_scaling") is not None:
            problems.append("rope_scaling is not supported (must be null)")
        tie = cfg.get("tie_word_embeddings", False)
        if not isinstance(tie, bool):
            problems.append(f"'tie_word_embeddings' must be true or false, got {tie!r}")

        use_sw = cfg.get("use_sliding_window", False)
        if not isinstance(use_sw, bool):
            problems.append(f"'use_sliding_window' must be true or false, got {use_sw!r}")
            use_sw = False
        window = get_int("sliding_window")
        max_window_layers = get_int("max_window_layers")
        if use_sw:
            if window is None or window <= 0:
                problems.append("use_sliding_window is true but 'sliding_window' is not a positive integer")
            if max_window_layers is None:
                max_window_layers = 0
            if max_window_layers < 0:
                problems.append("'max_window_layers' must not be negative")

        init = cfg.get("initializer_range", 0.02)
        if isinstance(init, bool) or not isinstance(init, (int, float)) or init < 0:
            problems.append(f"'initializer_range' must be a non-negative number, got {init!r}")

        eos = cfg.get("eos_token_id")
        if eos is None:
            eos_ids = []
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = [eos]
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = list(eos)
        else:
            problems.append(f"'eos_token_id' must be an integer or a list of integers, got {eos!r}")
            eos_ids = []
        for e in eos_ids:
            if not 0 <= e < vals["vocab_size"]:
                problems.append(f"eos_token_id {e} lies outside the vocabulary of {vals['vocab_size']}")

        if problems:
            raise ConfigError("Qwen2 config.json: " + "; ".join(problems))
        return cls(rope_theta=float(theta), head_dim=head_dim, rms_norm_eps=float(eps),
                   tie_word_embeddings=tie, hidden_act=act, use_sliding_window=use_sw,
                   sliding_window=window if use_sw else None,
                   max_window_layers=max_window_layers if use_sw else None,
                   initializer_range=float(init), eos_token_ids=eos_ids,
                   torch_dtype=cfg.get("torch_dtype"), **vals)

    def layer_window(self, layer: int) -> int:
        """Window of layer ``layer`` in tokens; 0 means all keys.

        With ``use_sliding_window`` the first ``max_window_layers`` layers see all
        keys and the layers after them the last ``sliding_window`` keys, the
        query's own included.  (The reference reads none of these keys; every
        layer sees all keys there.)
        """
        if self.use_sliding_window and layer >= self.max_window_layers:
            return int(self.sliding_window)
        return 0

    def to_dict(self) -> dict:
        d = {
            "architectures": ["Qwen2ForCausalLM"],
            "model_type": "qwen2",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "max_position_embeddings": self.max_position_embeddings,
            "vocab_size": self.vocab_size,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "use_sliding_window": self.use_sliding_window,
            "initializer_range": self.initializer_range,
        }
        if self.use_sliding_window:
            d["sliding_window"] = self.sliding_window
            d["max_window_layers"] = self.max_window_layers
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d


def qwen2_model_spec(c: Qwen2Config) -> ModelSpec:
    layers = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        norm = PartSpec("rmsnorm", {"size": c.hidden_size, "eps": c.rms_norm_eps})
        layers.append(LayerSpec(
            mixer=PartSpec("attention", {
                "hidden_size": c.hidden_size,
                "num_heads": c.num_attention_heads,
                "num_kv_heads": c.num_key_value_heads,
                "head_dim": c.head_dim,
                "qkv_bias": True,            # src/layers/attention.cpp:19-21
                "out_bias": False,           # src/layers/attention.cpp:22
                "window": c.layer_window(i),
                "position": PartSpec("rope", {"theta": c.rope_theta, "rotary_dim": c.head_dim,
                                              "pairing": "half"}),
            }),
            feed_forward=PartSpec("gated_mlp", {
                "hidden_size": c.hidden_size,
                "intermediate_size": c.intermediate_size,
                "activation": c.hidden_act,
            }),
            mixer_norm=norm,
            feed_forward_norm=PartSpec("rmsnorm", dict(norm.params)),
            block="prenorm",
            names={"mixer": p + "self_attn.", "feed_forward": p + "mlp.",
                   "mixer_norm": p + "input_layernorm.",
                   "feed_forward_norm": p + "post_attention_layernorm."},
        ))
    return ModelSpec(
        architecture="Qwen2ForCausalLM",
        hidden_size=c.hidden_size,
        vocab_size=c.vocab_size,
        layers=layers,
        run_order=[LayerCall(layer=i, cache=i) for i in range(c.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"size": c.hidden_size, "eps": c.rms_norm_eps}),
        tie_word_embeddings=c.tie_word_embeddings,
        max_position_embeddings=c.max_position_embeddings,
        stop_token_ids=list(c.eos_token_ids),
        ignored_tensors=["rotary_emb.inv_freq"],
        init_std=c.initializer_range,
        init_gain_std=c.initializer_range,
    )


@register_architecture("Qwen2ForCausalLM", "qwen")
def build_qwen2(config: dict):
    typed = Qwen2Config.from_dict(config)
    return typed, qwen2_model_spec(typed)
