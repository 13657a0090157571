"""A decoder put together from a ModelSpec: embedding, layers in their run order,
final norm, output product.

Flow of one step (src/model/qwen.cpp:291-328): ids -> embedding -> for each entry
of the run order, the layer's block on the residual stream -> final norm ->
lm_head.  Differences from the reference: the residual additions happen inside
the norm kernels; only the rows whose logits are wanted go through the final norm
and the output product (the reference computes logits for every token, :321-325);
the output matrix is the embedding table when ``tie_word_embeddings`` is set and a
tensor of its own otherwise (the reference overwrites the table with an untied
lm_head, :228-233,279-281).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.model_spec import ModelSpec
from ..csrc import ops
from .base import BLOCKS, FAMILIES, NORMS, ParamSpec, StepContext, Workspace, build_part
# importing the modules registers the built-in parts
from . import attention as _attention, block as _block, mlp as _mlp, norm as _norm, position as _position  # noqa: F401

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


MODEL_CLASSES: Dict[str, type] = {}


def register_model_class(name: str):
    """Registers a DecoderModel subclass under the name a ModelSpec's ``model_class`` gives."""
    def deco(cls):
        MODEL_CLASSES[name] = cls
        return cls
    return deco


def build_model(spec: ModelSpec, dtype: torch.dtype, device) -> "DecoderModel":
    if spec.model_class not in MODEL_CLASSES:
        raise ValueError(f"unknown model class {spec.model_class!r}; registered: {sorted(MODEL_CLASSES)}")
    return MODEL_CLASSES[spec.model_class](spec, dtype, device)


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        spec.validate()
        self.spec, self.dtype, self.device = spec, dtype, device
        self.hidden, self.vocab = spec.hidden_size, spec.vocab_size
        ctx = {"dtype": dtype, "device": device}
        self.blocks = []
        for i, ls in enumerate(spec.layers):
            if ls.block not in BLOCKS:
                raise ValueError(f"layer {i}: unknown block arrangement {ls.block!r}; registered: {sorted(BLOCKS)}")
            arrangement = BLOCKS[ls.block]
            if set(ls.parts) != set(arrangement.SLOTS):
                raise ValueError(f"layer {i}: arrangement {ls.block!r} takes the parts {sorted(arrangement.SLOTS)}, "
                                 f"the layer names {sorted(ls.parts)}")
            self.blocks.append(arrangement(**{
                slot: build_part(FAMILIES[family], family, ls.parts[slot], **ctx)
                for slot, family in arrangement.SLOTS.items()}))
        self.final_norm = build_part(NORMS, "norm", spec.final_norm, **ctx)
        self.embed: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        self._check_cache_sharing()

    # ------------------------------------------------------------------ cache
    def cache_specs(self) -> List[object]:
        """The cache need of every cache layer, in order (PagedKVSpec, StateSpec or None)."""
        specs: List[object] = [None] * self.spec.num_cache_layers
        for call in self.spec.run_order:
            if call.writes_cache:
                specs[call.cache] = self.blocks[call.layer].cache_spec()
        return specs

    def _check_cache_sharing(self) -> None:
        specs = self.cache_specs()
        for i, call in enumerate(self.spec.run_order):
            if not call.writes_cache:
                own = self.blocks[call.layer].cache_spec()
                if own != specs[call.cache]:
                    raise ValueError(f"run_order[{i}]: layer {call.layer} needs {own} but reads cache "
                                     f"{call.cache} of kind {specs[call.cache]}")

    # ---------------------------------------------------------------- tensors
    def param_specs(self) -> Dict[str, ParamSpec]:
        """Every tensor of the model under its checkpoint name."""
        s = self.spec
        out = {s.embed_name: ParamSpec((self.vocab, self.hidden))}
        for ls, blk in zip(s.layers, self.blocks):
            for slot, part in blk.parts.items():
                for local, ps in part.param_specs().items():
                    out[ls.names[slot] + local] = ps
        for local, ps in self.final_norm.param_specs().items():
            out[s.final_norm_prefix + local] = ps
        if not s.tie_word_embeddings:
            out[s.lm_head_name] = ParamSpec((self.vocab, self.hidden))
        return out

    def placement(self, role: str) -> torch.dtype:
        return self.dtype if role == "matrix" else torch.float32

    def load_params(self, tensors: Dict[str, torch.Tensor]) -> None:
        """``tensors``: checkpoint name -> device tensor in the role's type (see weights/loader.py)."""
        s = self.spec
        self.embed = tensors[s.embed_name].contiguous()
        self.lm_head = self.embed if s.tie_word_embeddings else tensors[s.lm_head_name].contiguous()
        for ls, blk in zip(s.layers, self.blocks):
            for slot, part in blk.parts.items():
                prefix = ls.names[slot]
                part.load_params({local: tensors[prefix + local] for local in part.param_specs()})
        self.final_norm.load_params({local: tensors[s.final_norm_prefix + local]
                                     for local in self.final_norm.param_specs()})

    def prepare_products(self, tune: bool = True, image_budget: Optional[int] = None) -> None:
        """Decide which product kernel runs for which shape and make the weights' tile images (parts/tuning.py)."""
        from .tuning import prepare_products
        prepare_products(self, tune, image_budget)

    def tensors(self) -> List[torch.Tensor]:
        """Every device tensor of the model once (a tied output matrix is the embedding table)."""
        seen, out = set(), []
        parts = [p for blk in self.blocks for p in blk.parts.values()] + [self.final_norm]
        for t in [self.embed, self.lm_head] + [t for p in parts for t in p.tensors()]:
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                out.append(t)
        return out

    def tile_images(self) -> List[torch.Tensor]:
        """The pre-tiled images of weight matrices that exist now (see prepare_products)."""
        mats = [(self.lm_head, 0)] + [pw for blk in self.blocks for p in blk.parts.values() for pw in p.product_weights()]
        imgs = [ops.tiled_weights_of(w, bool(g)) for w, g in mats if w is not None]
        return [i for i in imgs if i is not None]

    def weight_bytes(self) -> int:
        """Bytes of the matrices a decode step reads once (embedding rows excluded unless tied)."""
        total = 0
        for blk in self.blocks:
            for part in blk.parts.values():
                for v, _ in part.product_weights():
                    total += v.numel() * v.element_size()
        total += self.lm_head.numel() * self.lm_head.element_size()
        return total

    # -------------------------------------------------------------------- run
    def forward(self, step: StepContext, caches: List[object], ws: Workspace,
                logits: torch.Tensor) -> torch.Tensor:
        """Runs the step's tokens; fills and returns logits[:n_logit_rows] (float32 [rows, vocab])."""
        n = step.n_tokens
        residual = ws.take((n, self.hidden), torch.float32)
        delta = ws.take((n, self.hidden), self.dtype)
        carry = ws.take((2, ops.sumsq_parts(self.hidden), n), torch.float32)
        self.embed_tokens(step, residual)
        pending = False                 # what delta holds: see Block.forward
        order = self.spec.run_order
        for i, call in enumerate(order):
            following = self.blocks[order[i + 1].layer] if i + 1 < len(order) else None
            pending = self.blocks[call.layer].forward(residual, delta, pending, step, caches[call.cache],
                                                      call.writes_cache, ws, next_block=following, carry=carry)
        has_delta = bool(pending)
        m = step.n_logit_rows
        out = logits[:m]
        if m:
            normed = ws.take((m, self.hidden), self.dtype)
            self.final_norm.forward(residual, delta if has_delta else None, normed, step.logit_rows)
            self.head(normed, out)
        return out

    # Two places an architecture may differ at without touching its layers; a subclass registered with
    # register_model_class overrides them (and ModelSpec.model_class names it).
    def embed_tokens(self, step: StepContext, residual: torch.Tensor) -> None:
        """residual[t] = the embedding of token t in float32 (src/kernels/embedding_kernel.cu:20-28: no scaling)."""
        ops.embedding(self.embed, step.token_ids, residual)

    def head(self, normed: torch.Tensor, out: torch.Tensor) -> None:
        """out [rows, vocab] (float32) = logits of the normed rows (src/model/qwen.cpp:325: a product, no bias)."""
        ops.linear(normed, self.lm_head, out)

    def workspace_bytes(self, n_tokens: int, n_reqs: int, n_logit_rows: int) -> int:
        """Most bytes ``forward`` takes from the workspace for a step of this size: its own buffers plus the
        largest need of any block (each piece rounded up as Workspace.take rounds)."""
        el = torch.empty((), dtype=self.dtype).element_size()
        r = lambda b: (b + 255) // 256 * 256
        own = r(n_tokens * self.hidden * 4) + r(n_tokens * self.hidden * el) \
            + r(2 * ops.sumsq_parts(self.hidden) * n_tokens * 4) + r(n_logit_rows * self.hidden * el)
        return own + max((blk.workspace_bytes(n_tokens, n_reqs, self.hidden, self.dtype) for blk in self.blocks), default=0)


MODEL_CLASSES["decoder"] = DecoderModel
