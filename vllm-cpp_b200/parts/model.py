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
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, PagedKVSpec, ParamSpec, StateSpec, StepContext,
                   Workspace, build_part)
# importing the modules registers the built-in parts
from . import attention as _attention, block as _block, mlp as _mlp, norm as _norm, position as _position  # noqa: F401

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


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
            self.blocks.append(BLOCKS[ls.block](
                mixer=build_part(MIXERS, "mixer", ls.mixer, **ctx),
                feed_forward=build_part(FEED_FORWARDS, "feed-forward", ls.feed_forward, **ctx),
                mixer_norm=build_part(NORMS, "norm", ls.mixer_norm, **ctx),
                feed_forward_norm=build_part(NORMS, "norm", ls.feed_forward_norm, **ctx)))
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
                specs[call.cache] = self.blocks[call.layer].mixer.cache_spec()
        return specs

    def _check_cache_sharing(self) -> None:
        specs = self.cache_specs()
        for i, call in enumerate(self.spec.run_order):
            if not call.writes_cache:
                own = self.blocks[call.layer].mixer.cache_spec()
                if own != specs[call.cache]:
                    raise ValueError(f"run_order[{i}]: layer {call.layer} needs {own} but reads cache "
                                     f"{call.cache} of kind {specs[call.cache]}")

    # ---------------------------------------------------------------- tensors
    def param_specs(self) -> Dict[str, ParamSpec]:
        """Every tensor of the model under its checkpoint name."""
        s = self.spec
        out = {s.embed_name: ParamSpec((self.vocab, self.hidden))}
        for ls, blk in zip(s.layers, self.blocks):
            for slot in ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm"):
                for local, ps in getattr(blk, slot).param_specs().items():
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
            for slot in ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm"):
                prefix = ls.names[slot]
                part = getattr(blk, slot)
                part.load_params({local: tensors[prefix + local] for local in part.param_specs()})
        self.final_norm.load_params({local: tensors[s.final_norm_prefix + local]
                                     for local in self.final_norm.param_specs()})

    def prepare_products(self, tune: bool = True, image_budget: Optional[int] = None) -> None:
        """bfloat16 only: decide, for every shape of weight matrix and bucket of token counts, whether the
        engine's tcgen05 product or the library's runs when a step has few tokens, and make the pre-tiled
        images of the matrices the engine's kernel will read (see csrc/gemm_tcgen05.cu).  Both are
        measured here, on this device, in CUDA graphs.  A layer whose products all run on the engine's
        kernel needs no norm or activation kernels (parts/block.py), so the layers' products are
        measured together first: all on the engine's kernel if that beats the library's products with
        the kernels between them, else each product on its own merits; the output product is chosen
        by itself.
        ``image_budget``: bytes the images may take (None: no limit).  Gated images come first (without
        one the activation stays a kernel of its own), then the others by size; a matrix without an
        image is read through a tensor map, a few percent slower."""
        if self.dtype != torch.bfloat16:
            return
        layer_shapes, fusable_norms = {}, 0          # (shape, gated) -> matrices
        for blk in self.blocks:
            for part in (blk.mixer, blk.feed_forward):
                for v, gated in part.product_weights():
                    if v.dtype == torch.bfloat16:
                        layer_shapes.setdefault((tuple(v.shape), gated), []).append(v)
        if self.blocks:
            first = self.blocks[0]
            fusable_norms = sum(1 for nrm in (first.mixer_norm, first.feed_forward_norm) if nrm.split() is not None)
        tunable = {key: mats for key, mats in layer_shapes.items() if key[0][1] % 8 == 0}
        head_key = (tuple(self.lm_head.shape), 0)
        head_ok = self.lm_head.shape[1] % 8 == 0
        groups = dict(tunable)
        if head_ok and head_key not in groups:
            groups[head_key] = [self.lm_head]

        def image_bytes(key, mats):
            (rows, k), gated = key
            tiles = -(-gated // 64) if gated else -(-rows // 128)
            return len(mats) * tiles * -(-k // 64) * 16384

        imaged, spent = set(), 0
        for key in sorted(groups, key=lambda kk: (kk[1] == 0, -image_bytes(kk, groups[kk]))):
            need = image_bytes(key, groups[key])
            if image_budget is None or spent + need <= image_budget:
                imaged.add(key)
                spent += need
        gated_of = {key: (key[1] if key in imaged else 0) for key in groups}     # a gated product only with its image

        measure = tune and ops.linear_tuning()
        for key in imaged:
            for m in groups[key][:8]:             # the kernel is measured as it will run: on the images
                ops.tile_weights(m, key[1])
        if measure:
            whole = {}
            if len(tunable) == len(layer_shapes) and tunable:
                whole = ops.measure_layer([(mats[:8], gated_of[key]) for key, mats in tunable.items()], self.hidden,
                                          fusable_norms, self.dtype)
            times = None
            for bucket, _ in ops.TOKEN_BUCKETS:
                if bucket in whole and whole[bucket][0] <= whole[bucket][1]:
                    for key in tunable:                   # the layer as a whole is faster on the engine's kernel
                        ops.choose_linear(key[0][0], key[0][1], bucket, torch.bfloat16, True)
                    continue
                if times is None:
                    times = {key: ops.measure_linear(mats[:8], gated=gated_of[key]) for key, mats in tunable.items()}
                for key in tunable:                       # each product on its own merits
                    if bucket in times[key]:
                        t_ours, t_lib = times[key][bucket]
                        ops.choose_linear(key[0][0], key[0][1], bucket, torch.bfloat16, t_ours <= t_lib)
            if head_ok:
                for bucket, (t_ours, t_lib) in ops.measure_linear([self.lm_head], torch.float32).items():
                    ops.choose_linear(self.lm_head.shape[0], self.lm_head.shape[1], bucket, torch.float32, t_ours <= t_lib)
        for key, mats in groups.items():
            shape, gated = key
            out_dtype = torch.float32 if mats[0] is self.lm_head else torch.bfloat16
            chosen = any(ops._linear_choice.get((shape[0], shape[1], b, out_dtype), True) for b, _ in ops.TOKEN_BUCKETS)
            for m in mats:
                if chosen and key in imaged:
                    ops.tile_weights(m, gated)
                else:
                    ops.drop_tiled_weights(m)

    def weight_bytes(self) -> int:
        """Bytes of the matrices a decode step reads once (embedding rows excluded unless tied)."""
        total = 0
        for blk in self.blocks:
            for part in (blk.mixer, blk.feed_forward):
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
        ops.embedding(self.embed, step.token_ids, residual)
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
            ops.linear(normed, self.lm_head, out)
        return out
