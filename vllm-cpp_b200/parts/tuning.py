"""Which product runs where, decided at load by measurement on this device (bfloat16 only).

For every shape of weight matrix and bucket of token counts: the engine's tcgen05 product or the
library's, when a step has few tokens; and the pre-tiled images of the matrices the engine's kernel
will read (csrc/gemm_tcgen05.cu).  Both sides are measured in CUDA graphs.  A layer whose products
all run on the engine's kernel needs no norm or activation kernels (parts/block.py), so the layers'
products are measured together first: all on the engine's kernel if that beats the library's
products with the kernels between them, else each product on its own merits; the output product is
chosen by itself.  The reference's engine uses cuBLAS for every product (src/layers/linear.cpp:70-77).

The parts say which of their tensors are products (``Part.product_weights``: by default every 2-D
tensor, in the order the part runs them; the first reads the norm before the part, the last ends the
part's residual branch); nothing here knows a part's kind.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops


# What the all-own layer's time may be of the library's for buckets whose tiles are 32 columns and more
# (see prepare_products).
WIDE_TILE_MARGIN = 0.9


def prepare_products(model, tune: bool = True, image_budget: Optional[int] = None) -> None:
    """``image_budget``: bytes the images may take (None: no limit).  Gated images come first (without
    one the activation stays a kernel of its own), then the others by size; a matrix without an
    image is read through a tensor map, a few percent slower."""
    if model.dtype != torch.bfloat16:
        return
    layer_shapes, fusable_norms = {}, 0          # (shape, gated) -> matrices
    for blk in model.blocks:
        for part in blk.parts.values():
            for v, gated in part.product_weights():
                if v.dtype == torch.bfloat16:
                    layer_shapes.setdefault((tuple(v.shape), gated), []).append(v)
    if model.blocks:
        first = model.blocks[0]
        fusable_norms = sum(1 for name, part in first.parts.items()
                            if first.SLOTS[name] == "norm" and part.split() is not None)
    tunable = {key: mats for key, mats in layer_shapes.items() if key[0][1] % 8 == 0}
    head_key = (tuple(model.lm_head.shape), 0)
    head_ok = model.lm_head.shape[1] % 8 == 0
    groups = dict(tunable)
    if head_ok and head_key not in groups:
        groups[head_key] = [model.lm_head]

    imaged, spent = set(), 0
    for key in sorted(groups, key=lambda kk: (kk[1] == 0, -image_bytes(kk, len(groups[kk])))):
        need = image_bytes(key, len(groups[key]))
        if image_budget is None or spent + need <= image_budget:
            imaged.add(key)
            spent += need
    gated_of = {key: (key[1] if key in imaged else 0) for key in groups}     # a gated product only with its image

    measure = tune and ops.linear_tuning()
    if not measure:
        for (shape, _gated) in groups:            # what another engine of this process measured for these shapes
            ops.forget_choices(shape[0], shape[1])
    for key in imaged:
        for m in groups[key][:8]:             # the kernel is measured as it will run: on the images
            ops.tile_weights(m, key[1])
    if measure:
        # first the grid of the engine's own product per shape, at the token counts decode steps have
        for key, mats in groups.items():
            if key in imaged:
                for bucket, tokens in ops.TOKEN_BUCKETS[:3]:
                    is_head = mats[0] is model.lm_head
                    ops.choose_ctas(mats[:8], bucket, tokens, gated_of[key], torch.float32 if is_head else torch.bfloat16)
                    if key[0][0] == model.hidden and not gated_of[key] and not is_head:
                        ops.choose_ctas(mats[:8], bucket, tokens, residual=True)     # as it ends a residual branch
        whole = {}
        if len(tunable) == len(layer_shapes) and tunable:
            # the products in the order a layer runs them; a part's first product reads the norm before the
            # part, its last one ends the part's residual branch
            chain = []
            for part in model.blocks[0].parts.values():
                listed = [(v, gated) for v, gated in part.product_weights() if v.dtype == torch.bfloat16]
                for i, (v, gated) in enumerate(listed):
                    key = (tuple(v.shape), gated)
                    chain.append((tunable[key][:8], gated_of[key], i == 0, i == len(listed) - 1))
            whole = ops.measure_layer(chain, model.hidden, fusable_norms, model.dtype)
        model.tuning_report = {"layer_products_us": {b: (round(o, 1), round(t, 1)) for b, (o, t) in whole.items()}}
        times = None
        for bucket, _ in ops.TOKEN_BUCKETS:
            # Tiles of 32 columns and more run two CTAs an SM, which do not fit beside the attention kernel's:
            # in a step such a product cannot set itself up under the kernel before it as it does in the
            # measured chain, and starts 3-4 us later (seen in the step's timeline at 7B sizes).  The layer as a
            # whole has to win by that much.
            margin = 1.0 if bucket <= 16 else WIDE_TILE_MARGIN
            if bucket in whole and whole[bucket][0] <= margin * whole[bucket][1]:
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
            for bucket, (t_ours, t_lib) in ops.measure_linear([model.lm_head], torch.float32).items():
                ops.choose_linear(model.lm_head.shape[0], model.lm_head.shape[1], bucket, torch.float32, t_ours <= t_lib)
    for key, mats in groups.items():
        shape, gated = key
        out_dtype = torch.float32 if mats[0] is model.lm_head else torch.bfloat16
        chosen = any(ops._linear_choice.get((shape[0], shape[1], b, out_dtype), True) for b, _ in ops.TOKEN_BUCKETS)
        for m in mats:
            if chosen and key in imaged:
                ops.tile_weights(m, gated)
            else:
                ops.drop_tiled_weights(m)


def image_bytes(key, count: int) -> int:
    """Bytes of the tile images of ``count`` matrices of shape and gating ``key`` = ((rows, k), gated)."""
    (rows, k), gated = key
    tiles = -(-gated // 64) if gated else -(-rows // 128)
    return count * tiles * -(-k // 64) * 16384
