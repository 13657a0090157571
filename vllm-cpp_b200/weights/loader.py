"""Weights by tensor name, checked against what the model declares.

The reference looks tensors up by name in one ``model.safetensors``
(src/model/qwen.cpp:219-281), checks no shape, reads a missing tensor as an empty
vector and squeezes every value through half precision
(src/layers/linear.cpp:38-42).  Here the model's ``param_specs`` is the list of
expected tensors; names, shapes and tying are checked before anything is copied
and all faults are reported in one error.

Types on the device.  Matrices take the engine's compute type (bfloat16 values
are copied as they are; float32 mode upcasts exactly).  Biases and norm gains are
held in float32, since the arithmetic that uses them is float.  Other tensors an
architecture declares keep what the file stores: 32-bit floats stay 32-bit,
integer tables become int32.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Tuple

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile

SINGLE_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"


class WeightsError(ValueError):
    """Missing, unexpected or mis-shaped tensors; the message lists all of them."""


def open_checkpoint(model_path: str) -> Dict[str, SafetensorsFile]:
    """name -> file holding it, for a single file or an index with shards."""
    single = os.path.join(model_path, SINGLE_FILE)
    index = os.path.join(model_path, INDEX_FILE)
    if os.path.isfile(single):
        f = SafetensorsFile(single)
        return {n: f for n in f.names()}
    if os.path.isfile(index):
        with open(index) as fh:
            try:
                weight_map = json.load(fh)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise WeightsError(f"{index}: not a safetensors index (no 'weight_map')") from None
        files: Dict[str, SafetensorsFile] = {}
        out = {}
        for name, shard in weight_map.items():
            if shard not in files:
                files[shard] = SafetensorsFile(os.path.join(model_path, shard))
            if name not in files[shard].entries:
                raise WeightsError(f"{index} places {name!r} in {shard}, which does not hold it")
            out[name] = files[shard]
        return out
    raise WeightsError(f"no weights in {model_path}: neither {SINGLE_FILE} nor {INDEX_FILE}")


def check_names_and_shapes(expected: Dict[str, object], present: Dict[str, Tuple[int, ...]],
                           ignored_suffixes: List[str], tied_lm_head: str = "") -> None:
    missing = sorted(n for n in expected if n not in present)
    unexpected = sorted(n for n in present if n not in expected
                        and not any(n.endswith(s) for s in ignored_suffixes)
                        and n != tied_lm_head)
    wrong = sorted((n, tuple(present[n]), tuple(expected[n].shape)) for n in expected
                   if n in present and tuple(present[n]) != tuple(expected[n].shape))
    if missing or unexpected or wrong:
        lines = ["checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong))
        raise WeightsError("\n".join(lines))


def _place(t: torch.Tensor, role: str, compute_dtype: torch.dtype, device) -> torch.Tensor:
    if role == "matrix":
        target = compute_dtype
    elif role in ("bias", "gain"):
        target = torch.float32
    elif t.dtype.is_floating_point:
        target = torch.float32 if (t.dtype == torch.float32 or compute_dtype == torch.float32) else torch.bfloat16
    else:
        target = torch.int32
    return t.to(device=device, dtype=target)


def load_checkpoint(model, model_path: str) -> None:
    """Read ``model_path``'s safetensors into ``model`` (a parts.model.DecoderModel)."""
    expected = model.param_specs()
    try:
        where = open_checkpoint(model_path)
    except SafetensorsError as e:
        raise WeightsError(str(e)) from None
    present = {n: f.shape(n) for n, f in where.items()}
    spec = model.spec
    # A tied model may still store a copy of the output matrix; it is not read.
    tied_copy = spec.lm_head_name if spec.tie_word_embeddings else ""
    check_names_and_shapes(expected, present, spec.ignored_tensors, tied_copy)
    tensors = {}
    for name, ps in expected.items():
        tensors[name] = _place(where[name].tensor(name), ps.role, model.dtype, model.device)
    model.load_params(tensors)
    for f in set(where.values()):
        f.close()
