"""Random-weights mode: weights from a configuration and a seed.

Two uses.  ``write_random_model`` writes a model folder (config.json and
model.safetensors) that the ordinary loader then reads by name; tests and the
replay tool use it.  ``init_random_on_device`` fills a model's tensors on the GPU
without touching the disk; benchmarks at real layer sizes use it.  The reference
has no such mode.

Values: matrices and biases N(0, std), norm gains 1 + N(0, gain_std).  Each
tensor has its own generator, seeded from the seed and the tensor's name, so a
tensor's values do not depend on which other tensors exist or on their order.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Optional

import torch

from ..config.registry import resolve_architecture
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, shape, role: str, seed: int, std: float, gain_std: float,
                  device="cpu") -> torch.Tensor:
    """One tensor's float32 values."""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    t = torch.randn(tuple(shape), generator=g, dtype=torch.float32, device=device)
    if role == "gain":
        return 1.0 + gain_std * t
    return std * t


def write_random_model(path: str, config: dict, seed: int = 0, dtype: str = "bfloat16",
                       std: Optional[float] = None, gain_std: Optional[float] = None,
                       model_arch: str = "") -> Dict[str, torch.Tensor]:
    """Write ``path``/config.json and ``path``/model.safetensors; return the stored tensors.

    ``dtype`` is the stored type ("bfloat16" or "float32").  ``std`` and
    ``gain_std`` default to the architecture's (config.json's initializer_range).
    """
    from ..parts.model import TORCH_DTYPES, DecoderModel
    if dtype not in TORCH_DTYPES:
        raise ValueError(f"dtype must be one of {sorted(TORCH_DTYPES)}")
    _, spec = resolve_architecture(config, model_arch)
    model = DecoderModel(spec, TORCH_DTYPES[dtype], "meta")
    std = spec.init_std if std is None else std
    gain_std = spec.init_gain_std if gain_std is None else gain_std
    tensors = {}
    for name, ps in model.param_specs().items():
        tensors[name] = random_tensor(name, ps.shape, ps.role, seed, std, gain_std).to(TORCH_DTYPES[dtype])
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    write_safetensors(os.path.join(path, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
    return tensors


def init_random_on_device(model, seed: int, std: Optional[float] = None,
                          gain_std: Optional[float] = None) -> None:
    """Fill ``model`` with random tensors generated on its device."""
    spec = model.spec
    std = spec.init_std if std is None else std
    gain_std = spec.init_gain_std if gain_std is None else gain_std
    tensors = {}
    for name, ps in model.param_specs().items():
        t = random_tensor(name, ps.shape, ps.role, seed, std, gain_std, device=model.device)
        tensors[name] = t.to(model.placement(ps.role))
    model.load_params(tensors)
