"""Random-weights mode: weights from a configuration and a seed.

Two uses.  ``write_random_model`` writes a model folder (config.json and
model.safetensors) that the ordinary loader then reads by name; tests, the replay
tool and the reference arm of the benchmark use it.  ``init_random_on_device``
fills a model's tensors on the GPU without touching the disk; benchmarks at real
layer sizes use it.  The reference has no such mode.

Values: matrices and biases N(0, std), norm gains 1 + N(0, gain_std).  Element i of
a tensor is a function of (seed, tensor name, i) alone: a counter-based generator,
so a value does not depend on which other tensors exist, on the order of
generation, on how a tensor is cut into slices, or on where it is computed.
``normal_values`` below (numpy, on the host) and ``random_normal_kernel``
(csrc/random_init.cu, on the device) perform the same sequence of correctly rounded
float32 operations and integer steps and agree to the bit, so a host program can
reproduce any value of a model that was filled on the device.

    z      = splitmix64 finaliser of (key + (i + 1) * 0x9E3779B97F4A7C15),  key = sha256(seed:name)[:8]
    u1     = (bits 63..40 of z + 1) / 2^24;  radius = sqrt(-2 ln u1)
    angle  = 2 pi (bits 39..16 of z + 1/2) / 2^24
    value  = mean + std * radius * cos(angle)            (Box-Muller)

The logarithm and the cosine are short series of single float32 operations (no
library function: libm's and CUDA's differ in the last bit).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Optional

import numpy as np
import torch

from ..config.registry import resolve_architecture
from .safetensors_io import write_safetensors

_MASK64 = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor's stream of values."""
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little")


def _f(bits: int) -> np.float32:
    """A float32 constant by its bit pattern (the same words as in csrc/random_init.cu)."""
    return np.array(bits, dtype=np.uint32).view(np.float32)[()]


_SQRT2, _LN2, _HALF_PI, _TWO_M22 = _f(0x3fb504f3), _f(0x3f317218), _f(0x3fc90fdb), _f(0x34800000)
_LN_SERIES = (_f(0x3de38e39), _f(0x3e124925), _f(0x3e4ccccd), _f(0x3eaaaaab), np.float32(1.0))    # 1/9 1/7 1/5 1/3 1
_SIN_SERIES = (_f(0x3638ef1d), _f(0xb9500d01), _f(0x3c088889), _f(0xbe2aaaab), np.float32(1.0))   # 1/9! -1/7! 1/5! -1/3! 1
_COS_SERIES = (_f(0xb493f27e), _f(0x37d00d01), _f(0xbab60b61), _f(0x3d2aaaab), np.float32(-0.5), np.float32(1.0))
_ONE, _HALF, _TWO = np.float32(1.0), np.float32(0.5), np.float32(2.0)


def _horner(coeffs, x2: np.ndarray) -> np.ndarray:
    p = np.full_like(x2, coeffs[0])
    for c in coeffs[1:]:
        p = p * x2 + c          # two roundings, as __fadd_rn(__fmul_rn(p, x2), c) on the device
    return p


def standard_normal(key: int, first: int, count: int) -> np.ndarray:
    """float32 [count]: the standard-normal values of elements first .. first + count - 1 of the stream ``key``."""
    with np.errstate(over="ignore"):
        i = np.arange(first + 1, first + count + 1, dtype=np.uint64)
        z = np.uint64(key & _MASK64) + i * np.uint64(_GOLDEN)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    a = (z >> np.uint64(40)).astype(np.uint32)
    b = ((z >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.uint32)
    # ln((a + 1) / 2^24): a + 1 = m * 2^e with m in [1, 2), moved to (0.707, 1.414]; ln m = 2 atanh((m - 1) / (m + 1))
    mant, ex = np.frexp((a + np.uint32(1)).astype(np.float32))
    m = mant * _TWO
    e = ex.astype(np.int32) - 1
    big = m > _SQRT2
    m = np.where(big, m * _HALF, m)
    e = e + big
    s = (m + np.float32(-1.0)) / (m + _ONE)
    ln_m = (_TWO * s) * _horner(_LN_SERIES, s * s)
    ln_u = (e - 24).astype(np.float32) * _LN2 + ln_m
    radius = np.sqrt(np.float32(-2.0) * ln_u)
    # cos(2 pi (b + 1/2) / 2^24): quadrant from the two top bits, the rest folded into (0, pi/4]
    quadrant = b >> np.uint32(22)
    x = ((b & np.uint32(0x3FFFFF)).astype(np.float32) + _HALF) * _TWO_M22
    upper = x > _HALF
    y = np.where(upper, _ONE + (-x), x)
    t = y * _HALF_PI
    t2 = t * t
    sn = t * _horner(_SIN_SERIES, t2)
    cp = _horner(_COS_SERIES, t2)
    c = np.where(upper, sn, cp)
    sd = np.where(upper, cp, sn)
    cosine = np.select([quadrant == 0, quadrant == 1, quadrant == 2], [c, -sd, -c], sd)
    return (radius * cosine).astype(np.float32)


def normal_values(key: int, first: int, count: int, mean: float, std: float) -> np.ndarray:
    """float32 [count]: mean + std * standard_normal, a multiplication and an addition in float32."""
    out = np.empty(count, dtype=np.float32)
    chunk = 1 << 20
    for start in range(0, count, chunk):
        n = min(chunk, count - start)
        out[start: start + n] = np.float32(mean) + np.float32(std) * standard_normal(key, first + start, n)
    return out


def _mean_std(role: str, std: float, gain_std: float):
    return (1.0, gain_std) if role == "gain" else (0.0, std)


def random_tensor(name: str, shape, role: str, seed: int, std: float, gain_std: float,
                  dtype: torch.dtype = torch.float32, device="cpu") -> torch.Tensor:
    """One tensor's values in ``dtype`` (float32 values rounded to nearest even): by numpy on the host,
    by the kernel on a CUDA device.  Both give the same bits."""
    shape = tuple(int(s) for s in shape)
    numel = int(np.prod(shape)) if shape else 1
    mean, sd = _mean_std(role, std, gain_std)
    key = tensor_key(seed, name)
    if torch.device(device).type == "cuda":
        from ..csrc import ops
        out = torch.empty(shape, dtype=dtype, device=device)
        ops.random_normal(out, key, mean, sd)
        return out
    return torch.from_numpy(normal_values(key, 0, numel, mean, sd)).view(shape).to(dtype)


def random_rows(name: str, shape, rows, role: str, seed: int, std: float, gain_std: float) -> np.ndarray:
    """float32 [len(rows), width]: chosen rows of the 2-D tensor ``name`` as random_tensor would fill it,
    without making the rest (what a host check of a large model needs)."""
    width = int(shape[1])
    mean, sd = _mean_std(role, std, gain_std)
    key = tensor_key(seed, name)
    return np.stack([normal_values(key, int(r) * width, width, mean, sd) for r in rows])


def write_random_model(path: str, config: dict, seed: int = 0, dtype: str = "bfloat16",
                       std: Optional[float] = None, gain_std: Optional[float] = None,
                       model_arch: str = "", device="cpu") -> Dict[str, torch.Tensor]:
    """Write ``path``/config.json and ``path``/model.safetensors; return the stored tensors.

    ``dtype`` is the stored type ("bfloat16" or "float32").  ``std`` and
    ``gain_std`` default to the architecture's (config.json's initializer_range).
    ``device``: where the values are computed ("cuda" is much faster for a large
    model; the file is the same).
    """
    from ..parts.model import TORCH_DTYPES, build_model
    if dtype not in TORCH_DTYPES:
        raise ValueError(f"dtype must be one of {sorted(TORCH_DTYPES)}")
    _, spec = resolve_architecture(config, model_arch)
    model = build_model(spec, TORCH_DTYPES[dtype], "meta")
    std = spec.init_std if std is None else std
    gain_std = spec.init_gain_std if gain_std is None else gain_std
    tensors = {}
    for name, ps in model.param_specs().items():
        tensors[name] = random_tensor(name, ps.shape, ps.role, seed, std, gain_std,
                                      dtype=TORCH_DTYPES[dtype], device=device).cpu()
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    write_safetensors(os.path.join(path, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
    return tensors


def init_random_on_device(model, seed: int, std: Optional[float] = None,
                          gain_std: Optional[float] = None) -> None:
    """Fill ``model`` with the tensors ``write_random_model`` would store for the same seed, generated
    on its device directly in the type each role is held in."""
    spec = model.spec
    std = spec.init_std if std is None else std
    gain_std = spec.init_gain_std if gain_std is None else gain_std
    tensors = {}
    for name, ps in model.param_specs().items():
        held = model.placement(ps.role)
        if held == torch.float32 and model.dtype != torch.float32:
            # a bias or gain of a bfloat16 model: the value a bfloat16 checkpoint would hold, kept in float32
            t = random_tensor(name, ps.shape, ps.role, seed, std, gain_std, dtype=model.dtype, device=model.device).to(held)
        else:
            t = random_tensor(name, ps.shape, ps.role, seed, std, gain_std, dtype=held, device=model.device)
        tensors[name] = t
    model.load_params(tensors)
