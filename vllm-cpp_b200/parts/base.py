"""Interfaces and registries of the parts a decoder is put together from.

A part is built from its own parameters only (sizes, constants), declares its
tensors with local names, and runs on what the step hands it.  Five kinds are
registered by name: mixers, feed-forwards, norms, position encodings and block
arrangements.  The reference has these as fixed classes wired inside QwenModel
(src/layers/attention.cpp, src/layers/mlp.cpp, src/kernels/layernorm.cu,
src/kernels/rotary_embedding.cu, src/model/qwen.cpp:300-318).

Adding a part: subclass the interface, decorate the class with the matching
``register_*`` and name it in a ``PartSpec``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch


# ----------------------------------------------------------------- parameters
@dataclass
class ParamSpec:
    """One tensor of a part.

    role "matrix": a product's weight, held in the compute type, random N(0, std).
    role "bias":   added in float, held in float32, random N(0, std).
    role "gain":   a norm's scale, held in float32, random 1 + N(0, gain_std).
    """
    shape: Tuple[int, ...]
    role: str = "matrix"


# -------------------------------------------------------------------- caches
@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values in pages.  ``window`` 0: all keys are kept; > 0: only the
    last ``window`` keys are read, pages left of the window are given back."""
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size, one slot per live request, zero at admission."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class PagedKVView:
    """What a mixer sees of a paged cache layer."""
    pages: torch.Tensor          # [num_pages, 2, num_kv_heads, page_size * head_dim], a block laid out as csrc/common.cuh says (kv_pos)
    group: int                   # index into StepContext.block_tables
    page_size: int


@dataclass
class StateView:
    slots: torch.Tensor          # [num_slots, *shape]


# ------------------------------------------------------------------ the step
@dataclass
class StepContext:
    """One batch as the parts see it: device arrays plus host copies of the small ones.

    Tokens are laid out request by request; request r owns rows
    ``q_start[r] : q_start[r + 1]`` at positions ``ctx_lens[r] + 0, 1, …``.  A kernel that keeps state
    per request finds everything it needs on the device: token t belongs to request
    ``req_of_token[t]``, whose state lives in slot ``state_slots[r]``; it is the first token the
    request ever brought iff ``positions[t] == 0`` (the slot is zeroed at admission), and the first of
    this step iff ``t == q_start[r]``.
    """
    n_tokens: int
    n_reqs: int
    token_ids: torch.Tensor              # int32 [n_tokens]
    positions: torch.Tensor              # int32 [n_tokens]
    req_of_token: torch.Tensor           # int32 [n_tokens]
    q_start: torch.Tensor                # int32 [n_reqs + 1]
    ctx_lens: torch.Tensor               # int32 [n_reqs], tokens in the cache before this step
    block_tables: List[torch.Tensor]     # per paged group: int32 [n_reqs, max_blocks]
    state_slots: torch.Tensor            # int32 [n_reqs]
    logit_rows: torch.Tensor             # int32 [n_wanted]
    n_logit_rows: int
    h_q_start: List[int]
    h_ctx_lens: List[int]
    h_state_slots: List[int]
    decode_only: bool                    # every request brings exactly one token
    max_q_len: int
    max_total_len: int                   # longest context after this step
    split_len: int = 0                   # max_total_len rounded up to a power of two (stable kernel shapes)
    extras: Dict[str, object] = field(default_factory=dict)   # per-step device arrays of kernels
    shapes: Dict[str, int] = field(default_factory=dict)      # launch shapes the parts' builders chose for the step


class Workspace:
    """Bump allocator for a step's temporaries, reset at the start of each step.

    ``take`` hands out views of one device buffer, so a step of a given size
    touches the same addresses every time (needed under CUDA graphs) and makes no
    device allocation once the buffer has reached its size.  The buffer grows on
    demand outside graph capture.
    """

    def __init__(self, device, nbytes: int = 0):
        self.device = device
        self.buf = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        self.offset = 0
        self.high_water = 0
        self.frozen = False

    def reset(self) -> None:
        self.offset = 0

    def mark(self) -> int:
        return self.offset

    def release(self, mark: int) -> None:
        self.offset = mark

    def take(self, shape, dtype: torch.dtype) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * dtype.itemsize
        start = (self.offset + 255) // 256 * 256
        end = start + nbytes
        if end > self.buf.numel():
            if self.frozen:
                raise RuntimeError(f"workspace of {self.buf.numel()} bytes is too small for this step "
                                   f"({end} needed) and may not grow now")
            new = torch.empty(max(end, int(self.buf.numel() * 1.5)), dtype=torch.uint8, device=self.device)
            self.buf = new                   # views handed out earlier keep the old buffer alive
        self.offset = end
        self.high_water = max(self.high_water, end)
        return self.buf[start:end].view(dtype).view(*shape)


# --------------------------------------------------------------------- parts
class Part:
    """Common to all parts: declared tensors and their placement."""

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def load_params(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the tensors of ``param_specs`` (on the device, roles' types applied)."""

    def tensors(self) -> List[torch.Tensor]:
        """Every device tensor the part holds (its own attributes and those of parts inside it)."""
        out = []
        for v in vars(self).values():
            if isinstance(v, torch.Tensor):
                out.append(v)
            elif isinstance(v, Part):
                out.extend(v.tensors())
        return out

    def product_weights(self):
        """The weight matrices of this part's products as (matrix, gated) pairs in the order the part runs
        them, for the model's choice of kernels at load: ``gated`` is 0, or the number of gate features of
        a gate-and-up matrix that the part multiplies with ops.linear_gated."""
        return [(v, 0) for v in vars(self).values() if isinstance(v, torch.Tensor) and v.dim() == 2]

    def step_arrays(self):
        """Work lists the part wants built on the host for every step: name -> builder(HostStep) -> int32
        numpy array.  The step function builds each once per step, uploads it with the step's other
        arrays and hands it over as ``StepContext.extras[name]``; a builder may record a launch shape
        it derived in ``HostStep.shapes`` (it reaches the part as ``StepContext.shapes`` and is part
        of the key under which a decode step is captured).  Any part of any family may have some."""
        return {}

    def reserve(self, n_tokens: int, n_reqs: int, device) -> None:
        """Called once when the engine is built: allocate at its largest what the part keeps outside the
        step's workspace (scratch that kernels merge partial results through), so that it does not move
        later: a buffer that moves makes every captured step stale."""

    def workspace_bytes(self, n_tokens: int, n_reqs: int) -> int:
        """Most bytes of step workspace (Workspace.take) this part takes at once for a step of
        ``n_tokens`` tokens of ``n_reqs`` requests; the engine sizes its memory plan with it."""
        return 0


class PositionEncoding(Part):
    """How positions enter a mixer.

    ``fused()`` returns the arguments of the built-in rotation
    (``rotary_dim``, ``pairing``, ``denom``) when the encoding is one that the
    fused bias + rotation + cache-write kernel performs, else None; then
    ``apply`` is called on the biased q and k before the cache write.
    """

    def fused(self) -> Optional[dict]:
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """In place.  q: [n, heads, d] and k: [n, kv_heads, d] strided views."""
        raise NotImplementedError


class Norm(Part):
    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor,
                row_index: Optional[torch.Tensor] = None) -> None:
        """residual += delta (float32, in place, unless rows are gathered); out = norm(residual)."""
        raise NotImplementedError

    def split(self):
        """(gain, eps) if the norm is y = x * rsqrt(mean(x^2) + eps) * gain with a float32 gain vector:
        then the product before it may apply the gain and the product after it the per-row factor
        (see ops.ResidualNorm, ops.RowScale), and no norm kernel runs.  None: the norm runs by itself."""
        return None


class Mixer(Part):
    """Mixes information between the tokens of a request (attention here)."""

    def cache_spec(self):
        """PagedKVSpec, StateSpec or None."""
        return None

    def fuses_norm(self, n_tokens: int) -> bool:
        """True if, for a step of ``n_tokens``, ``forward`` accepts ``x_scale`` (an ops.RowScale its first
        product applies to x) and ``fuse`` (an ops.ResidualNorm its last product performs instead of
        writing ``out`` plainly).  The block passes those keywords only after a yes."""
        return False

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext, cache, writes_cache: bool,
                ws: Workspace) -> None:
        """x, out: [n_tokens, hidden] in the compute type."""
        raise NotImplementedError


class FeedForward(Part):
    def fuses_norm(self, n_tokens: int) -> bool:
        """As Mixer.fuses_norm."""
        return False

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext, ws: Workspace) -> None:
        raise NotImplementedError


class Block:
    """Arrangement of a layer's parts around the residual stream.

    ``SLOTS`` names the arrangement's slots and the family of part each takes ("mixer",
    "feed_forward" or "norm"); the model builds one part per slot from the layer's spec and hands
    them over by name.  They are kept as attributes (``self.mixer`` ...) and, in the order of
    ``SLOTS``, in ``self.parts``.  The model, the loader and the step function walk ``self.parts``;
    none of them knows the slots' names.  An arrangement with other parts (a third norm, two
    feed-forwards) declares them in its own ``SLOTS``."""

    SLOTS: Dict[str, str] = {"mixer": "mixer", "feed_forward": "feed_forward",
                             "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def __init__(self, **parts):
        missing = [n for n in self.SLOTS if n not in parts]
        extra = [n for n in parts if n not in self.SLOTS]
        if missing or extra:
            raise ValueError(f"{type(self).__name__} takes the parts {sorted(self.SLOTS)}; "
                             f"missing {missing}, not known {extra}")
        self.parts: Dict[str, Part] = {n: parts[n] for n in self.SLOTS}
        for name, part in self.parts.items():
            setattr(self, name, part)

    def cache_spec(self):
        """The cache need of the layer: that of its one part of the mixer family."""
        mixers = [p for n, p in self.parts.items() if self.SLOTS[n] == "mixer"]
        if len(mixers) != 1:
            raise ValueError(f"{type(self).__name__} has {len(mixers)} mixers; it must say itself what its cache is")
        return mixers[0].cache_spec()

    def step_arrays(self):
        """Per-step work lists of the arrangement itself, as Part.step_arrays (its parts are asked apart)."""
        return {}

    def workspace_bytes(self, n_tokens: int, n_reqs: int, hidden: int, dtype: torch.dtype) -> int:
        """Most bytes of step workspace the layer holds at once in a model of width ``hidden`` computing in
        ``dtype``.  Here: what its greediest part takes (the parts run one after the other and give back
        what they took); an arrangement adds its own buffers."""
        return max((p.workspace_bytes(n_tokens, n_reqs) for p in self.parts.values()), default=0)

    def accepts_prenormed(self, n_tokens: int):
        """(gain, eps) of the norm this block starts with if, for a step of ``n_tokens``, the block can
        take its input as ``delta`` = residual * gain with the rows' factor still to be applied
        (``pending`` an ops.RowScale); None if it wants the residual stream as it is."""
        return None

    def forward(self, residual: torch.Tensor, delta: torch.Tensor, pending, step: StepContext,
                cache, writes_cache: bool, ws: Workspace, next_block: "Optional[Block]" = None,
                carry: Optional[torch.Tensor] = None):
        """Runs the layer.  ``pending`` says what ``delta`` holds: False nothing, True an addition to
        ``residual`` that has not been made yet, an ops.RowScale the pre-normed input (see
        accepts_prenormed; only given to a block that accepts it).  ``next_block`` runs after this
        one (None: the model's final norm does); ``carry`` is float32 scratch
        [2, ops.sumsq_parts(hidden), n_tokens] that lives for the whole step.  Returns the new
        ``pending``."""
        raise NotImplementedError


# ----------------------------------------------------------------- registries
MIXERS: Dict[str, Callable] = {}
FEED_FORWARDS: Dict[str, Callable] = {}
NORMS: Dict[str, Callable] = {}
POSITION_ENCODINGS: Dict[str, Callable] = {}
BLOCKS: Dict[str, Callable] = {}
# family name (the values of Block.SLOTS) -> registry of the parts of that family
FAMILIES: Dict[str, Dict[str, Callable]] = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS}


def _register(table, name):
    def deco(cls):
        table[name] = cls
        return cls
    return deco


def register_mixer(name): return _register(MIXERS, name)
def register_feed_forward(name): return _register(FEED_FORWARDS, name)
def register_norm(name): return _register(NORMS, name)
def register_position_encoding(name): return _register(POSITION_ENCODINGS, name)
def register_block(name): return _register(BLOCKS, name)


def workspace_piece(shape, dtype: torch.dtype) -> int:
    """Bytes one Workspace.take of this shape and type advances the workspace by."""
    n = dtype.itemsize
    for d in shape:
        n *= int(d)
    return (n + 255) // 256 * 256


def build_part(table: Dict[str, Callable], what: str, spec, **context):
    if spec.kind not in table:
        raise ValueError(f"unknown {what} {spec.kind!r}; registered: {sorted(table)}")
    return table[spec.kind](**spec.params, **context)
