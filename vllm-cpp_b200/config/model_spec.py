"""Architecture-neutral description of a decoder, as data.

An architecture's configuration (``config.json``) is turned into a
:class:`ModelSpec`: one :class:`LayerSpec` per layer naming its parts (mixer,
feed-forward, norms, arrangement) with every size and constant as a parameter,
and a run order (:class:`LayerCall` list).  The builder in ``parts/model.py``
looks each part's ``kind`` up in the part registries; no part learns which
model it is in.

The reference hard-wires this into ``QwenModel`` (src/model/qwen.cpp:165-199
builds the layers, :300-318 is the run order).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class PartSpec:
    """``kind`` selects a registered part; ``params`` are its constructor arguments."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


class LayerSpec:
    """One layer: a block arrangement and the parts that fill its slots.

    ``block`` names a registered arrangement; the arrangement declares its slots and which family
    of part each takes (``Block.SLOTS`` in parts/base.py).  "prenorm" has ``mixer``,
    ``feed_forward``, ``mixer_norm`` (before the mixer) and ``feed_forward_norm`` (before the
    feed-forward); another arrangement may have other slots, e.g. a third norm.  ``parts`` maps slot
    names to PartSpecs (slots may also be given as keyword arguments); ``names`` maps the same slot
    names to the checkpoint prefixes of the parts' tensors, e.g.
    {"mixer": "model.layers.3.self_attn.", "mixer_norm": "model.layers.3.input_layernorm."}.
    """

    def __init__(self, parts: Optional[Dict[str, PartSpec]] = None, block: str = "prenorm",
                 names: Optional[Dict[str, str]] = None, **slots: PartSpec):
        self.parts: Dict[str, PartSpec] = dict(parts or {}, **slots)
        self.block = block
        self.names: Dict[str, str] = dict(names or {})

    def __getattr__(self, slot):                  # spec.mixer_norm reads spec.parts["mixer_norm"]
        parts = self.__dict__.get("parts", {})
        if slot in parts:
            return parts[slot]
        raise AttributeError(slot)

    def __repr__(self):
        return f"LayerSpec(block={self.block!r}, parts={self.parts!r}, names={self.names!r})"


@dataclass
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` (an index may appear twice: the same
    weights run again).  ``cache`` names the cache layer that this call's mixer
    uses; ``writes_cache`` False means the call only reads what an earlier call
    with the same ``cache`` wrote in this step and in earlier ones.
    """
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: List[LayerSpec]
    run_order: List[LayerCall]
    final_norm: PartSpec
    tie_word_embeddings: bool
    max_position_embeddings: int
    # Checkpoint names of the tensors outside the layers.
    embed_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    lm_head_name: str = "lm_head.weight"
    # Token ids that end a request unless it asks to ignore them.
    stop_token_ids: List[int] = field(default_factory=list)
    # Tensor names that a checkpoint may hold and the engine ignores.
    ignored_tensors: List[str] = field(default_factory=list)
    # Standard deviations of the random-weights mode.
    init_std: float = 0.02
    init_gain_std: float = 0.02
    # The registered model class that is built from this spec (parts/model.py MODEL_CLASSES).  "decoder" is
    # embedding -> layers -> final norm -> output product; an architecture that scales its embeddings,
    # caps its logits or adds an output bias registers a subclass that overrides embed() or head().
    model_class: str = "decoder"

    def validate(self) -> None:
        n_cache = 1 + max((c.cache for c in self.run_order), default=-1)
        writers = {}
        for i, call in enumerate(self.run_order):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"run_order[{i}] names layer {call.layer}, model has {len(self.layers)}")
            if call.writes_cache:
                if call.cache in writers:
                    raise ValueError(
                        f"run_order[{i}] writes cache {call.cache}, already written by entry {writers[call.cache]}")
                writers[call.cache] = i
            elif call.cache not in writers:
                raise ValueError(f"run_order[{i}] reads cache {call.cache} before any entry wrote it")
        missing = [c for c in range(n_cache) if c not in writers]
        if missing:
            raise ValueError(f"cache layers {missing} are never written")

    @property
    def num_cache_layers(self) -> int:
        return 1 + max((c.cache for c in self.run_order), default=-1)
