"""A model as data: which parts each layer is made of, and the order in which layers run.

An architecture turns its typed configuration into a ``ModelPlan``; the engine builds
the parts the plan names from the part registry (``camelid_b200.parts``) and knows
nothing else about the architecture. The reference's precedent is a per-layer plan
with a layer-kind switch inside one forward loop (src/model.rs:439-518).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ..errors import ConfigError


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered ``kind``, its sizes and constants, and the prefix of its
    tensors' names in the model folder (e.g. ``model.layers.3.self_attn.``)."""
    kind: str
    params: dict = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement of its parts (``prenorm``: x + mixer(norm(x)), then
    r + ffn(norm(r))) and the parts themselves. Layers of one model may differ. A layer
    without ``ffn`` (and ``norm2``) has only the first sublayer; ``shift`` names a part that
    stands between the first norm and the mixer (a token shift). The ``sandwich`` arrangement
    also norms every sublayer's output before it is added, x + scale * post_norm(sublayer(norm(x))),
    with ``post_norm1`` / ``post_norm2`` and ``residual_scale``. The ``postnorm`` arrangement norms the stream itself after
    every sum, x <- norm1(a x + mixer(x)), x <- norm2(a x + ffn(x)), with a = ``residual_scale``; the sublayers read x as
    it is. ``after`` names a part (role ``layer_input``) that runs at the end of the layer and adds what it makes from the
    stream and the step's tokens."""
    arrangement: str
    norm1: PartSpec
    mixer: PartSpec
    norm2: Optional[PartSpec] = None
    ffn: Optional[PartSpec] = None
    shift: Optional[PartSpec] = None
    post_norm1: Optional[PartSpec] = None
    post_norm2: Optional[PartSpec] = None
    residual_scale: float = 1.0
    after: Optional[PartSpec] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``layer`` indexes ``ModelPlan.layers`` and may occur in several
    entries (the layer's weights are then shared, each entry keeping a cache of its own).
    ``cache_source`` names an earlier entry of the schedule whose keys and values this
    entry reads instead of making its own. ``pass_number`` t marks the first layer of the
    t-th pass over a stretch of layers that runs several times: the plan's ``pass_input`` part
    runs right before it."""
    layer: int
    cache_source: Optional[int] = None
    pass_number: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    embedding: PartSpec
    layers: tuple
    schedule: tuple
    final_norm: PartSpec
    head: PartSpec
    hidden_size: int
    vocab_size: int
    max_position: int
    stop_token_ids: tuple = ()
    pass_input: Optional[PartSpec] = None       # what happens to the stream before each pass of a looped stretch

    def __post_init__(self):
        for i, e in enumerate(self.schedule):
            if e.pass_number is not None and self.pass_input is None:
                raise ConfigError("schedule", f"schedule entry {i} starts pass {e.pass_number} but the plan has no pass_input part")
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError("schedule", f"schedule entry {i} names layer {e.layer}, the plan has {len(self.layers)}")
            if e.cache_source is not None:
                if not 0 <= e.cache_source < i:
                    raise ConfigError("schedule", f"schedule entry {i} reads the cache of entry {e.cache_source}, which does not run before it")
                if self.schedule[e.cache_source].cache_source is not None:
                    raise ConfigError("schedule", f"schedule entry {i} reads entry {e.cache_source}, which has no cache of its own")
