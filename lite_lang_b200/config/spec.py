"""Data that describes a model to the engine: parts, layers and their order.

An architecture's typed configuration turns its ``config.json`` into a
``ModelSpec``.  Everything below the configuration (weights, parts, cache,
step function) reads sizes and constants from the spec only.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: which implementation (``kind``) and its constants.

    ``prefix`` is the checkpoint prefix under which the part's tensors live,
    e.g. ``model.layers.3.self_attn.``.
    """

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (``block``) and the parts it arranges, by role.

    Which roles there are is the block kind's business: the pre-norm block takes ``mixer``,
    ``feed_forward``, ``mixer_norm`` and ``feed_forward_norm``; a block with norms after its parts, or with
    two mixers, names its own.  The block kind also says which family (mixer, feed_forward, norm) each
    role's part is built from.
    """

    block: str
    parts: Mapping[str, PartSpec]


@dataclass(frozen=True)
class RunStep:
    """One entry of the order in which layers run.

    ``layer`` indexes ``ModelSpec.layers`` and may occur more than once (the
    layer's weights are then used again).  ``cache`` names the cache plane the
    mixer works on: ``None`` gives the entry a plane of its own; the index of
    an earlier entry makes it read that entry's plane without writing to it.
    """

    layer: int
    cache: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole causal language model as data."""

    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[RunStep, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()
