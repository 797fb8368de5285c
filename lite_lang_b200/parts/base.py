"""Interfaces of the parts a layer is put together from, and their registries.

A *part* is built from a ``PartSpec`` (kind + constants) alone; it never sees
the model configuration or knows which model it is in.  Five kinds exist:

``Norm``              y = f(x); optionally fused with the residual sum.
``PositionEncoding``  acts on the q and k heads of the step's tokens.
``Mixer``             mixes information across a request's tokens and owns
                      per-request memory through the cache manager (pages of
                      keys and values, or a record of fixed size).
``FeedForward``       acts on each token alone (dense or routed).
``Block``             the arrangement of the four above in a layer.

All parts declare their checkpoint tensors (``tensors``) with names relative to
their prefix, and receive them in ``load``.  Adding a part is: subclass,
``register_part("mixer", "my_kind", MyMixer)``, and name ``my_kind`` in a
``PartSpec`` of some architecture's ``model_spec``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple, Type

import torch

from ..config.spec import PartSpec


# --------------------------------------------------------------------------
# declarations
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class TensorDecl:
    """A checkpoint tensor a part reads.

    ``role`` decides how it is kept on the device and how random weights are
    drawn: ``matrix`` (compute dtype, N(0, s_matrix)), ``bias`` (float32,
    N(0, s_bias)), ``norm`` (float32, 1 + N(0, s_norm)), ``table`` (int32).
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


@dataclass(frozen=True)
class PagedKVNeed:
    """Per-token keys and values in pages.  Planes with equal needs share a cache group."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None   # None: every earlier position stays readable


@dataclass(frozen=True)
class StateNeed:
    """A record of fixed size per request (zeroed when the request slot is opened)."""

    shape: Tuple[int, ...]
    dtype: str = "float32"         # "float32", "bfloat16" or "compute" (the engine's dtype)


class Part:
    kind_family = ""

    def __init__(self, spec: PartSpec):
        self.spec = spec
        self.prefix = spec.prefix

    def tensors(self) -> Dict[str, TensorDecl]:
        """Checkpoint tensors of this part, names relative to ``self.prefix``."""
        return {}

    def load(self, fetch: Callable[[str], Optional[torch.Tensor]], dtype: torch.dtype, device: torch.device) -> None:
        """Take the tensors (``fetch(relative_name)`` gives a CPU tensor or None) onto the device."""

    def kernel_libraries(self) -> Sequence[str]:
        """Kernel libraries this part launches from (compiled before the first step)."""
        return ("core",)


class Norm(Part):
    kind_family = "norm"

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor],
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """residual += delta (in place, unless ``rows`` selects rows), then the norm of it.

        The default is the unfused form; a part with a fused kernel overrides it.
        ``delta`` may also be float32 partial sums [parts, tokens, hidden] of a product that was
        split over its inner dimension; they are added up first.
        """
        if delta is not None and delta.dim() == 3:
            delta = delta.sum(0).to(residual.dtype)
        if rows is not None:
            picked = residual.index_select(0, rows.long())
            if delta is not None:
                picked = (picked.float() + delta.index_select(0, rows.long()).float()).to(residual.dtype)
            return self.forward(picked)
        if delta is not None:
            residual.copy_((residual.float() + delta.float()).to(residual.dtype))
        return self.forward(residual)


class PositionEncoding(Part):
    kind_family = "position"
    # True if `fused_table()` gives a cos/sin table that the fused
    # bias+rotation+store kernel understands (half-split pairs).
    fuses_with_store = False

    def apply(self, qkv: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int,
              head_dim: int, num_tokens: int) -> None:
        """Encode positions into the q and k heads of ``qkv`` [tokens, (nh+2nkv)*hd], in place."""
        raise NotImplementedError

    def prepare(self, device: torch.device) -> None:
        """Build device tables (called once after ``load``)."""


class StepView:
    """What a part may know about the step that is running.  See engine/batch.py."""


class Mixer(Part):
    kind_family = "mixer"

    def cache_need(self):
        """``PagedKVNeed``, ``StateNeed`` or None."""
        return None

    def prepare(self, device: torch.device, dtype: torch.dtype) -> None:
        pass

    # True: ``forward`` takes ``residual=h`` and may add its output to the residual stream itself (in its
    # last product's epilogue), returning None instead of the output
    accumulates = False

    def forward(self, x: torch.Tensor, step: "StepView", cache: Any) -> torch.Tensor:
        """x [tokens, hidden] -> [tokens, hidden].  ``cache`` is the view of this run-step's plane."""
        raise NotImplementedError


class FeedForward(Part):
    kind_family = "feed_forward"
    accumulates = False   # as for a mixer

    def forward(self, x: torch.Tensor, step: "StepView") -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of a mixer, a feed-forward and their norms.

    ``forward`` gets the residual stream ``h`` and a pending ``delta`` that has
    not been added to it yet (so that the sum can be fused into the next norm)
    and returns the same pair.
    """

    kind_family = "block"

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def parts(self) -> List[Part]:
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], step: "StepView", cache: Any):
        raise NotImplementedError


# --------------------------------------------------------------------------
# registries
# --------------------------------------------------------------------------

_REGISTRY: Dict[str, Dict[str, Any]] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {}, "embedding": {}, "head": {},
}


def register_part(family: str, kind: str, cls: Any) -> None:
    if family not in _REGISTRY:
        raise KeyError(f"unknown part family {family!r}; families: {sorted(_REGISTRY)}")
    _REGISTRY[family][kind] = cls


def part_class(family: str, kind: str):
    try:
        return _REGISTRY[family][kind]
    except KeyError:
        raise KeyError(
            f"no {family} part of kind {kind!r} is registered; known: {sorted(_REGISTRY.get(family, {}))}"
        ) from None


def build_part(family: str, spec: PartSpec):
    return part_class(family, spec.kind)(spec)
