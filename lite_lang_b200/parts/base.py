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
from typing import Any, Callable, Dict, List, Mapping, NamedTuple, Optional, Sequence, Tuple, Type

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
    """Per-token memory in pages: a key plane and a value plane.  Planes with equal needs share a cache group.

    The two planes may have different widths (``value_head_dim``; None: as wide as the keys), and a mixer
    that keeps one vector per token only (a latent that serves as key and value) asks for
    ``value_head_dim=0``: its group then has no value plane at all.
    """

    num_kv_heads: int
    head_dim: int                          # width of a key
    window: Optional[int] = None           # None: every earlier position stays readable
    value_head_dim: Optional[int] = None   # width of a value; None: head_dim; 0: no value plane


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

    def split_params(self) -> Optional[Tuple[torch.Tensor, float]]:
        """(weight float32 [hidden], eps) if the norm is y = x / sqrt(mean(x^2) + eps) * weight, so that the
        products around it may split it between them (``NormSplit``); None otherwise."""
        return None

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
    """What a part may know about the step that is running (``engine/batch.py`` fills it in).

    On the device, valid in every step, captured in a CUDA graph or not (int32 tensors):
      ``token_ids [tokens]``, ``positions [tokens]`` (place of each token in its request),
      ``token_req [tokens]`` (entry of each token), ``cu_q [entries + 1]`` (first token of each entry),
      ``ctx_len [entries]`` (tokens of the request cached before this step), ``req_slot [entries]``
      (the request's slot: the row of its block table and of its state record; -1 marks a padding entry,
      which a part skips or gives a defined output), ``status [1]`` (error word).
    On the host: ``num_tokens``, ``num_entries`` (padding included), ``num_single`` (the leading entries
    that bring exactly one token: single-token entries always come first), ``max_kv_len``, ``scratch`` (a
    dict that lives as long as the step, for plans shared by all layers).
    Only in steps that are not captured: ``entries`` (the host's list of entries, with their tokens) and
    ``entry_ctx``.  A step made of single-token entries only may be captured once and replayed with other
    contents of the device arrays: then ``captured`` is true, the arrays are padded to the bucket's size,
    and whatever a part does must depend on the device arrays alone: no host list, no ``.item()``, no
    shape that depends on the step's contents.  A portion of several tokens is never captured.
    """


class NormEntry(NamedTuple):
    """What the product before a norm has to know to prepare the norm's input for the part after the norm
    (``NormSplit``): the norm's weight and eps, and whether that part takes such an input for rows shaped like the
    residual rows it is asked about."""
    weight: torch.Tensor                          # float32 [hidden]
    eps: float
    accepts: Callable[[torch.Tensor], bool]


class NormSplit(NamedTuple):
    """A norm's input as the product before the norm left it, for the product after the norm: the residual rows
    (already summed and written back) times the norm's weight, and the rows' sums of squares in parts.  The product
    after the norm multiplies ``scaled`` and scales each row of its result by 1 / sqrt(sum / width + eps), so the
    norm needs no kernel of its own between two products of a decode step."""
    scaled: torch.Tensor      # [tokens, hidden], the engine's dtype
    sumsq: torch.Tensor       # float32 [parts, 32]: sums of squares of the rows' values, a part per 16 columns
    eps: float


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
    # True: ``forward`` also takes ``into_norm=NormEntry`` (the norm after this part and what comes after it) and
    # may, for steps where that pays and the part after the norm accepts it, add its output to the residual stream
    # and return a ``NormSplit`` instead
    splits_norm = False

    def forward(self, x: torch.Tensor, step: "StepView", cache: Any) -> torch.Tensor:
        """x [tokens, hidden] -> [tokens, hidden].  ``cache`` is the view of this run-step's plane.

        The result may also be float32 partial sums [parts, tokens, hidden] of a last product that was
        split over its inner dimension: ``Norm.add_forward`` adds them up with the residual; a block that
        does anything else with the result passes it through ``whole_output`` first."""
        raise NotImplementedError


def whole_output(out: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A part's output as one [tokens, hidden] tensor of ``dtype`` (partial sums added up)."""
    if out.dim() == 3:
        return out.sum(0).to(dtype)
    return out


class FeedForward(Part):
    kind_family = "feed_forward"
    accumulates = False   # as for a mixer
    # True: ``forward`` accepts a ``NormSplit`` in place of the normalised rows where ``accepts_norm_split`` says so
    takes_norm_split = False

    def accepts_norm_split(self, rows: torch.Tensor) -> bool:
        """Whether a ``NormSplit`` may stand for normalised rows shaped like ``rows`` (the residual rows) in this step."""
        return False

    def forward(self, x: torch.Tensor, step: "StepView") -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """An arrangement of parts in a layer.

    ``roles`` names the parts a block kind is made of and the family each is built from; the layer's
    ``LayerSpec.parts`` gives a ``PartSpec`` for every role.  Every built part is also an attribute of the
    block under its role's name.  ``forward`` gets the residual stream ``h``, a pending ``delta`` that has not
    been added to it yet (so that the sum can be fused into the next norm), and ``caches``: for every role
    of the mixer family, the view of that mixer's cache plane in this run-step (None if it keeps nothing).
    It returns ``(h, delta)`` again.
    """

    kind_family = "block"
    roles: Mapping[str, str] = {}      # role -> family ("mixer", "feed_forward", "norm")

    def __init__(self, parts: Mapping[str, Part]):
        self.named: Dict[str, Part] = dict(parts)
        for role, part in self.named.items():
            setattr(self, role, part)

    def parts(self) -> List[Part]:
        return [self.named[role] for role in self.roles]

    def mixers(self) -> List[Tuple[str, "Mixer"]]:
        """The block's mixers with their roles, in the order of ``roles``."""
        return [(role, self.named[role]) for role, family in self.roles.items() if family == "mixer"]

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], step: "StepView", caches: Mapping[str, Any]):
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
