"""The generic causal language model: parts assembled from a ``ModelSpec``.

Structure of the reference's model (``litelang/models/qwen2/model.py:23-59``):
embedding, the layers in order, final norm, lm_head.  Here the layers are
``Block`` parts built from the spec, and the order in which they run is the
spec's ``order`` list: an entry may name a layer a second time (its weights are
used again, on a cache plane of its own) or point at an earlier entry's cache
plane (it then reads that plane and writes nothing).

The model also derives the *cache groups* from the mixers' needs: run-steps
whose mixers need the same kind of memory share a group (one page pool and one
block table per request, or one array of fixed-size records), and each writing
run-step gets a plane in its group.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..cache.manager import PagedGroupSpec, StateGroupSpec
from ..config.spec import ModelSpec
from ..parts import base as parts_base
from ..parts.base import PagedKVNeed, StateNeed, TensorDecl, build_part, part_class


@dataclass(frozen=True)
class PlannedCache:
    group: Optional[int]     # cache group, None if the mixer keeps nothing
    plane: int
    writable: bool


@dataclass(frozen=True)
class PlannedStep:
    """A run-step with the cache plane of each of its block's mixers (by role)."""

    layer: int
    caches: Dict[str, PlannedCache]

    def _first(self) -> PlannedCache:
        return next(iter(self.caches.values())) if self.caches else PlannedCache(None, 0, False)

    # a block with one mixer (the usual case): that mixer's plane
    @property
    def group(self) -> Optional[int]:
        return self._first().group

    @property
    def plane(self) -> int:
        return self._first().plane

    @property
    def writable(self) -> bool:
        return self._first().writable


class CausalLM:
    def __init__(self, spec: ModelSpec):
        import lite_lang_b200.parts  # noqa: F401  (registers the built-in parts)

        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.blocks = []
        for i, ls in enumerate(spec.layers):
            block_cls = part_class("block", ls.block)
            roles = dict(block_cls.roles)
            missing = sorted(set(roles) - set(ls.parts))
            unexpected = sorted(set(ls.parts) - set(roles))
            if missing or unexpected:
                raise ValueError(f"layer {i}: a {ls.block!r} block is made of {sorted(roles)}; "
                                 f"missing {missing}, unexpected {unexpected}")
            self.blocks.append(block_cls({role: build_part(family, ls.parts[role]) for role, family in roles.items()}))
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self.plan, self.cache_groups = self._plan_cache()
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None

    # ------------------------------------------------------------------
    def _plan_cache(self) -> Tuple[List[PlannedStep], List[object]]:
        keys: List[object] = []            # need of each group
        planes: List[int] = []             # planes of each group
        plan: List[PlannedStep] = []
        for i, rs in enumerate(self.spec.order):
            if not (0 <= rs.layer < len(self.blocks)):
                raise ValueError(f"run order entry {i} names layer {rs.layer}, which does not exist")
            if rs.cache is not None and not (0 <= rs.cache < i):
                raise ValueError(f"run order entry {i} reads the cache of entry {rs.cache}, which is not earlier")
            caches: Dict[str, PlannedCache] = {}
            for role, mixer in self.blocks[rs.layer].mixers():
                need = mixer.cache_need()
                if need is None:
                    caches[role] = PlannedCache(None, 0, False)
                    continue
                if rs.cache is not None:
                    src = plan[rs.cache].caches.get(role)
                    if src is None or src.group is None or keys[src.group] != need or not src.writable:
                        raise ValueError(f"run order entry {i} cannot read the cache of entry {rs.cache}: "
                                         "the needs differ or that entry owns no plane")
                    caches[role] = PlannedCache(src.group, src.plane, False)
                    continue
                if need in keys:
                    g = keys.index(need)
                else:
                    keys.append(need)
                    planes.append(0)
                    g = len(keys) - 1
                caches[role] = PlannedCache(g, planes[g], True)
                planes[g] += 1
            plan.append(PlannedStep(rs.layer, caches))
        groups: List[object] = []
        for need, n in zip(keys, planes):
            if isinstance(need, PagedKVNeed):
                vd = need.head_dim if need.value_head_dim is None else need.value_head_dim
                groups.append(PagedGroupSpec(need.num_kv_heads, need.head_dim, need.window, n, vd))
            elif isinstance(need, StateNeed):
                groups.append(StateGroupSpec(tuple(need.shape), need.dtype, n))
            else:
                raise TypeError(f"a mixer asked for {need!r}; PagedKVNeed, StateNeed or None are understood")
        return plan, groups

    # ------------------------------------------------------------------
    def _all_parts(self):
        yield self.embedding
        for b in self.blocks:
            for p in b.parts():
                yield p
        yield self.final_norm
        yield self.head

    def declared_tensors(self) -> Dict[str, TensorDecl]:
        """Full checkpoint name -> declaration, for every part."""
        out: Dict[str, TensorDecl] = {}
        for part in self._all_parts():
            for rel, decl in part.tensors().items():
                name = part.prefix + rel
                if name in out and out[name] != decl:
                    raise ValueError(f"tensor {name} is declared twice with different shapes")
                out[name] = decl
        return out

    def load(self, fetch: Callable[[str], Optional[torch.Tensor]], dtype: torch.dtype, device: torch.device) -> None:
        self.dtype, self.device = dtype, device
        for part in self._all_parts():
            prefix = part.prefix
            part.load(lambda rel, _p=prefix: fetch(_p + rel), dtype, device)
        tied = getattr(self.head, "tied_to", None)
        if tied is not None:
            if tied != self.embedding.prefix + "weight":
                raise ValueError(f"the head is tied to {tied}, which is not the embedding table")
            self.head.tie(self.embedding.weight)
        for b in self.blocks:
            for _role, mixer in b.mixers():
                mixer.prepare(device, dtype)

    def kernel_libraries(self) -> List[str]:
        libs: List[str] = []
        for part in self._all_parts():
            for name in part.kernel_libraries():
                if name not in libs:
                    libs.append(name)
        return libs

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a step reads once: every layer that runs, the final norm and the head."""
        n = 0
        for ps in self.plan:
            blk = self.blocks[ps.layer]
            for part in blk.parts():
                if hasattr(part, "weight_bytes"):
                    n += part.weight_bytes()
                elif getattr(part, "weight", None) is not None:
                    n += part.weight.numel() * part.weight.element_size()
        n += self.final_norm.weight.numel() * self.final_norm.weight.element_size()
        n += self.head.weight.numel() * self.head.weight.element_size()
        return n

    # ------------------------------------------------------------------
    def forward(self, step, storage) -> Optional[torch.Tensor]:
        """Run the step's tokens through every run-step; float32 logits [wanted rows, vocab]."""
        n = step.num_tokens
        h = self.embedding.forward(step.token_ids, n, step.status)
        delta = None
        for ps in self.plan:
            caches = {}
            for role, pc in ps.caches.items():
                if pc.group is None:
                    caches[role] = None
                elif self.cache_groups[pc.group].kind == "paged":
                    caches[role] = storage.paged_view(pc.group, pc.plane, step.slot_maps[pc.group], pc.writable)
                else:
                    caches[role] = storage.state_view(pc.group, pc.plane, pc.writable)
            h, delta = self.blocks[ps.layer].forward(h, delta, step, caches)
        if step.num_logits == 0:
            return None
        x = self.final_norm.add_forward(h, delta, rows=step.logit_rows)
        return self.head.forward(x)
