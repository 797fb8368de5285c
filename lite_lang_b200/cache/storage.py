"""Device side of the cache: page pools, block-table mirrors, state records.

Layout of a paged group: keys and values are separate tensors
``[planes, num_pages, kv_heads, page_size, width]`` so that the keys of one
(page, kv head) are one contiguous tile; the width of the values may differ from
the keys', and a group whose mixers keep one vector per token has no value tensor.  The reference stores
``[layers, tokens, 2*kv_heads, head_dim]`` with one token per slot
(``litelang/models/cache.py:196-205``).

The block tables are decided on the host (``CacheManager``); ``sync`` pushes the
rows that changed since the last step and zeroes the state records of request
slots opened since then.  Rows travel through pinned staging buffers guarded by
events, so the host may run ahead of the device.

The pools start as zeros.  No kernel may depend on that, nor on what an earlier
owner left in a page: with ``LITE_LANG_B200_CACHE_FILL=nan`` in the environment
the pools start as NaN instead, and the results must be the same (the replay
tests run that way).
"""

from __future__ import annotations

from dataclasses import dataclass
import os
from typing import Dict, List, Optional

import torch

from .manager import CacheManager

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@dataclass
class PagedKVView:
    """What a mixer sees of its cache plane during one step."""

    k: torch.Tensor              # [num_pages, kv_heads, page_size, head_dim]
    v: Optional[torch.Tensor]    # [num_pages, kv_heads, page_size, value width], None if the group keeps no values
    block_table: torch.Tensor    # int32 [request slots, max_blocks]
    slot_map: Optional[torch.Tensor]   # int32 [tokens]: where each new token's k/v go
    page_size: int
    writable: bool
    group: int
    plane: int


@dataclass
class StateView:
    """A mixer's fixed-size records: ``state[slot]`` belongs to the request in that slot."""

    state: torch.Tensor          # [request slots, *shape]
    group: int
    plane: int
    writable: bool = True


class CacheStorage:
    def __init__(self, manager: CacheManager, dtype: torch.dtype, device: torch.device):
        self.manager = manager
        self.device = device
        self.dtype = dtype
        self.k: Dict[int, torch.Tensor] = {}
        self.v: Dict[int, torch.Tensor] = {}
        self.block_table: Dict[int, torch.Tensor] = {}
        self.state: Dict[int, torch.Tensor] = {}
        self._stage: Dict[int, List[torch.Tensor]] = {}
        self._stage_events: Dict[int, List[Optional[torch.cuda.Event]]] = {}
        self._stage_turn: Dict[int, int] = {}
        pinned = device.type == "cuda"
        for g in manager.paged_ids:
            spec = manager.groups[g]
            n = manager.allocators[g].num_pages
            shape = (spec.planes, n, spec.num_kv_heads, manager.page_size)
            fill = float("nan") if os.environ.get("LITE_LANG_B200_CACHE_FILL", "") == "nan" else 0.0
            self.k[g] = torch.full(shape + (spec.head_dim,), fill, dtype=dtype, device=device)
            if spec.value_dim > 0:
                self.v[g] = torch.full(shape + (spec.value_dim,), fill, dtype=dtype, device=device)
            self.block_table[g] = torch.full((manager.max_requests, manager.max_blocks), -1, dtype=torch.int32,
                                             device=device)
            self._stage[g] = [torch.empty((manager.max_requests, manager.max_blocks), dtype=torch.int32,
                                          pin_memory=pinned) for _ in range(2)]
            self._stage_events[g] = [None, None]
            self._stage_turn[g] = 0
        for g in manager.state_ids:
            spec = manager.groups[g]
            dt = dtype if spec.dtype == "compute" else _TORCH_DTYPES[spec.dtype]
            self.state[g] = torch.zeros((spec.planes, manager.max_requests) + tuple(spec.shape), dtype=dt,
                                        device=device)

    def bytes(self) -> int:
        n = 0
        for t in list(self.k.values()) + list(self.v.values()) + list(self.state.values()):
            n += t.numel() * t.element_size()
        return n

    def sync(self) -> None:
        """Bring the device in line with the manager before a step is launched."""
        m = self.manager
        opened = m.take_opened_slots()
        if opened and self.state:
            idx = torch.tensor(opened, dtype=torch.long, device=self.device)
            for g, st in self.state.items():
                st.index_fill_(1, idx, 0)
        for g in m.paged_ids:
            rows = m.take_dirty_rows(g)
            if not rows:
                continue
            turn = self._stage_turn[g]
            self._stage_turn[g] = 1 - turn
            ev = self._stage_events[g][turn]
            if ev is not None:
                ev.synchronize()
            stage = self._stage[g][turn]
            host = m.block_tables[g]
            dev = self.block_table[g]
            if len(rows) * 4 >= m.max_requests:
                stage.copy_(torch.from_numpy(host))
                dev.copy_(stage, non_blocking=True)
            else:
                for i, r in enumerate(rows):
                    stage[i].copy_(torch.from_numpy(host[r]))
                    dev[r].copy_(stage[i], non_blocking=True)
            if self.device.type == "cuda":
                if self._stage_events[g][turn] is None:
                    self._stage_events[g][turn] = torch.cuda.Event()
                self._stage_events[g][turn].record()

    def paged_view(self, group: int, plane: int, slot_map: Optional[torch.Tensor], writable: bool) -> PagedKVView:
        v = self.v.get(group)
        return PagedKVView(self.k[group][plane], None if v is None else v[plane], self.block_table[group],
                           slot_map if writable else None, self.manager.page_size, writable, group, plane)

    def state_view(self, group: int, plane: int, writable: bool = True) -> StateView:
        return StateView(self.state[group][plane], group, plane, writable)
