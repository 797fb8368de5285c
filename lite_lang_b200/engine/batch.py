"""The descriptor of one step: a flat batch of (request, its next tokens).

The reference's descriptor is ``RunnerBatch`` (``litelang/models/runner_batch.py:
8-35,88-102``): flat tokens, ``position_ids``, ``b_start_idx``, ``b_seq_len``,
``b_shared_seq_len`` and the cache slot ids, built from Python lists with six
host-to-device copies per step, and a step is either all prompts or all single
tokens.  Here an entry is any portion of a request (a whole prompt, a piece of
one, a decoded token), all index arrays of a step live in one pinned buffer that
goes to the device in one copy, and single-token entries are put first so that
kernels specialised for them can take a prefix of the batch.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..parts.base import StepView


@dataclass
class StepEntry:
    """One request's part in a step."""

    slot: int                          # request slot in the cache manager
    tokens: Sequence[int]              # its next tokens (at least one)
    want: Sequence[int] = ()           # places among `tokens` whose logits are asked for
    feed: int = -1                     # >= 0 (single-token entries only): the token is not known to the host yet,
                                       # it is the feed-th token sampled by the step before and is taken on the device


class StepBatch(StepView):
    """Device arrays and host facts of the running step (what parts may read)."""

    num_tokens: int                    # tokens in the arrays (padding included)
    num_entries: int                   # entries in the arrays (padding included)
    real_tokens: int
    real_entries: int
    num_single: int                    # leading entries that bring exactly one token
    num_logits: int
    token_ids: torch.Tensor            # int32 [num_tokens]
    positions: torch.Tensor            # int32 [num_tokens] position of each token in its request
    token_req: torch.Tensor            # int32 [num_tokens] entry index of each token
    feed: torch.Tensor                 # int32 [num_tokens] place in the last step's sampled tokens, or -1
    has_feed: bool                     # some token of the step is taken from the last step's results
    entry_ctx: list                    # host copy of ctx_len for the real entries
    cu_q: torch.Tensor                 # int32 [num_entries + 1] first token of each entry
    ctx_len: torch.Tensor              # int32 [num_entries] tokens cached before this step
    req_slot: torch.Tensor             # int32 [num_entries] request slot (-1: padding)
    logit_rows: torch.Tensor           # int32 [num_logits] token rows whose logits are wanted
    slot_maps: Dict[int, torch.Tensor]  # per paged group: int32 [num_tokens] cache slot of each token
    status: Optional[torch.Tensor]     # int32 [1] error word of the kernels
    max_q_len: int
    max_kv_len: int
    entries: List[StepEntry]           # in the order of the arrays
    scratch: dict                      # per-step memo for parts (e.g. split plans shared by all layers)


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class BatchBuilder:
    """Builds ``StepBatch`` objects in fixed device buffers (so that steps can be captured)."""

    def __init__(self, manager: CacheManager, max_tokens: int, max_entries: int, device: torch.device,
                 status: Optional[torch.Tensor] = None, ring: int = 3):
        self.manager = manager
        self.max_tokens = int(max_tokens)
        self.max_entries = int(max_entries)
        self.device = device
        self.status = status
        T, R = _align(self.max_tokens), _align(self.max_entries + 1)
        self._off: Dict[str, Tuple[int, int]] = {}
        off = 0
        for name, size in (("token_ids", T), ("positions", T), ("token_req", T), ("logit_rows", T), ("feed", T),
                           ("cu_q", R), ("ctx_len", R), ("req_slot", R)):
            self._off[name] = (off, size)
            off += size
        for g in manager.paged_ids:
            self._off[f"slot_map{g}"] = (off, T)
            off += T
        self.total = off
        pinned = device.type == "cuda"
        self._host = [torch.zeros(self.total, dtype=torch.int32, pin_memory=pinned) for _ in range(ring)]
        self._events: List[Optional[torch.cuda.Event]] = [None] * ring
        self._turn = 0
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=device)

    def _view(self, buf, name: str, n: Optional[int] = None):
        off, size = self._off[name]
        return buf[off:off + (size if n is None else n)]

    def build(self, entries: Sequence[StepEntry], pad_entries: Optional[int] = None,
              views: bool = True) -> StepBatch:
        """Fill the buffers for ``entries`` and start their copy to the device.

        ``views=False`` leaves out the device views of the arrays (a replayed graph already holds them).

        Single-token entries come first in the arrays; ``logit_rows`` keeps the
        caller's order of entries and of their ``want`` lists.  ``pad_entries``
        pads a step of single-token entries up to that many entries with
        entries of slot -1, which kernels skip.
        """
        m = self.manager
        ps = m.page_size
        n_real = len(entries)
        num_single = sum(1 for e in entries if len(e.tokens) == 1)
        if num_single == n_real:
            order, arranged, t_real = range(n_real), list(entries), n_real
        else:
            order = sorted(range(n_real), key=lambda i: 0 if len(entries[i].tokens) == 1 else 1)
            arranged = [entries[i] for i in order]
            t_real = sum(len(e.tokens) for e in arranged)
        n_all, t_all = n_real, t_real
        if pad_entries is not None:
            if num_single != n_real:
                raise ValueError("only steps of single-token entries can be padded")
            n_all = max(n_real, pad_entries)
            t_all = t_real + (n_all - n_real)
        if n_all > self.max_entries or t_all > self.max_tokens:
            raise ValueError(f"step of {n_all} entries / {t_all} tokens exceeds the builder's "
                             f"{self.max_entries} / {self.max_tokens}")
        if n_all == 0:
            raise ValueError("a step needs at least one entry")

        turn = self._turn
        self._turn = (turn + 1) % len(self._host)
        if self._events[turn] is not None:
            self._events[turn].synchronize()
        host = self._host[turn]
        h = host.numpy()

        def hv(name):
            off, size = self._off[name]
            return h[off:off + size]

        token_ids, positions, token_req = hv("token_ids"), hv("positions"), hv("token_req")
        cu_q, ctx_len, req_slot, logit_rows = hv("cu_q"), hv("ctx_len"), hv("req_slot"), hv("logit_rows")
        slot_maps = {g: hv(f"slot_map{g}") for g in m.paged_ids}
        feed = hv("feed")
        feed[:t_all] = -1

        t = 0
        max_q, max_kv = 1, 1
        starts = []
        if num_single == n_real and n_real > 0:
            # a decode step: every entry brings one token; filled with array operations, no loop
            slots = np.fromiter((e.slot for e in arranged), dtype=np.int64, count=n_real)
            ctx = m.lengths[slots]
            cu_q[:n_real] = np.arange(n_real, dtype=np.int32)
            ctx_len[:n_real] = ctx
            req_slot[:n_real] = slots
            token_ids[:n_real] = np.fromiter((e.tokens[0] for e in arranged), dtype=np.int32, count=n_real)
            feed[:n_real] = np.fromiter((e.feed for e in arranged), dtype=np.int32, count=n_real)
            positions[:n_real] = ctx
            token_req[:n_real] = cu_q[:n_real]
            for g in m.paged_ids:
                pages = m.block_tables[g][slots, ctx // ps]
                if (pages < 0).any():
                    raise RuntimeError("a decode step without reserved pages")
                slot_maps[g][:n_real] = pages * ps + ctx % ps
            starts = list(range(n_real))
            t = n_real
            max_kv = int(ctx.max()) + 1
            arranged_loop = ()
        else:
            arranged_loop = arranged
        for i, e in enumerate(arranged_loop):
            q = len(e.tokens)
            if q == 0:
                raise ValueError("an entry without tokens")
            if e.feed >= 0:
                if q != 1:
                    raise ValueError("only a single-token entry can take its token from the step before")
                feed[t] = e.feed
            c = m.length(e.slot)
            starts.append(t)
            cu_q[i] = t
            ctx_len[i] = c
            req_slot[i] = e.slot
            token_ids[t:t + q] = np.asarray(e.tokens, dtype=np.int32)
            pos = np.arange(c, c + q, dtype=np.int32)
            positions[t:t + q] = pos
            token_req[t:t + q] = i
            for g in m.paged_ids:
                pages = m.block_tables[g][e.slot, pos // ps]
                if (pages < 0).any():
                    raise RuntimeError(f"slot {e.slot}: pages for positions {c}..{c + q - 1} are not reserved")
                slot_maps[g][t:t + q] = pages * ps + pos % ps
            t += q
            max_q = max(max_q, q)
            max_kv = max(max_kv, c + q)
        if n_all > n_real:                    # padding entries, one token each
            pad = n_all - n_real
            cu_q[n_real:n_all] = np.arange(t, t + pad, dtype=np.int32)
            ctx_len[n_real:n_all] = 0
            req_slot[n_real:n_all] = -1
            token_ids[t:t + pad] = 0
            positions[t:t + pad] = 0
            token_req[t:t + pad] = np.arange(n_real, n_all, dtype=np.int32)
            for g in m.paged_ids:
                slot_maps[g][t:t + pad] = -1
            t += pad
        cu_q[n_all] = t

        new_index = {orig: i for i, orig in enumerate(order)}
        k = 0
        for orig, e in enumerate(entries):
            for w in e.want:
                if not (0 <= w < len(e.tokens)):
                    raise ValueError(f"wanted place {w} lies outside an entry of {len(e.tokens)} tokens")
                logit_rows[k] = starts[new_index[orig]] + w
                k += 1
        num_logits = k
        if pad_entries is not None:
            for i in range(k, n_all):   # a captured step computes a fixed number of rows
                logit_rows[i] = 0

        self.dev.copy_(host, non_blocking=True)
        if self.device.type == "cuda":
            if self._events[turn] is None:
                self._events[turn] = torch.cuda.Event()
            self._events[turn].record()

        b = StepBatch()
        b.num_tokens, b.num_entries = t_all, n_all
        b.real_tokens, b.real_entries = t_real, n_real
        b.num_single = num_single if pad_entries is None else n_all
        b.num_logits = num_logits if pad_entries is None else n_all
        b.real_logits = num_logits
        b.status = self.status
        b.max_q_len, b.max_kv_len = max_q, max_kv
        b.entries = arranged
        b.scratch = {}
        b.has_feed = bool((feed[:t_all] >= 0).any())
        b.entry_ctx = [int(c) for c in ctx_len[:n_real]]       # host copy: tokens cached before the step, per entry
        if not views:
            return b
        d = self.dev
        b.token_ids = self._view(d, "token_ids", t_all)
        b.positions = self._view(d, "positions", t_all)
        b.token_req = self._view(d, "token_req", t_all)
        b.feed = self._view(d, "feed", t_all)
        b.cu_q = self._view(d, "cu_q", n_all + 1)
        b.ctx_len = self._view(d, "ctx_len", n_all)
        b.req_slot = self._view(d, "req_slot", n_all)
        b.logit_rows = self._view(d, "logit_rows", b.num_logits)
        b.slot_maps = {g: self._view(d, f"slot_map{g}", t_all) for g in m.paged_ids}
        return b
