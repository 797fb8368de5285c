"""How many pages each cache group gets from a budget of bytes.

The reference sizes its one pool as ``free memory * mem_usage / 2`` over the bytes of a token
(``litelang/models/cache.py:185-194,218-223``).  Here the budget is first reduced by the fixed-size state
records (they exist for every request slot, used or not); the rest is shared out so that every group can
hold the same number of *requests' worth* of context: a group that keeps every position gets N pages, a
group with a window no more than its requests can ever hold (window + the tokens of one step, for every
request slot), and what that saves goes to the others.
"""

from __future__ import annotations

import math
from typing import List, Sequence

_ELT = {"float32": 4, "bfloat16": 2}


def page_bytes(group, page_size: int, elt: int) -> int:
    """Bytes of one page of a paged group, over all its planes (keys and values)."""
    return group.planes * group.num_kv_heads * page_size * (group.head_dim + group.value_dim) * elt


def state_bytes(group, max_requests: int, elt: int) -> int:
    """Bytes of a state group: one record per request slot and plane."""
    size = elt if group.dtype == "compute" else _ELT[group.dtype]
    return group.planes * max_requests * int(math.prod(group.shape)) * size


def plan_pages(groups: Sequence[object], budget_bytes: int, page_size: int, elt: int, max_requests: int,
               max_model_len: int, step_tokens: int) -> List[int]:
    """Pages for each paged group (in the order of the groups), at least one each."""
    paged = [g for g in groups if g.kind == "paged"]
    if not paged:
        return []
    budget = budget_bytes - sum(state_bytes(g, max_requests, elt) for g in groups if g.kind == "state")
    most = [max_requests * g.pages_a_request_needs(max_model_len, page_size, step_tokens) for g in paged]
    bpp = [page_bytes(g, page_size, elt) for g in paged]
    pages = [0] * len(paged)
    open_ids = list(range(len(paged)))
    # water-filling: the same N for every group, except that a group stops at what its requests can ever use
    while open_ids:
        n = max(0, budget) // max(1, sum(bpp[i] for i in open_ids))
        capped = [i for i in open_ids if most[i] <= n]
        if not capped:
            for i in open_ids:
                pages[i] = n
            break
        for i in capped:
            pages[i] = most[i]
            budget -= most[i] * bpp[i]
            open_ids.remove(i)
    return [max(1, p) for p in pages]
