"""Token choice: greedy and temperature sampling.

The reference always takes ``logits.argmax`` (``litelang/models/qwen2/layer/
post_layer.py:75-77``); its sampler with temperature, top-p and top-k is
commented out (``post_layer.py:47-73``) although the request fields
``temperature``, ``top_p``, ``top_k`` and ``do_sample`` exist
(``litelang/apis/api_server.py:16-31``).  Here ``temperature == 0`` or
``do_sample == False`` is greedy (ties to the lowest index); otherwise the token
is drawn from softmax(logits / temperature) by inverse CDF in index order.

The uniform number of a draw comes from a counter-based generator keyed by
(seed, request id, index of the token in the request's output), so a sample
does not depend on what else is in the batch or on how prompts were cut.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops

_MASK = (1 << 64) - 1


def _mix(x: int) -> int:
    """splitmix64 finaliser."""
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform_for(seed: int, request_id: int, token_index: int) -> float:
    """A number in [0, 1) that depends on the three keys only (24 random bits: exact in float32)."""
    x = _mix(seed & _MASK)
    x = _mix(x ^ (request_id & _MASK))
    x = _mix(x ^ (token_index & _MASK))
    return (x >> 40) / float(1 << 24)


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0          # accepted for the reference's request format; 1.0 is the only value built
    top_k: int = -1             # likewise; -1 (off) or 1 (greedy)
    do_sample: bool = True      # False forces greedy, as in the reference's request format
    max_new_tokens: Optional[int] = None
    ignore_eos: bool = False
    seed: Optional[int] = None

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        if self.top_p != 1.0:
            raise ValueError("top_p other than 1.0 is not built (the reference's top-p code is disabled too)")
        if self.top_k not in (-1, 0, 1):
            raise ValueError("top_k other than 1 (greedy) or -1 (off) is not built")

    @property
    def greedy(self) -> bool:
        return (not self.do_sample) or self.temperature == 0.0 or self.top_k == 1


class Sampler:
    """Runs the sampling kernel on the rows of a step's logits."""

    def __init__(self, device: torch.device, max_rows: int, out: Optional[torch.Tensor] = None):
        self.device = device
        self.max_rows = max_rows
        self.out = out if out is not None else torch.zeros(max_rows, dtype=torch.int32, device=device)
        pinned = device.type == "cuda"
        # a ring of host buffers: a step may be prepared while the copy of the step before has not run yet
        self._hosts = [torch.zeros((2, max_rows), dtype=torch.float32, pin_memory=pinned) for _ in range(4)]
        self._turn = 0
        self._dev = torch.zeros((2, max_rows), dtype=torch.float32, device=device)

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], uniforms: Sequence[float]) -> torch.Tensor:
        """Device int32 tokens for each row.  temperatures[i] <= 0 means greedy."""
        n = logits.shape[0]
        if n > self.max_rows:
            raise ValueError("more rows than the sampler was sized for")
        if all(t <= 0 for t in temperatures):
            ops.sample(logits, self.out, None, None, n)
            return self.out[:n]
        host = self._hosts[self._turn]
        self._turn = (self._turn + 1) % len(self._hosts)
        h = host.numpy()
        h[0, :n] = np.asarray(temperatures, dtype=np.float32)
        h[1, :n] = np.asarray(uniforms, dtype=np.float32)
        self._dev.copy_(host, non_blocking=True)
        ops.sample(logits, self.out, self._dev[0], self._dev[1], n)
        return self.out[:n]
