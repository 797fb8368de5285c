"""RMSNorm part: y = x / sqrt(mean(x^2) + eps) * w, computed in float32.

Formula: ``litelang/kernel/develop_rmsnorm/rms_norm.py:11-17,43-53``; used before
the mixer, before the feed-forward and before the lm_head
(``litelang/models/qwen2/layer/transformer_layer.py:86-92``, ``post_layer.py:43-45``).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import Norm, TensorDecl, register_part


class RMSNorm(Norm):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden_size = int(spec.params["hidden_size"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((self.hidden_size,), "norm")}

    def load(self, fetch, dtype, device) -> None:
        self.weight = fetch("weight").to(torch.float32).to(device).contiguous()

    def split_params(self):
        return self.weight, self.eps

    def forward(self, x, out=None):
        if out is None:
            out = torch.empty_like(x)
        ops.rmsnorm(out, x, self.weight, self.eps)
        return out

    def add_forward(self, residual, delta, rows=None):
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, residual.shape[1]), dtype=residual.dtype, device=residual.device)
        ops.add_rmsnorm(out, residual, delta, self.weight, self.eps, rows)
        return out


register_part("norm", "rms_norm", RMSNorm)
