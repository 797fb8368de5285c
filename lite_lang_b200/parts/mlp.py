"""SiLU-gated feed-forward: down(silu(gate(x)) * up(x)), no biases.

``litelang/models/qwen2/layer/transformer_layer.py:79-83``; gate and up are fused
into one projection whose first I columns are the gate
(``litelang/models/qwen2/layer_weights/load_weights.py:160-172``).  The
activation is evaluated in float32 (``litelang/kernel/develop_silu_and_mul/
silu_and_mul.py:43-50`` rounds the gate's SiLU first; here the whole expression is
rounded once).
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import FeedForward, NormSplit, TensorDecl, register_part


class GatedMLP(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden_size = int(spec.params["hidden_size"])
        self.intermediate_size = int(spec.params["intermediate_size"])
        act = spec.params.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"gated_mlp: activation {act!r} is not built (only 'silu')")
        self.w_gate_up = None
        self.w_down = None

    def tensors(self) -> Dict[str, TensorDecl]:
        h, i = self.hidden_size, self.intermediate_size
        return {
            "gate_proj.weight": TensorDecl((i, h)),
            "up_proj.weight": TensorDecl((i, h)),
            "down_proj.weight": TensorDecl((h, i)),
        }

    def load(self, fetch, dtype, device) -> None:
        gate = fetch("gate_proj.weight").to(dtype)
        up = fetch("up_proj.weight").to(dtype)
        self.w_gate_up = torch.cat((gate, up), dim=0).to(device).contiguous()
        self.w_down = fetch("down_proj.weight").to(dtype).to(device).contiguous()

    def kernel_libraries(self):
        bf16 = self.w_down is not None and self.w_down.dtype == torch.bfloat16
        return ["core", "gemm_smallm", "gemm_stream", "gemm_tc", "gemm_pair"] if bf16 else ["core"]

    def weight_bytes(self) -> int:
        return self.w_gate_up.numel() * self.w_gate_up.element_size() + self.w_down.numel() * self.w_down.element_size()

    accumulates = True
    takes_norm_split = True

    def accepts_norm_split(self, rows) -> bool:
        return ops.gated_scaled_supported(rows, self.w_gate_up)

    def forward(self, x, step, residual=None):
        if isinstance(x, NormSplit):    # the norm before this part, left to its first product
            act = ops.gemm_stream_gated_scaled(x.scaled, self.w_gate_up, x.sumsq, x.eps, step.status)
        else:
            act = ops.gated_linear(x, self.w_gate_up)
        if residual is not None and ops.accumulate_preferred(act, self.w_down):
            ops.linear_accumulate(act, self.w_down, residual)
            return None
        return ops.linear(act, self.w_down, partial_ok=True)


register_part("feed_forward", "gated_mlp", GatedMLP)
