"""Token embedding and the lm_head.

Embedding: ``litelang/models/qwen2/layer/pre_layer.py:15-19``.  Head:
``litelang/models/qwen2/layer/post_layer.py:20-22``; with tied embeddings it is
the embedding table itself (``layer_weights/post_layer_weights.py:10-15``), kept
as one buffer.  Logits are float32 on both paths.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import Part, TensorDecl, register_part


class TokenEmbedding(Part):
    kind_family = "embedding"

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab_size = int(spec.params["vocab_size"])
        self.hidden_size = int(spec.params["hidden_size"])
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((self.vocab_size, self.hidden_size))}

    def load(self, fetch, dtype, device) -> None:
        self.weight = fetch("weight").to(dtype).to(device).contiguous()

    def forward(self, token_ids: torch.Tensor, num_tokens: int, status) -> torch.Tensor:
        out = torch.empty((num_tokens, self.hidden_size), dtype=self.weight.dtype, device=self.weight.device)
        ops.embed_gather(out, self.weight, token_ids[:num_tokens], status)
        return out


class LMHead(Part):
    kind_family = "head"

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab_size = int(spec.params["vocab_size"])
        self.hidden_size = int(spec.params["hidden_size"])
        self.tied_to = spec.params.get("tied_to")
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorDecl]:
        # With tied embeddings a checkpoint may or may not repeat the table under lm_head.
        return {"weight": TensorDecl((self.vocab_size, self.hidden_size), optional=self.tied_to is not None)}

    def load(self, fetch, dtype, device) -> None:
        if self.tied_to is None:
            self.weight = fetch("weight").to(dtype).to(device).contiguous()

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, out_dtype=torch.float32)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
