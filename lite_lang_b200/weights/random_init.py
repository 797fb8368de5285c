"""Random weights: a model folder (config.json, model.safetensors) from a configuration and a seed.

The reference has no such mode (its benchmarks need a real checkpoint,
``test/generate_token.py:24-40``).  Each tensor is drawn from its own generator,
seeded by the seed and the tensor's name, so a tensor's values do not depend on
which other tensors exist or in which order they are made: matrices
N(0, s_matrix), biases N(0, s_bias), norm weights 1 + N(0, s_norm), rounded to
the checkpoint dtype.
"""

from __future__ import annotations

import json
import os
import zlib
from typing import Callable, Dict, Mapping, Optional

import torch
from safetensors.torch import save_file

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def draw_tensor(name: str, decl, seed: int, scales: Mapping[str, float], dtype: torch.dtype,
                device: str = "cpu") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) % (2 ** 63))
    shape = tuple(decl.shape)
    if decl.role == "norm":
        t = 1.0 + scales["norm"] * torch.randn(shape, generator=gen, dtype=torch.float32, device=device)
    elif decl.role == "bias":
        t = scales["bias"] * torch.randn(shape, generator=gen, dtype=torch.float32, device=device)
    elif decl.role == "table":
        return torch.randint(0, 2 ** 15, shape, generator=gen, dtype=torch.int32, device=device)
    else:
        t = scales["matrix"] * torch.randn(shape, generator=gen, dtype=torch.float32, device=device)
    return t.to(dtype)


def random_fetch(model, seed: int, scales: Mapping[str, float], dtype: torch.dtype,
                 device: str = "cpu") -> Callable[[str], Optional[torch.Tensor]]:
    """A ``fetch(full_name)`` that draws declared, non-optional tensors on demand."""
    declared = model.declared_tensors()

    def fetch(name: str):
        d = declared.get(name)
        if d is None or d.optional:
            return None
        return draw_tensor(name, d, seed, scales, dtype, device)

    return fetch


def write_random_model(folder: str, config, seed: int, scales: Optional[Mapping[str, float]] = None,
                       dtype: Optional[str] = None) -> str:
    """Write ``folder/config.json`` and ``folder/model.safetensors`` for ``config``; returns the folder."""
    from ..engine.model import CausalLM

    os.makedirs(folder, exist_ok=True)
    d = config.to_dict()
    if dtype is not None:
        d["torch_dtype"] = dtype
    store = _DTYPES[d.get("torch_dtype", "bfloat16")]
    sc = dict(config.init_scales())
    if scales:
        sc.update(scales)
    model = CausalLM(config.model_spec())
    tensors: Dict[str, torch.Tensor] = {}
    for name, decl in model.declared_tensors().items():
        if decl.optional:
            continue
        tensors[name] = draw_tensor(name, decl, seed, sc, store).contiguous()
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(d, fh, indent=1)
    return folder
