"""Weights from safetensors, by tensor name.

The reference walks an index file or ``model.safetensors``, puts every tensor
into a CPU dict and lets each layer pick its names, with a bare ``KeyError`` on
a missing one (``litelang/models/qwen2/model.py:61-97``,
``qwen2/layer_weights/load_weights.py:87-172``).  Here the model *declares* the
tensors it reads (full name, shape, role); the checkpoint's names and shapes are
compared with that declaration before anything is read, and every problem
(missing, unexpected, wrong shape) is reported in one error.

How tensors are kept on the device: matrices and embedding tables in the
engine's dtype (bfloat16, or float32 on the 32-bit path); norm weights and
biases in float32, which is exact for bfloat16 checkpoints and leaves a tensor
stored in 32-bit as it is; integer tables as int32.
"""

from __future__ import annotations

import json
import os
from typing import Callable, Dict, List, Mapping, Optional, Tuple

import torch
from safetensors import safe_open


class WeightError(RuntimeError):
    """The checkpoint does not fit the model; the message lists every misfit."""


class Checkpoint:
    """Names, shapes and lazy reads of a folder's safetensors files (each file opened once)."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        files: List[str]
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as fh:
                weight_map = json.load(fh)["weight_map"]
            files = sorted(set(weight_map.values()))
        elif os.path.isfile(single):
            files = ["model.safetensors"]
        else:
            raise WeightError(f"{model_dir!r} holds neither model.safetensors nor model.safetensors.index.json")
        self._handles = {}
        self._where: Dict[str, str] = {}
        self.shapes: Dict[str, Tuple[int, ...]] = {}
        for f in files:
            path = os.path.join(model_dir, f)
            if not os.path.isfile(path):
                raise WeightError(f"the index names {f!r}, which is not in {model_dir!r}")
            h = safe_open(path, framework="pt")
            self._handles[f] = h
            for name in h.keys():
                self._where[name] = f
                self.shapes[name] = tuple(h.get_slice(name).get_shape())

    def names(self) -> List[str]:
        return sorted(self._where)

    def get(self, name: str) -> torch.Tensor:
        return self._handles[self._where[name]].get_tensor(name)


def check_against(declared: Mapping[str, object], shapes: Mapping[str, Tuple[int, ...]], where: str) -> None:
    """Raise one WeightError that lists missing, unexpected and wrongly shaped tensors."""
    missing = [n for n, d in declared.items() if n not in shapes and not d.optional]
    unexpected = [n for n in shapes if n not in declared]
    wrong = [(n, tuple(d.shape), tuple(shapes[n])) for n, d in declared.items()
             if n in shapes and tuple(shapes[n]) != tuple(d.shape)]
    if not (missing or unexpected or wrong):
        return
    lines = [f"the weights in {where} do not fit the model:"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): "
                     + "; ".join(f"{n} expected {list(e)} found {list(f)}" for n, e, f in sorted(wrong)))
    raise WeightError("\n".join(lines))


def load_weights(model, model_dir: str, dtype: torch.dtype, device: torch.device) -> None:
    """Check the folder's tensors against ``model.declared_tensors()`` and load every part."""
    ckpt = Checkpoint(model_dir)
    declared = model.declared_tensors()
    check_against(declared, ckpt.shapes, repr(model_dir))

    def fetch(name: str) -> Optional[torch.Tensor]:
        return ckpt.get(name) if name in ckpt.shapes else None

    model.load(fetch, dtype, device)
