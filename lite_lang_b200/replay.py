"""Trace replay: feeds given token ids through a model step by step and writes logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

It samples nothing and has no forward pass, cache or loader of its own: it
drives the model, step function, cache manager and kernels that generation uses.
Steps come on standard input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``DIR/<step>.f32`` receives the logits
at the wanted places, in the order of the entries and of ``want``, as
little-endian float32 [wanted, vocab].  After every step a line ``done <step>``
is printed and flushed.  ``--max-tokens`` sizes the cache pool: the most tokens
that live requests hold at any time, each request's count rounded up to a
multiple of 64, so pages are used again when requests end.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True, dest="max_tokens")
    ap.add_argument("--page-size", type=int, default=16, dest="page_size",
                    help="tokens per cache page (default 16; must divide 64 or be a multiple of it)")
    ap.add_argument("--max-requests", type=int, default=8, dest="max_requests")
    ap.add_argument("--no-cuda-graphs", action="store_true", dest="no_graphs")
    args = ap.parse_args(argv)

    import torch
    from . import models as _models  # noqa: F401
    from .cache.manager import CacheManager
    from .config.base import load_config
    from .engine.batch import StepEntry
    from .engine.model import CausalLM
    from .engine.runner import ModelRunner
    from .weights.loader import load_weights

    if not torch.cuda.is_available():
        print("trace_run needs a CUDA device; none is visible", file=sys.stderr)
        return 2
    ps = args.page_size
    if ps <= 0 or (64 % ps != 0 and ps % 64 != 0):
        print("--page-size must divide 64 or be a multiple of 64", file=sys.stderr)
        return 2
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    os.makedirs(args.out, exist_ok=True)
    config = load_config(args.model)
    model = CausalLM(config.model_spec())
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    load_weights(model, args.model, dtype, device)
    unit = max(ps, 64)
    pool_tokens = (args.max_tokens + unit - 1) // unit * unit
    num_pages = pool_tokens // ps
    max_len = min(model.spec.max_positions, pool_tokens)
    n_paged = sum(1 for g in model.cache_groups if g.kind == "paged")
    manager = CacheManager(model.cache_groups, [num_pages] * n_paged, ps, args.max_requests, max_len)
    max_step_tokens = max(pool_tokens, 64)
    runner = ModelRunner(model, manager, device, max_step_tokens, cuda_graphs=not args.no_graphs)

    slots: Dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            toks = [int(t) for t in e["tokens"]]
            if rid not in slots:
                s = manager.open()
                if s is None:
                    print(f"step {step}: more than {args.max_requests} live requests", file=sys.stderr)
                    return 3
                slots[rid] = s
            if not runner.reserve(slots[rid], len(toks)):
                print(f"step {step}: request {rid} needs more cache than --max-tokens {args.max_tokens} leaves",
                      file=sys.stderr)
                return 3
            entries.append(StepEntry(slots[rid], toks, tuple(int(w) for w in e.get("want", []))))
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                arr = logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(args.out, f"{step}.f32"))
            runner.check_status()
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                manager.close(slots.pop(rid))
        print(f"done {step}", flush=True)
    print(f"trace_run: {runner.steps_run} steps, {runner.graph_replays} graph replays, "
          f"pages handed out {manager.pages_handed_out}, pages reused {manager.pages_reused}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
