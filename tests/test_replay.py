"""Trace replay through bin/trace_run against the plain implementation (GPU).

The same requests are replayed whole, with the last 32 tokens one by one, in
portions of changing size (down to two tokens), and mixed (up to four live
requests, portions beside single tokens, a pool so small that pages are used
again), in float32 and in bfloat16.
"""
import re

import numpy as np
import pytest
import torch

from helpers import TINY, TOL, TraceRun, make_model_folder, random_tokens, rel_err
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [100, 37, 64, 81, 5, 128], "B": [150, 33, 97, 64, 1, 120], "C": [200, 45, 130, 17, 96, 160]}


@pytest.fixture(scope="module", params=["A", "B", "C"])
def case(request):
    name = request.param
    folder = make_model_folder(name, sharpen=TINY[name]["sharpen"])
    cfg, w = P.read_model_folder(folder)
    seqs = [random_tokens(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(LENGTHS[name])]
    refs = [P.forward_logits(cfg, w, s).numpy() for s in seqs]
    return name, folder, seqs, refs


def _check(got, ref, dtype, what):
    err = rel_err(got, ref)
    assert err <= TOL[dtype], f"{what}: relative error {err:.3e} above {TOL[dtype]:.0e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_last32_and_portions(case, dtype):
    name, folder, seqs, refs = case
    ps = TINY[name]["page_size"]
    tr = TraceRun(folder, dtype, max_tokens=256, page_size=ps)
    try:
        # 1. each request alone and whole, logits everywhere
        for i in (0, 1, 4):
            n = len(seqs[i])
            got = tr.step([{"id": f"w{i}", "tokens": seqs[i], "want": list(range(n))}], end=[f"w{i}"])
            _check(got, refs[i], dtype, f"{name} whole request {i}")
        # 2. most in one step, the last 32 tokens one by one
        for i in (0, 2):
            n = len(seqs[i])
            head = n - 32
            got = tr.step([{"id": f"d{i}", "tokens": seqs[i][:head], "want": [head - 1]}])
            _check(got, refs[i][head - 1:head], dtype, f"{name} request {i} head")
            for t in range(head, n):
                got = tr.step([{"id": f"d{i}", "tokens": [seqs[i][t]], "want": [0]}],
                              end=[f"d{i}"] if t == n - 1 else [])
                _check(got, refs[i][t:t + 1], dtype, f"{name} request {i} token {t} decoded alone")
        # 3. portions of changing size, down to two tokens
        sizes = [7, 2, 13, 2, 5, 31, 2, 3, 17, 2, 64, 2, 9]
        for i in (0, 3, 5):
            n, t, k = len(seqs[i]), 0, 0
            while t < n:
                c = min(sizes[k % len(sizes)], n - t)
                k += 1
                got = tr.step([{"id": f"p{i}", "tokens": seqs[i][t:t + c], "want": list(range(c))}],
                              end=[f"p{i}"] if t + c == n else [])
                _check(got, refs[i][t:t + c], dtype, f"{name} request {i} portion {t}..{t + c}")
                t += c
    finally:
        assert tr.close() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_with_pages_used_again(case, dtype):
    name, folder, seqs, refs = case
    ps = TINY[name]["page_size"]
    # four live requests of at most 64-rounded lengths: the pool is just large enough for them
    order = [0, 1, 2, 3, 4, 5, 1, 3]
    need = sorted(((len(seqs[i]) + 63) // 64 * 64 for i in order), reverse=True)[:4]
    # (the pools start as NaN: nothing may depend on what a page held before its owner wrote to it)
    tr = TraceRun(folder, dtype, max_tokens=sum(need), page_size=ps, cache_fill="nan")
    rng = np.random.default_rng(7)
    try:
        waiting = list(enumerate(order))
        live = {}            # rid -> [seq index, next position]
        steps = 0
        while waiting or live:
            while waiting and len(live) < 4:
                k, i = waiting.pop(0)
                live[f"m{k}"] = [i, 0]
            entries, expect, ends = [], [], []
            for rid, (i, t) in list(live.items()):
                n = len(seqs[i])
                if len(live) > 1 and rng.random() < 0.2:
                    continue                                   # left out of this step, goes on later
                if n - t > 24:
                    c = int(rng.integers(2, 19))               # a portion of a prompt
                else:
                    c = 1                                      # a single token, as in decoding
                c = min(c, n - t)
                want = list(range(c)) if rng.random() < 0.8 else [c - 1]
                entries.append({"id": rid, "tokens": seqs[i][t:t + c], "want": want})
                expect.append(refs[i][[t + w for w in want]])
                live[rid][1] = t + c
                if t + c == n:
                    ends.append(rid)
                    del live[rid]
            if not entries:
                continue
            got = tr.step(entries, end=ends)
            _check(got, np.concatenate(expect, axis=0), dtype, f"{name} mixed step {steps}")
            steps += 1
    finally:
        assert tr.close() == 0
    assert tr.pages_reused() > 0, "the pool was meant to be so small that pages are used again"
