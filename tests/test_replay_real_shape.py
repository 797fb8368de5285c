"""Trace replay at the layer sizes of the benchmark models, through bin/trace_run (GPU).

Two layers at the sizes of Qwen2-1.5B (hidden 1536, 12/2 heads of 128, intermediate 8960, vocabulary
151936, tied head; float32 and bfloat16) and of Qwen2-7B (hidden 3584, 28/4 heads, 7 query heads a kv head,
an lm_head of its own; bfloat16), under the four cuttings of tests/test_replay.py: whole; most in one step
and the last 32 tokens one by one; portions of changing size down to two tokens; and mixed, up to four live
requests in a pool that is handed out completely, so that later requests get pages that others gave back.

The tiny configurations never reach the kernels that serving uses; these steps do.  The mixed trace holds a
step with more than a thousand prompt tokens beside two decoded ones (the two-SM tcgen05 q|k|v projection
with rotation and cache write over all tokens of the step, the decode attention on the first entries and
the tcgen05 prefill attention on the rest, library products that add into the residual stream), steps of 32
and of about 100 tokens (the tcgen05 weight-streaming products), portions of two tokens beside decoded
tokens, and the cache pools start as NaN, so that nothing can lean on what a page held before.
"""
import numpy as np
import pytest
import torch

from helpers import TOL, TraceRun, random_tokens, rel_err
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, rope_theta=1000000.0, rms_norm_eps=1e-6,
            max_position_embeddings=4096, use_sliding_window=False, torch_dtype="bfloat16")
SIZES = {
    "1.5b": dict(hidden_size=1536, num_attention_heads=12, num_key_value_heads=2, intermediate_size=8960,
                 vocab_size=151936, tie_word_embeddings=True),
    "7b": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944,
               vocab_size=152064, tie_word_embeddings=False),
}
# lengths of the requests A..F and the large portion of the mixed trace (the q|k|v projection goes to the
# two-SM kernel when its tiles of 256 x 256 fill a good part of the SM pairs)
LENGTHS = {"1.5b": dict(A=1400, B=700, C=330, D=90, E=200, F=64, big=1100),
           "7b": dict(A=760, B=300, C=200, D=90, E=100, F=64, big=600)}
DTYPES = {"1.5b": ["bfloat16", "float32"], "7b": ["bfloat16"]}
DEV = "cuda:0"


class Case:
    """A model folder, its requests, and the plain implementation's last hidden states of each request."""

    def __init__(self, size, folder):
        from lite_lang_b200 import ops
        from lite_lang_b200.config import config_from_dict
        from lite_lang_b200.weights import write_random_model
        self.size, self.folder = size, folder
        write_random_model(folder, config_from_dict(dict(BASE, **SIZES[size])), seed=31,
                           scales={"matrix": 0.03, "bias": 0.05, "norm": 0.05})
        ops.configure_matmul_precision()                    # the plain formulas in true float32 on the device
        self.cfg, self.w = P.read_model_folder(folder, device=DEV)
        self.lengths = LENGTHS[size]
        self.seqs = {k: random_tokens(n, self.cfg["vocab_size"], 300 + i)
                     for i, (k, n) in enumerate(self.lengths.items()) if k != "big"}
        self.hidden = {}
        for k, toks in self.seqs.items():
            tok = torch.as_tensor(toks, dtype=torch.long, device=DEV)
            h = P.embedding(self.w["model.embed_tokens.weight"], tok)
            pos = torch.arange(len(toks), device=DEV)
            for layer in range(self.cfg["num_hidden_layers"]):
                h = P.decoder_layer(h, pos, self.w, layer, self.cfg)
            self.hidden[k] = h
        self.head = (self.w["model.embed_tokens.weight"] if self.cfg.get("tie_word_embeddings")
                     else self.w["lm_head.weight"])

    def logits(self, key, rows):
        y = P.rms_norm(self.hidden[key][list(rows)], self.w["model.norm.weight"], float(self.cfg["rms_norm_eps"]))
        return P.linear(y, self.head).cpu().numpy()


@pytest.fixture(scope="module", params=["1.5b", "7b"])
def case(request, tmp_path_factory):
    c = Case(request.param, str(tmp_path_factory.mktemp(f"replay_{request.param.replace('.', '_')}")))
    yield c
    c.w = c.hidden = c.head = None
    torch.cuda.empty_cache()


def _check(got, ref, dtype, what):
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = rel_err(got, ref)
    assert err <= TOL[dtype], f"{what}: relative error {err:.3e} above {TOL[dtype]:.0e}"


def _dtypes(case):
    return DTYPES[case.size]


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_whole_last32_and_portions_at_real_sizes(case, dtype):
    if dtype not in _dtypes(case):
        pytest.skip("the 7B sizes are replayed in bfloat16 only")
    seqs = case.seqs
    tr = TraceRun(case.folder, dtype, max_tokens=2048, page_size=16)
    try:
        # 1. whole, logits at the edges of the kernels' tiles and at the end
        for key in ("A", "D", "F"):
            n = len(seqs[key])
            want = sorted({0, 1, 15, 16, 63, 64, 127, 128, 255, 256, 511, 512, 1023, 1024, n - 2, n - 1} & set(range(n)))
            got = tr.step([{"id": f"w{key}", "tokens": seqs[key], "want": want}], end=[f"w{key}"])
            _check(got, case.logits(key, want), dtype, f"{case.size} whole request {key}")
        # 2. most in one step, the last 32 tokens one by one
        for key in ("B", "D"):
            n = len(seqs[key])
            head = n - 32
            got = tr.step([{"id": f"d{key}", "tokens": seqs[key][:head], "want": [head - 1]}])
            _check(got, case.logits(key, [head - 1]), dtype, f"{case.size} request {key} head")
            for t in range(head, n):
                got = tr.step([{"id": f"d{key}", "tokens": [seqs[key][t]], "want": [0]}],
                              end=[f"d{key}"] if t == n - 1 else [])
                _check(got, case.logits(key, [t]), dtype, f"{case.size} request {key} token {t} decoded alone")
        # 3. portions of changing size, down to two tokens
        sizes = [7, 2, 130, 2, 13, 70, 2, 5, 33, 2, 64, 3, 17]
        for key in ("C", "E"):
            n, t, k = len(seqs[key]), 0, 0
            while t < n:
                c = min(sizes[k % len(sizes)], n - t)
                k += 1
                want = sorted({0, c // 2, c - 1})
                got = tr.step([{"id": f"p{key}", "tokens": seqs[key][t:t + c], "want": want}],
                              end=[f"p{key}"] if t + c == n else [])
                _check(got, case.logits(key, [t + x for x in want]), dtype, f"{case.size} request {key} portion {t}..{t + c}")
                t += c
    finally:
        assert tr.close() == 0


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_mixed_at_real_sizes_with_pages_used_again(case, dtype):
    if dtype not in _dtypes(case):
        pytest.skip("the 7B sizes are replayed in bfloat16 only")
    from lite_lang_b200 import ops
    seqs, L = case.seqs, case.lengths
    big = L["big"]
    if dtype == "bfloat16":
        # the step with the large portion is one whose q|k|v projection the two-SM kernel takes
        nh, nkv = SIZES[case.size]["num_attention_heads"], SIZES[case.size]["num_key_value_heads"]
        hidden = SIZES[case.size]["hidden_size"]
        x = torch.empty(big + 2, hidden, dtype=torch.bfloat16, device=DEV)
        w_qkv = torch.empty((nh + 2 * nkv) * 128, hidden, dtype=torch.bfloat16, device=DEV)
        assert ops.pair_qkv_supported(x, w_qkv, 128, 128) and ops.pair_qkv_preferred(x, w_qkv)
        del x, w_qkv
    # the pool holds exactly the four first requests, each rounded up to 64 tokens
    first = ["A", "B", "C", "D"]
    pool = sum((L[k] + 63) // 64 * 64 for k in first)
    tr = TraceRun(case.folder, dtype, max_tokens=pool, page_size=16, cache_fill="nan")
    rng = np.random.default_rng(11)
    done_at = {}                       # request id -> position reached
    live = {}                          # request id -> sequence key
    later = [("F2", "F"), ("E2", "E"), ("C2", "C"), ("D2", "D")]
    steps = 0

    def run(plan):
        """plan: request id -> number of its next tokens in this step."""
        nonlocal steps
        entries, expect, ends = [], [], []
        for rid, c in plan.items():
            key = live[rid]
            t, n = done_at[rid], len(seqs[key])
            c = min(c, n - t)
            want = [0] if c == 1 else sorted({0, c // 2, c - 1})
            entries.append({"id": rid, "tokens": seqs[key][t:t + c], "want": want})
            expect.append(case.logits(key, [t + x for x in want]))
            done_at[rid] = t + c
            if t + c == n:
                ends.append(rid)
        got = tr.step(entries, end=ends)
        _check(got, np.concatenate(expect, axis=0), dtype,
               f"{case.size} mixed step {steps} ({', '.join(f'{r}:{c}' for r, c in plan.items())})")
        for rid in ends:
            del live[rid]
        steps += 1

    try:
        for rid in first:
            live[rid], done_at[rid] = rid, 0
        run({"B": L["B"] - 40, "C": L["C"] - 30})
        run({"B": 1, "C": 1, "A": big})              # two decoded tokens beside a large portion
        run({"B": 1, "C": 1, "D": 30})               # 32 tokens in all
        run({"B": 1, "C": 1, "D": 58, "A": 40})      # 100 tokens in all
        run({"A": 2, "B": 1, "C": 1, "D": 2})        # portions of two tokens beside decoded tokens
        run({"A": 1, "B": 2})
        while live or later:
            # (what the live requests hold, each rounded up to 64 tokens, stays within the pool)
            held = sum((L[key] + 63) // 64 * 64 for key in live.values())
            while later and len(live) < 4 and held + (L[later[0][1]] + 63) // 64 * 64 <= pool:
                rid, key = later.pop(0)
                live[rid], done_at[rid] = key, 0
                held += (L[key] + 63) // 64 * 64
            plan = {}
            for rid, key in live.items():
                left = len(seqs[key]) - done_at[rid]
                if len(live) > 1 and rng.random() < 0.2:
                    continue                          # left out of this step, goes on later
                if left > 24:
                    plan[rid] = int(rng.integers(2, 150))
                else:
                    plan[rid] = 1 if rng.random() < 0.8 else 2
            if plan:
                run(plan)
    finally:
        assert tr.close() == 0
    assert tr.pages_reused() > 0, "the pool was meant to be so small that pages are used again"
