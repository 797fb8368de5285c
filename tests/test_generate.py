"""Generation through the Python entry point and the command line (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import ROOT, TINY, TOL, make_model_folder, random_tokens, rel_err
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu


def engine(folder, dtype, name, **kw):
    from lite_lang_b200 import Engine, EngineConfig
    cfg = dict(dtype=dtype, page_size=TINY[name]["page_size"], num_pages=64, max_batch_size=4,
               max_input_length=100, max_output_length=16, max_tokens_per_step=64)
    cfg.update(kw)
    return Engine(folder, EngineConfig(**cfg))


def _assert_greedy_or_near_tie(cfg, w, prompt, out, margin):
    """Every token of ``out`` is the plain argmax, up to the first place where the plain top two
    logits are closer than ``margin`` of the largest logit (after which the sequences may part)."""
    seq = list(prompt)
    for tok in out:
        logits = P.forward_logits(cfg, w, seq)[-1]
        top2 = torch.topk(logits, 2).values
        if float(top2[0] - top2[1]) <= margin * float(logits.abs().max()):
            return
        assert tok == int(torch.argmax(logits)), (len(prompt), len(seq))
        seq.append(tok)


@pytest.mark.parametrize("name,lengths", [("A", [5, 11, 17]), ("B", [1, 7, 23, 40]), ("C", [60, 3, 33])])
def test_greedy_generation_equals_the_plain_continuation(name, lengths):
    """float32: token for token, unless the plain top two logits are closer than the engine's error."""
    folder = make_model_folder(name, scales={"matrix": 0.08})
    cfg, w = P.read_model_folder(folder)
    prompts = [random_tokens(n, cfg["vocab_size"], 50 + i) for i, n in enumerate(lengths)]
    from lite_lang_b200 import SamplingParams
    eng = engine(folder, "float32", name, max_tokens_per_step=8 if name == "B" else 64)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        assert len(out) == 8
        seq = list(prompt)
        for tok in out:
            logits = P.forward_logits(cfg, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) > 1e-4 * float(logits.abs().max()):
                assert tok == int(torch.argmax(logits)), (name, len(prompt), len(seq))
            seq.append(tok)
    st = eng.stats()
    assert st["finished"] == len(prompts) and eng.manager.num_free_pages() == eng.manager.total_pages()


def _assert_within_rounding(cfg, w, prompt, out, tol):
    """Every token of ``out`` is, given the tokens before it, the plain argmax up to the engine's rounding:
    logits that differ from the plain ones by at most ``tol`` of the largest can only move the argmax to a
    token whose plain logit lies within 2 * tol of the plain maximum.  The check follows the engine's own
    tokens, so it holds at every place, whatever was chosen before."""
    seq = list(prompt)
    for k, tok in enumerate(out):
        logits = P.forward_logits(cfg, w, seq)[-1]
        slack = 2 * tol * float(logits.abs().max())
        assert float(logits[tok]) >= float(logits.max()) - slack, (len(prompt), k, tok, int(torch.argmax(logits)))
        seq.append(tok)


def test_bfloat16_generation_runs_captured_steps_and_equals_the_plain_continuation_up_to_rounding():
    from lite_lang_b200 import SamplingParams
    folder = make_model_folder("C", scales={"matrix": 0.08})
    cfg, w = P.read_model_folder(folder)
    prompts = [random_tokens(n, cfg["vocab_size"], 70 + i) for i, n in enumerate([40, 9, 21])]
    sp = SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True)
    a = engine(folder, "bfloat16", "C").generate(prompts, sp)
    eng = engine(folder, "bfloat16", "C", cuda_graphs=False, max_tokens_per_step=16)
    b = eng.generate(prompts, sp)
    e2 = engine(folder, "bfloat16", "C")
    a2 = e2.generate(prompts, sp)
    assert a == a2                                     # the same run twice: the same tokens
    assert e2.stats()["graph_replays"] > 0
    # captured steps or not, prompts whole or in portions of 16: every token against the plain logits
    for prompt, x, y in zip(prompts, a, b):
        assert len(x) == len(y) == 12
        _assert_within_rounding(cfg, w, prompt, x, TOL["bfloat16"])
        _assert_within_rounding(cfg, w, prompt, y, TOL["bfloat16"])


def test_temperature_sampling_is_seeded_and_independent_of_batching():
    from lite_lang_b200 import SamplingParams
    folder = make_model_folder("B", scales={"matrix": 0.08})
    cfg, w = P.read_model_folder(folder)
    prompts = [random_tokens(n, cfg["vocab_size"], 80 + i) for i, n in enumerate([1, 7, 23, 40])]
    sp = SamplingParams(temperature=0.7, max_new_tokens=8, ignore_eos=True, seed=1234)
    together = engine(folder, "float32", "B", max_tokens_per_step=8).generate(prompts, sp)
    again = engine(folder, "float32", "B", max_tokens_per_step=8).generate(prompts, sp)
    assert together == again
    other = engine(folder, "float32", "B").generate(prompts, SamplingParams(temperature=0.7, max_new_tokens=8,
                                                                            ignore_eos=True, seed=99))
    assert other != together
    # every drawn token lies in the CDF interval of its uniform number under the plain distribution
    from lite_lang_b200.sampling import uniform_for
    for rid, (prompt, out) in enumerate(zip(prompts, together)):
        seq = list(prompt)
        for k, tok in enumerate(out):
            p = P.temperature_probs(P.forward_logits(cfg, w, seq)[-1], 0.7)
            cdf = torch.cumsum(p, 0)
            u = uniform_for(1234, rid, k)
            lo = float(cdf[tok - 1]) if tok > 0 else 0.0
            assert lo - 1e-3 <= u <= float(cdf[tok]) + 1e-3, (rid, k)
            seq.append(tok)
    # greedy requests beside sampled ones; do_sample False forces greedy as in the reference's request format
    mixed = engine(folder, "float32", "B").generate(
        prompts[:2], [SamplingParams(temperature=0.7, do_sample=False, max_new_tokens=4, ignore_eos=True),
                      SamplingParams(temperature=0.0, max_new_tokens=4, ignore_eos=True)])
    for prompt, out in zip(prompts[:2], mixed):
        assert len(out) == 4
        _assert_greedy_or_near_tie(cfg, w, prompt, out, 1e-4)


def test_preemption_under_a_small_pool_does_not_change_the_tokens():
    from lite_lang_b200 import SamplingParams
    folder = make_model_folder("A", scales={"matrix": 0.08})
    cfg, w = P.read_model_folder(folder)
    prompts = [random_tokens(n, cfg["vocab_size"], 90 + i) for i, n in enumerate([20, 20, 20])]
    sp = SamplingParams(temperature=0.0, max_new_tokens=20, ignore_eos=True)
    roomy = engine(folder, "float32", "A", num_pages=64, max_output_length=20).generate(prompts, sp)
    eng = engine(folder, "float32", "A", num_pages=22, max_output_length=20, busy_scale=1.0)
    eng.scheduler._fits = lambda cand: True            # admit everything: the pool must run out
    tight = eng.generate(prompts, sp)
    assert eng.stats()["preemptions"] > 0
    assert eng.manager.num_free_pages() == 22
    for a, b, prompt in zip(roomy, tight, prompts):
        assert len(a) == len(b) == 20
        seq = list(prompt)
        for ta, tb in zip(a, b):
            if ta != tb:           # only a near tie of the plain logits may differ
                logits = P.forward_logits(cfg, w, seq)[-1]
                top2 = torch.topk(logits, 2).values
                assert float(top2[0] - top2[1]) <= 1e-4 * float(logits.abs().max())
                break
            seq.append(ta)


def test_eos_ends_a_request():
    from lite_lang_b200 import SamplingParams
    folder = make_model_folder("B", scales={"matrix": 0.08})
    cfg, w = P.read_model_folder(folder)
    prompt = random_tokens(9, cfg["vocab_size"], 5)
    free = P.greedy_generate(cfg, w, prompt, 6)
    eos = free[2]
    cfg2 = dict(cfg, eos_token_id=eos)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(cfg2, fh)
    out = engine(folder, "float32", "B").generate([prompt], SamplingParams(max_new_tokens=6))[0]
    assert out == free[:free.index(eos) + 1]
    out = engine(folder, "float32", "B").generate([prompt], SamplingParams(max_new_tokens=6, ignore_eos=True))[0]
    assert out == free


def test_steps_launched_ahead_give_the_same_tokens_and_end_requests_on_time():
    """Decode steps are launched before the host has seen the tokens of the step before (their token ids
    are fed on the device).  Requests that end by length, by an eos id in the middle, and a request that
    arrives while others decode must come out as without the pipelining."""
    from lite_lang_b200 import SamplingParams
    folder = make_model_folder("C", scales={"matrix": 0.08})
    cfg, w = P.read_model_folder(folder)
    prompts = [random_tokens(n, cfg["vocab_size"], 90 + i) for i, n in enumerate([12, 30, 5, 19])]
    plain = [P.greedy_generate(cfg, w, p, 14) for p in prompts]
    # request 1 ends in the middle by an eos id that the other requests never produce within their limits
    elsewhere = set(plain[0][:14]) | set(plain[2][:3]) | set(plain[3][:9])
    eos = next(t for t in plain[1][2:12] if t not in elsewhere)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(dict(cfg, eos_token_id=eos), fh)
    params = [SamplingParams(temperature=0.0, max_new_tokens=n) for n in (14, 14, 3, 9)]
    late = random_tokens(8, cfg["vocab_size"], 99)

    def run(pipeline):
        eng = engine(folder, "float32", "C", max_output_length=16)
        eng._pipeline = pipeline
        reqs = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]
        steps = 0
        while eng.scheduler.has_work():
            eng.step()
            steps += 1
            if steps == 4:                              # arrives while the others decode
                reqs.append(eng.add_request(late, SamplingParams(temperature=0.7, seed=5, max_new_tokens=6,
                                                                 ignore_eos=True)))
        assert eng.manager.num_free_pages() == eng.manager.total_pages()
        eng.manager.check_invariants()
        return [list(r.output) for r in reqs], [r.finish_reason for r in reqs], eng.stats()

    out_a, why_a, st_a = run(True)
    out_b, why_b, st_b = run(False)
    assert out_a == out_b and why_a == why_b
    assert why_a[:4] == ["length", "eos", "length", "length"]
    assert out_a[1] == plain[1][:plain[1].index(eos) + 1]
    assert out_a[2] == plain[2][:3]
    assert st_a["graph_replays"] > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_random_serving_runs_equal_the_plain_continuation(seed, dtype):
    """Random prompts, limits, an eos id taken from the plain continuations, requests arriving while others run,
    tight page pools (requests leave and are recomputed), steps launched ahead or not: every request's tokens
    equal the plain greedy continuation, and every page comes back.  In bfloat16 every token is checked against
    the plain logits of the tokens before it, within twice the tolerance of the logits."""
    import random
    from lite_lang_b200 import Engine, EngineConfig, SamplingParams
    rng = random.Random(1000 + seed)
    name = "ABC"[seed % 3]
    folder = make_model_folder(name, scales={"matrix": 0.08})
    cfg, w = P.read_model_folder(folder)
    n_req = rng.randint(3, 8)
    prompts = [random_tokens(rng.randint(1, 60), cfg["vocab_size"], seed * 100 + i) for i in range(n_req)]
    max_new = [rng.randint(1, 14) for _ in range(n_req)]
    plain = [P.greedy_generate(cfg, w, p, m) for p, m in zip(prompts, max_new)]
    eos = None
    if rng.random() < 0.6:
        cand = plain[rng.randrange(n_req)]
        eos = cand[rng.randrange(len(cand))]
        with open(os.path.join(folder, "config.json"), "w") as fh:
            json.dump(dict(cfg, eos_token_id=eos), fh)
    ps = TINY[name]["page_size"]
    need = max((len(p) + m + ps) // ps + 1 for p, m in zip(prompts, max_new))
    pages = rng.randint(need, need + 3) if rng.random() < 0.7 else rng.randint(need, need * 3)
    eng = Engine(folder, EngineConfig(dtype=dtype, page_size=ps, num_pages=pages, max_batch_size=rng.choice([2, 4]),
                                      max_input_length=100, max_output_length=16,
                                      max_tokens_per_step=rng.choice([8, 16, 64])))
    eng._pipeline = rng.random() < 0.8
    order = list(range(n_req))
    rng.shuffle(order)
    first = order[:rng.randint(1, n_req)]
    later = order[len(first):]
    reqs = {i: eng.add_request(prompts[i], SamplingParams(temperature=0.0, max_new_tokens=max_new[i])) for i in first}
    steps = 0
    while eng.scheduler.has_work() or later:
        if later and (steps % 3 == 2 or not eng.scheduler.has_work()):
            i = later.pop()
            reqs[i] = eng.add_request(prompts[i], SamplingParams(temperature=0.0, max_new_tokens=max_new[i]))
        eng.step()
        steps += 1
        assert steps < 5000
    eng.manager.check_invariants()
    assert eng.manager.num_free_pages() == eng.manager.total_pages()
    for i in range(n_req):
        if dtype == "bfloat16":
            got = list(reqs[i].output)
            if reqs[i].finish_reason == "cache_full":
                continue
            _assert_within_rounding(cfg, w, prompts[i], got, TOL["bfloat16"])
            if eos is not None and eos in got:
                assert got.index(eos) == len(got) - 1 and reqs[i].finish_reason == "eos"
            else:
                assert len(got) == max_new[i] and reqs[i].finish_reason == "length"
            continue
        want = plain[i]
        if eos is not None and eos in want:
            want = want[:want.index(eos) + 1]
        got = list(reqs[i].output)
        if reqs[i].finish_reason == "cache_full" or got == want:
            continue
        k = next((j for j, (a, b) in enumerate(zip(got, want)) if a != b), min(len(got), len(want)))
        logits = P.forward_logits(cfg, w, prompts[i] + want[:k])[-1]
        top2 = torch.topk(logits, 2).values          # only a near-tie in the plain logits excuses a difference
        assert float(top2[0] - top2[1]) <= 1e-4 * float(logits.abs().max()), (i, got, want)


def test_command_line():
    folder = make_model_folder("A", scales={"matrix": 0.08})
    cfg, w = P.read_model_folder(folder)
    prompt = random_tokens(6, cfg["vocab_size"], 3)
    ids = os.path.join(folder, "prompt.json")
    with open(ids, "w") as fh:
        json.dump([prompt], fh)
    cmd = [sys.executable, "-m", "lite_lang_b200.cli", "--model_path", folder, "--prompt_ids", ids, "--dtype", "fp32",
           "--max_output_length", "5", "--page_size", "4", "--num_pages", "32", "--max_batch_size", "2",
           "--temperature", "0", "--ignore_eos"]
    res = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    out = json.loads(res.stdout.strip().splitlines()[-1])
    assert out["outputs"][0] == P.greedy_generate(cfg, w, prompt, 5)
    bad = subprocess.run(cmd + ["--tp", "2"], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert bad.returncode != 0 and "tp" in (bad.stderr + bad.stdout)


def _write_word_tokenizer(folder, vocab_size):
    """A word-level tokenizer made on the spot (no download): word ``w<i>`` is token i, token 0 is unknown."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    vocab = {"[UNK]": 0}
    for i in range(1, vocab_size):
        vocab[f"w{i}"] = i
    tok = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.save(os.path.join(folder, "tokenizer.json"))
    with open(os.path.join(folder, "tokenizer_config.json"), "w") as fh:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "[UNK]"}, fh)


def test_text_prompts_go_through_the_folders_tokenizer():
    """Text in, text out (the reference tokenizes every request: litelang/scheduler/tokenizer/tokenizer.py:4-31);
    here the tokenizer is loaded only when a prompt is text."""
    try:
        import tokenizers  # noqa: F401
        from transformers import AutoTokenizer  # noqa: F401
    except ImportError:
        pytest.skip("text prompts need the transformers and tokenizers packages")
    from lite_lang_b200 import SamplingParams
    folder = make_model_folder("A", scales={"matrix": 0.08})
    cfg, w = P.read_model_folder(folder)
    _write_word_tokenizer(folder, cfg["vocab_size"])
    ids = [t or 1 for t in random_tokens(7, cfg["vocab_size"], 21)]          # (token 0 is the unknown word)
    text = " ".join(f"w{t}" for t in ids)
    eng = engine(folder, "float32", "A")
    assert eng._tokenizer is None                       # not loaded before a text prompt asks for it
    sp = SamplingParams(temperature=0.0, max_new_tokens=5, ignore_eos=True)
    out_ids = eng.generate([ids], sp)[0]
    assert eng._tokenizer is None
    out_text = eng.generate_text([text], sp)[0]
    assert eng._tokenizer is not None
    want = P.greedy_generate(cfg, w, ids, 5)
    _assert_greedy_or_near_tie(cfg, w, ids, out_ids, 1e-4)
    assert out_text == eng.tokenizer().decode(out_ids)
    if out_ids == want:
        assert out_text.split() == [("[UNK]" if t == 0 else f"w{t}") for t in want]
    # the command line with --prompt TEXT
    cmd = [sys.executable, "-m", "lite_lang_b200.cli", "--model_path", folder, "--prompt", text, "--dtype", "fp32",
           "--max_output_length", "5", "--page_size", "4", "--num_pages", "32", "--max_batch_size", "2",
           "--temperature", "0", "--ignore_eos"]
    res = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    out = json.loads(res.stdout.strip().splitlines()[-1])
    assert out["outputs"][0] == out_ids and out["texts"][0] == out_text
