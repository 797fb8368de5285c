"""The plain implementation against the reference's own model, run on the GPU (GPU).

tests/plain/qwen2_plain.py is written from the reference's formulas; its single functions are compared with
the reference's pure-torch helpers in tests/test_plain.py.  How the functions are put together (pre-norm
order and in-place residual sums, ``qwen2/layer/transformer_layer.py:46-77``; bias before rotation, rotation
of q and k only, ``:94-116``; row selection, final norm and lm_head, ``layer/post_layer.py:14-45``; the tied
head, ``layer_weights/post_layer_weights.py:10-15``) is pinned here: the unmodified reference, installed under
``baseline/_ref``, computes a prefill of three prompts and eight decode steps in a process of its own
(tests/reference/run_reference_model.py), and every row of logits it produced is compared with the plain
implementation's logits for the same tokens.

The reference computes in float16 (weights, activations, rotation tables, residual sums), so the comparison
has float16's tolerance.  It hard-codes theta = 1e6 and eps = 1e-6 in the layers, which the model folder's
config.json repeats, and eps = 1e-5 in the last norm (``post_layer.py:12``), which changes a normalised row
by a few parts in a million at these sizes and is left as it is.  The layer sizes are those of the benchmark
(hidden 1536, 12/2 heads of 128, intermediate 8960), the shapes at which the reference's kernels are known to
run on this GPU; the vocabulary is small.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import ROOT, random_tokens, rel_err
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

REF_ROOT = os.path.join(ROOT, "baseline", "_ref")
TOL_FLOAT16 = 2e-2       # of the row's largest logit; set before the first run
CFG = dict(architectures=["Qwen2ForCausalLM"], hidden_size=1536, num_hidden_layers=2, num_attention_heads=12,
           num_key_value_heads=2, intermediate_size=8960, vocab_size=4099, rope_theta=1000000.0, rms_norm_eps=1e-6,
           max_position_embeddings=4096, use_sliding_window=False, torch_dtype="float16")


@pytest.mark.parametrize("tied", [True, False])
def test_plain_implementation_equals_the_reference_model(tied, tmp_path):
    if not os.path.isdir(os.path.join(REF_ROOT, "litelang")):
        pytest.skip("the reference is not installed under baseline/_ref")
    try:
        import triton  # noqa: F401
    except ImportError:
        pytest.skip("the reference's kernels need triton")
    from lite_lang_b200.config import config_from_dict
    from lite_lang_b200.weights import write_random_model

    folder = str(tmp_path / "model")
    cfg_d = dict(CFG, tie_word_embeddings=tied)
    write_random_model(folder, config_from_dict(cfg_d), seed=71, scales={"matrix": 0.03, "bias": 0.05, "norm": 0.05},
                       dtype="float16")
    prompts = [random_tokens(n, cfg_d["vocab_size"], 700 + i) for i, n in enumerate([37, 64, 150])]
    n_decode = 8
    prompts_json, out_npz = str(tmp_path / "prompts.json"), str(tmp_path / "reference.npz")
    with open(prompts_json, "w") as fh:
        json.dump(prompts, fh)
    script = os.path.join(ROOT, "tests", "reference", "run_reference_model.py")
    res = subprocess.run([sys.executable, script, REF_ROOT, folder, prompts_json, str(n_decode), out_npz],
                         capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-3000:]
    got = np.load(out_npz)
    ref_logits, ref_tokens = got["logits"], got["tokens"]          # [steps, requests, vocab], [steps, requests]
    assert ref_logits.shape == (1 + n_decode, len(prompts), cfg_d["vocab_size"])

    cfg, w = P.read_model_folder(folder, device="cuda:0")
    torch.backends.cuda.matmul.allow_tf32 = False
    worst = 0.0
    for r, prompt in enumerate(prompts):
        seq = list(prompt) + [int(t) for t in ref_tokens[:-1, r]]   # the reference fed its own tokens
        plain = P.forward_logits(cfg, w, seq).cpu().numpy()
        for step in range(1 + n_decode):
            row = plain[len(prompt) - 1 + step]
            err = rel_err(ref_logits[step, r][None], row[None])
            worst = max(worst, err)
            assert err <= TOL_FLOAT16, f"request {r} step {step}: relative error {err:.3e}"
            # the token the reference chose is the plain argmax, unless the plain top two are within rounding
            top2 = np.sort(row)[-2:]
            if top2[1] - top2[0] > 2 * TOL_FLOAT16 * np.abs(row).max():
                assert int(ref_tokens[step, r]) == int(row.argmax()), (r, step)
    print(f"largest relative error against the reference's float16 logits: {worst:.3e}")
