"""Randomly drawn tiny configurations (head sizes in steps of 16, any number of heads and groups, widths and
vocabularies that are no power of two, windows, page sizes) through the runner in both dtypes against the plain
implementation: a prompt cut at a random place, then decoded tokens beside a second request (GPU)."""
import random

import numpy as np
import pytest
import torch

from helpers import TOL, rel_err, random_tokens
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(seed)
    nkv = rng.choice([1, 2, 3, 4])
    window = rng.choice([None, None, 24, 70])
    cfg = dict(architectures=["Qwen2ForCausalLM"], hidden_size=rng.choice([8, 16, 24, 40]) * rng.choice([3, 5, 7, 8, 9]),
               num_hidden_layers=rng.choice([1, 2, 3]), num_attention_heads=nkv * rng.choice([1, 2, 3, 4, 5, 7, 8, 9, 12]),
               num_key_value_heads=nkv, head_dim=rng.choice([16, 32, 48, 64, 80, 96, 128, 64, 128]),
               intermediate_size=rng.choice([8, 24, 40]) * rng.choice([3, 5, 8, 11]),
               vocab_size=rng.choice([97, 256, 331, 1000, 1537]), rope_theta=rng.choice([1e4, 1e6]),
               rms_norm_eps=rng.choice([1e-6, 1e-5]), tie_word_embeddings=rng.random() < 0.5,
               max_position_embeddings=512, use_sliding_window=window is not None, torch_dtype="bfloat16")
    if window is not None:
        cfg.update(sliding_window=window, max_window_layers=rng.choice([0, 1]))
    return rng, cfg, rng.choice([4, 8, 16, 32, 64])


@pytest.mark.parametrize("seed", range(500, 516))
def test_a_random_configuration(seed, tmp_path):
    from lite_lang_b200.cache import CacheManager
    from lite_lang_b200.config import config_from_dict, load_config
    from lite_lang_b200.engine.batch import StepEntry
    from lite_lang_b200.engine.model import CausalLM
    from lite_lang_b200.engine.runner import ModelRunner
    from lite_lang_b200.weights import load_weights, write_random_model

    rng, cfgd, page = draw(seed)
    folder, dev = str(tmp_path), torch.device("cuda:0")
    write_random_model(folder, config_from_dict(cfgd), seed, {"matrix": 0.05, "bias": 0.05, "norm": 0.1})
    cfg, w = P.read_model_folder(folder)
    n_prompt, n_dec = rng.choice([5, 37, 90, 150]), 5
    toks = random_tokens(n_prompt + n_dec, cfg["vocab_size"], seed)
    ref = P.forward_logits(cfg, w, toks).numpy()
    cut = rng.randint(1, n_prompt)
    for dtype in ("float32", "bfloat16"):
        m = CausalLM(load_config(folder).model_spec())
        load_weights(m, folder, torch.bfloat16 if dtype == "bfloat16" else torch.float32, dev)
        paged = sum(1 for g in m.cache_groups if g.kind == "paged")
        mgr = CacheManager(m.cache_groups, [2 * (256 // page + 4)] * paged, page, 4, 256)
        runner = ModelRunner(m, mgr, dev, 256, cuda_graphs=True)
        a, b = mgr.open(), mgr.open()
        assert runner.reserve(a, n_prompt)
        lg = [runner.step([StepEntry(a, toks[:cut], tuple(range(cut)))]).float().cpu().numpy()]
        if cut < n_prompt:
            lg.append(runner.step([StepEntry(a, toks[cut:n_prompt], tuple(range(n_prompt - cut)))]).float().cpu().numpy())
        assert rel_err(np.concatenate(lg), ref[:n_prompt]) <= TOL[dtype], (dtype, cfgd)
        for i in range(n_dec):
            assert runner.reserve(a, 1) and runner.reserve(b, 1)
            out = runner.step([StepEntry(a, [toks[n_prompt + i]], (0,)), StepEntry(b, [toks[i]], (0,))]).float().cpu().numpy()
            assert rel_err(out, np.stack([ref[n_prompt + i], ref[i]])) <= TOL[dtype], (dtype, i, cfgd)
        runner.check_status()
