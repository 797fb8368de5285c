"""The engine at the layer sizes of the benchmark model (Qwen2-1.5B: hidden 1536, 12/2 heads of 128,
intermediate 8960, vocabulary 151936, tied), with two layers, against the plain implementation (GPU).

The tiny configurations never reach the kernels that serving uses at real sizes (the TMA weight-streaming
product, the tensor-core attention with clusters, the wide lm_head); this test does, in bfloat16 and in
float32, whole and decoded token by token.
"""
import numpy as np
import pytest
import torch

from helpers import TOL, rel_err, random_tokens
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

CFG = dict(architectures=["Qwen2ForCausalLM"], hidden_size=1536, num_hidden_layers=2, num_attention_heads=12,
           num_key_value_heads=2, intermediate_size=8960, vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
           tie_word_embeddings=True, max_position_embeddings=4096, use_sliding_window=False, torch_dtype="bfloat16")


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    from lite_lang_b200.config import config_from_dict
    from lite_lang_b200.weights import write_random_model
    folder = str(tmp_path_factory.mktemp("real_shape"))
    write_random_model(folder, config_from_dict(CFG), seed=21, scales={"matrix": 0.03, "bias": 0.05, "norm": 0.05})
    cfg, w = P.read_model_folder(folder)
    toks = random_tokens(56, cfg["vocab_size"], 77)
    ref = P.forward_logits(cfg, w, toks).numpy()
    return folder, toks, ref


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_whole_then_token_by_token(model, dtype):
    from lite_lang_b200.cache import CacheManager
    from lite_lang_b200.config import load_config
    from lite_lang_b200.engine.batch import StepEntry
    from lite_lang_b200.engine.model import CausalLM
    from lite_lang_b200.engine.runner import ModelRunner
    from lite_lang_b200.weights import load_weights

    folder, toks, ref = model
    dev = torch.device("cuda:0")
    m = CausalLM(load_config(folder).model_spec())
    load_weights(m, folder, torch.bfloat16 if dtype == "bfloat16" else torch.float32, dev)
    mgr = CacheManager(m.cache_groups, [32], 16, 8, 256)
    runner = ModelRunner(m, mgr, dev, 128, cuda_graphs=True)
    a, b = mgr.open(), mgr.open()
    # request a: 40 tokens at once, then 16 one by one (captured steps), request b beside it from step 2 on
    assert runner.reserve(a, 40)
    lg = runner.step([StepEntry(a, toks[:40], tuple(range(40)))]).float().cpu().numpy()
    assert rel_err(lg, ref[:40]) <= TOL[dtype]
    for i in range(40, 56):
        entries = [StepEntry(a, [toks[i]], (0,))]
        want = [ref[i:i + 1]]
        assert runner.reserve(a, 1)
        if i >= 42:
            j = i - 42
            assert runner.reserve(b, 1)
            entries.append(StepEntry(b, [toks[j]], (0,)))
            want.append(ref[j:j + 1])
        lg = runner.step(entries).float().cpu().numpy()
        err = rel_err(lg, np.concatenate(want))
        assert err <= TOL[dtype], (i, err)
    runner.check_status()
    assert runner.graph_replays == 16


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_long_portion_through_the_two_sm_kernels(model, dtype):
    """A prompt portion of 1,300 tokens in one step: at these sizes the q|k|v projection (with bias, rotation
    and cache write in its epilogue) and the gated feed-forward go to the two-SM tcgen05 kernel in bfloat16.
    Logits at the edges of its 256-token tiles, then three decoded tokens, which read the cache it wrote."""
    from lite_lang_b200 import ops
    from lite_lang_b200.cache import CacheManager
    from lite_lang_b200.config import load_config
    from lite_lang_b200.engine.batch import StepEntry
    from lite_lang_b200.engine.model import CausalLM
    from lite_lang_b200.engine.runner import ModelRunner
    from lite_lang_b200.weights import load_weights

    folder, _, _ = model
    dev = torch.device("cuda:0")
    n_prompt, n_dec = 1300, 3
    cfg, w = P.read_model_folder(folder, device="cuda:0")          # the plain formulas, float32, on the device
    toks = random_tokens(n_prompt + n_dec, cfg["vocab_size"], 78)
    places = [0, 127, 128, 255, 256, 1023, 1024, 1279, 1280, n_prompt - 1] + list(range(n_prompt, n_prompt + n_dec))
    ops.configure_matmul_precision()
    tok = torch.as_tensor(toks, dtype=torch.long, device=dev)
    h = P.embedding(w["model.embed_tokens.weight"], tok)
    for layer in range(cfg["num_hidden_layers"]):
        h = P.decoder_layer(h, torch.arange(len(toks), device=dev), w, layer, cfg)
    y = P.rms_norm(h[places], w["model.norm.weight"], float(cfg["rms_norm_eps"]))
    ref = P.linear(y, w["model.embed_tokens.weight"]).cpu().numpy()

    m = CausalLM(load_config(folder).model_spec())
    load_weights(m, folder, torch.bfloat16 if dtype == "bfloat16" else torch.float32, dev)
    if dtype == "bfloat16":
        x = torch.empty(n_prompt, cfg["hidden_size"], dtype=torch.bfloat16, device=dev)
        mixer = m.blocks[0].mixer
        assert ops.pair_qkv_supported(x, mixer.w_qkv, mixer.head_dim, mixer.head_dim) and ops.pair_qkv_preferred(x, mixer.w_qkv)
    mgr = CacheManager(m.cache_groups, [96], 16, 2, 1536)
    runner = ModelRunner(m, mgr, dev, 1536, cuda_graphs=False)
    a = mgr.open()
    assert runner.reserve(a, n_prompt)
    want = tuple(p for p in places if p < n_prompt)
    lg = runner.step([StepEntry(a, toks[:n_prompt], want)]).float().cpu().numpy()
    assert rel_err(lg, ref[:len(want)]) <= TOL[dtype]
    for i in range(n_dec):
        assert runner.reserve(a, 1)
        lg = runner.step([StepEntry(a, [toks[n_prompt + i]], (0,))]).float().cpu().numpy()
        err = rel_err(lg, ref[len(want) + i:len(want) + i + 1])
        assert err <= TOL[dtype], (i, err)
    runner.check_status()


OTHER_SIZES = {
    "0.5b": dict(hidden_size=896, num_attention_heads=14, num_key_value_heads=2, intermediate_size=4864,
                 vocab_size=151936, tie_word_embeddings=True),          # head 64, a width that is no multiple of 256
    "7b": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944,
               vocab_size=152064, tie_word_embeddings=False),           # 7 query heads a kv head, its own lm_head
}


@pytest.mark.parametrize("size", sorted(OTHER_SIZES))
def test_other_model_sizes_in_bfloat16(size, tmp_path):
    """Two layers at the layer sizes of other Qwen2 models: a prompt in two portions (450 + 250 tokens), then six
    decoded tokens in captured steps, against the plain formulas (float32, on the device)."""
    from lite_lang_b200 import ops
    from lite_lang_b200.cache import CacheManager
    from lite_lang_b200.config import config_from_dict, load_config
    from lite_lang_b200.engine.batch import StepEntry
    from lite_lang_b200.engine.model import CausalLM
    from lite_lang_b200.engine.runner import ModelRunner
    from lite_lang_b200.weights import load_weights, write_random_model

    dev = torch.device("cuda:0")
    folder = str(tmp_path)
    write_random_model(folder, config_from_dict(dict(CFG, **OTHER_SIZES[size])), seed=3,
                       scales={"matrix": 0.03, "bias": 0.05, "norm": 0.05})
    cfg, w = P.read_model_folder(folder, device="cuda:0")
    n_prompt, cut, n_dec = 700, 450, 6
    toks = random_tokens(n_prompt + n_dec, cfg["vocab_size"], 5)
    places = [0, 255, 256, cut - 1, cut, n_prompt - 1] + list(range(n_prompt, n_prompt + n_dec))
    ops.configure_matmul_precision()
    h = P.embedding(w["model.embed_tokens.weight"], torch.as_tensor(toks, dtype=torch.long, device=dev))
    for layer in range(cfg["num_hidden_layers"]):
        h = P.decoder_layer(h, torch.arange(len(toks), device=dev), w, layer, cfg)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    ref = P.linear(P.rms_norm(h[places], w["model.norm.weight"], float(cfg["rms_norm_eps"])), head).cpu().numpy()
    del w, h

    m = CausalLM(load_config(folder).model_spec())
    load_weights(m, folder, torch.bfloat16, dev)
    mgr = CacheManager(m.cache_groups, [64], 16, 2, 1024)
    runner = ModelRunner(m, mgr, dev, 1024, cuda_graphs=True)
    a = mgr.open()
    assert runner.reserve(a, n_prompt)
    first = tuple(p for p in places if p < cut)
    second = tuple(p - cut for p in places if cut <= p < n_prompt)
    lg1 = runner.step([StepEntry(a, toks[:cut], first)]).float().cpu().numpy()
    lg2 = runner.step([StepEntry(a, toks[cut:n_prompt], second)]).float().cpu().numpy()
    assert rel_err(np.concatenate([lg1, lg2]), ref[:len(first) + len(second)]) <= TOL["bfloat16"]
    for i in range(n_dec):
        assert runner.reserve(a, 1)
        lg = runner.step([StepEntry(a, [toks[n_prompt + i]], (0,))]).float().cpu().numpy()
        k = len(first) + len(second) + i
        assert rel_err(lg, ref[k:k + 1]) <= TOL["bfloat16"], i
    runner.check_status()
    assert runner.graph_replays == n_dec


def test_decode_steps_split_the_norm_after_the_attention_between_two_products(model, monkeypatch):
    """In bfloat16 steps of up to 64 tokens the norm after the attention has no kernel of its own: the o
    projection leaves its input ready (``ops.gemm_stream_into_norm``) and the gated product applies the rows'
    factors.  The steps' logits equal the plain ones, and those of the same steps with the norm as a kernel of its
    own (``ops.NORM_SPLIT`` off) up to bfloat16 rounding; a larger step keeps the norm's kernel."""
    from lite_lang_b200 import ops
    from lite_lang_b200.cache import CacheManager
    from lite_lang_b200.config import load_config
    from lite_lang_b200.engine.batch import StepEntry
    from lite_lang_b200.engine.model import CausalLM
    from lite_lang_b200.engine.runner import ModelRunner
    from lite_lang_b200.weights import load_weights

    folder, toks, ref = model
    dev = torch.device("cuda:0")
    m = CausalLM(load_config(folder).model_spec())
    load_weights(m, folder, torch.bfloat16, dev)
    calls = {"into_norm": 0, "scaled": 0}
    real_into, real_scaled = ops.gemm_stream_into_norm, ops.gemm_stream_gated_scaled

    def into(*a, **k):
        calls["into_norm"] += 1
        return real_into(*a, **k)

    def scaled(*a, **k):
        calls["scaled"] += 1
        return real_scaled(*a, **k)

    monkeypatch.setattr(ops, "gemm_stream_into_norm", into)
    monkeypatch.setattr(ops, "gemm_stream_gated_scaled", scaled)
    layers = m.spec.num_layers if hasattr(m.spec, "num_layers") else len(m.blocks)

    def run(split):
        monkeypatch.setattr(ops, "NORM_SPLIT", split)
        mgr = CacheManager(m.cache_groups, [32], 16, 8, 256)
        runner = ModelRunner(m, mgr, dev, 128, cuda_graphs=False)
        a, b, c = mgr.open(), mgr.open(), mgr.open()
        assert runner.reserve(a, 40) and runner.reserve(b, 9) and runner.reserve(c, 30)
        first_calls = dict(calls)
        runner.step([StepEntry(a, toks[:40], ()), StepEntry(b, toks[:9], ()), StepEntry(c, toks[:30], ())])
        mgr.close(c)
        before = dict(calls)
        if split:      # (a step of more than 64 tokens, here 79 of three prompts, keeps the norm's own kernel)
            assert first_calls == before, (first_calls, before)
        out = []
        for i in range(3):     # two requests, a token each: the split path
            assert runner.reserve(a, 1) and runner.reserve(b, 1)
            out.append(runner.step([StepEntry(a, [toks[40 + i]], (0,)), StepEntry(b, [toks[9 + i]], (0,))]).float().cpu().numpy())
        during = {k: calls[k] - before[k] for k in calls}
        runner.check_status()
        return np.concatenate(out), during

    got_split, n_split = run(True)
    got_whole, n_whole = run(False)
    assert n_split == {"into_norm": 3 * layers, "scaled": 3 * layers}, n_split
    assert n_whole == {"into_norm": 0, "scaled": 0}
    want = np.concatenate([np.stack([ref[40 + i], ref[9 + i]]) for i in range(3)])
    assert rel_err(got_split, want) <= TOL["bfloat16"]
    assert rel_err(got_whole, want) <= TOL["bfloat16"]
    assert rel_err(got_split, got_whole) <= TOL["bfloat16"]


def test_one_and_two_requests_with_a_very_long_context(tmp_path):
    """A request of 17,000 tokens, decoded alone and beside a short one, in captured steps: with so few requests
    and so many keys the decode attention gives a (request, kv head) eight clusters, each with a range of the keys,
    that meet through scratch memory (a class of context length of its own has its own graph and plan); the prompt goes in portions of 2,048 tokens, the
    later ones behind many thousands of cached tokens.  (That no part of the keys goes missing is the kernel test's
    matter: one far key among 9,000 that outweighs all others.)"""
    from lite_lang_b200 import ops
    from lite_lang_b200.cache import CacheManager
    from lite_lang_b200.config import config_from_dict, load_config
    from lite_lang_b200.engine.batch import StepEntry
    from lite_lang_b200.engine.model import CausalLM
    from lite_lang_b200.engine.runner import ModelRunner
    from lite_lang_b200.weights import load_weights, write_random_model

    cfg_d = dict(CFG, vocab_size=4099, max_position_embeddings=20000, tie_word_embeddings=False)
    folder = str(tmp_path / "long")
    write_random_model(folder, config_from_dict(cfg_d), seed=23, scales={"matrix": 0.03, "bias": 0.05, "norm": 0.05})
    dev = torch.device("cuda:0")
    ops.configure_matmul_precision()
    cfg, w = P.read_model_folder(folder, device=dev)
    T, head = 17040, 17000
    toks = random_tokens(T, cfg["vocab_size"], 91)
    short = random_tokens(40, cfg["vocab_size"], 92)
    ref = P.forward_logits(cfg, w, toks)[head - 1:].cpu().numpy()
    ref_short = P.forward_logits(cfg, w, short).cpu().numpy()
    del w
    torch.cuda.empty_cache()

    m = CausalLM(load_config(folder).model_spec())
    load_weights(m, folder, torch.bfloat16, dev)
    mgr = CacheManager(m.cache_groups, [(T + 64) // 16 + 8], 16, 4, 20000)
    runner = ModelRunner(m, mgr, dev, 2048, cuda_graphs=True)
    a = mgr.open()
    assert runner.reserve(a, head)
    for c0 in range(0, head, 2048):
        c1 = min(head, c0 + 2048)
        lg = runner.step([StepEntry(a, toks[c0:c1], (c1 - c0 - 1,) if c1 == head else ())])
    assert rel_err(lg.float().cpu().numpy(), ref[:1]) <= TOL["bfloat16"]
    plans = []
    real_plan = type(m.blocks[0].mixer)._plan_mma

    def spy(self, step, entries, max_kv_len, sms):
        plan = real_plan(self, step, entries, max_kv_len, sms)
        plans.append((entries, max_kv_len, plan[1], plan[4]))
        return plan

    type(m.blocks[0].mixer)._plan_mma = spy
    try:
        b = None
        for i in range(head, T):
            entries = [StepEntry(a, [toks[i]], (0,))]
            want = [ref[i - head + 1:i - head + 2]]
            assert runner.reserve(a, 1)
            if i >= head + 10:                      # a short request beside it: prompt whole, then token by token
                j = i - head - 10
                if b is None:
                    b = mgr.open()
                    assert runner.reserve(b, 8)
                    runner.step([StepEntry(b, short[:8], ())])
                assert runner.reserve(b, 1)
                entries.append(StepEntry(b, [short[8 + j]], (0,)))
                want.append(ref_short[8 + j:9 + j])
            got = runner.step(entries).float().cpu().numpy()
            err = rel_err(got, np.concatenate(want))
            assert err <= TOL["bfloat16"], (i, err)
    finally:
        type(m.blocks[0].mixer)._plan_mma = real_plan
    runner.check_status()
    assert runner.graph_replays == T - head
    assert {(e, nouter) for e, _, _, nouter in plans} == {(1, 8), (2, 8)}, plans     # 8 clusters of 4 CTAs a kv head
    assert all(n == 4 and kv == 20000 for _, kv, n, _ in plans), plans
