"""The plain implementation against the reference's own per-op helpers (stored outputs) and by its
own properties (no GPU)."""
import os

import numpy as np
import torch

from helpers import TINY, make_model_folder, random_tokens
from plain import qwen2_plain as P

A = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "op_anchors.npz"))


def t(name):
    return torch.from_numpy(A[name])


def close(a, b, tol=2e-6):
    return float((a.double() - b.double()).abs().max()) <= tol * max(1.0, float(b.abs().max()))


def test_rope_equals_the_references_helpers():
    assert close(P.apply_rope(t("rope_x"), t("rope_cos"), t("rope_sin")), t("rope_y"))
    cos, sin = P.rope_tables(16, 10000.0, torch.arange(9))
    assert close(P.apply_rope(t("rope_x"), cos, sin), t("rope_theta_y"), 1e-5)


def test_silu_and_rmsnorm_equal_the_references_helpers():
    gu = t("silu_in")
    assert close(P.silu_and_mul(gu[:, :12], gu[:, 12:]), t("silu_out"))
    assert close(P.rms_norm(t("rms_x"), t("rms_w"), 1e-5), t("rms_y"))


def test_attention_equals_the_references_helpers():
    q, k, v = t("att_q"), t("att_k"), t("att_v")
    lens = [int(x) for x in A["att_lens"]]
    start = 0
    for n in lens:                     # prefill: every request alone and whole
        o = P.attention(q[start:start + n], k[start:start + n], v[start:start + n])
        assert close(o, t("att_o")[start:start + n], 1e-5)
        start += n
    # decode: the reference's query attends to all of its request's keys; equal to our last row
    # when the query is placed last
    start = 0
    for i, n in enumerate(lens):
        qq = torch.cat([q[start:start + n - 1], t("dec_q")[i:i + 1]], dim=0)
        o = P.attention(qq, k[start:start + n], v[start:start + n])
        assert close(o[-1], t("dec_o")[i], 1e-5)
        start += n


def test_logits_are_causal_and_deterministic():
    folder = make_model_folder("B")
    cfg, w = P.read_model_folder(folder)
    toks = random_tokens(12, cfg["vocab_size"], 3)
    full = P.forward_logits(cfg, w, toks)
    part = P.forward_logits(cfg, w, toks[:7])
    assert close(part, full[:7], 1e-5)
    assert full.shape == (12, cfg["vocab_size"])
    other = list(toks)
    other[9] = (other[9] + 1) % cfg["vocab_size"]
    assert close(P.forward_logits(cfg, w, other)[:9], full[:9], 1e-6)
    assert not close(P.forward_logits(cfg, w, other)[9:], full[9:], 1e-6)


def test_window_limits_what_a_position_sees():
    g = torch.Generator().manual_seed(1)
    q, k, v = torch.randn(10, 2, 8, generator=g), torch.randn(10, 1, 8, generator=g), torch.randn(10, 1, 8, generator=g)
    full = P.attention(q, k, v)
    win = P.attention(q, k, v, window=4)
    assert close(win[:4], full[:4])                       # the first 4 positions see everything anyway
    v2 = v.clone()
    v2[0] += 100.0                                        # position 0 is outside the window of positions >= 4
    assert close(P.attention(q, k, v2, window=4)[4:], win[4:])
    assert not close(P.attention(q, k, v2)[4:], full[4:])
    assert P.layer_window({"use_sliding_window": True, "sliding_window": 4, "max_window_layers": 2}, 1) is None
    assert P.layer_window({"use_sliding_window": True, "sliding_window": 4, "max_window_layers": 2}, 2) == 4
    assert P.layer_window({"use_sliding_window": False, "sliding_window": 4}, 2) is None


def test_greedy_generation_extends_the_sequence():
    folder = make_model_folder("B")
    cfg, w = P.read_model_folder(folder)
    prompt = random_tokens(6, cfg["vocab_size"], 9)
    out = P.greedy_generate(cfg, w, prompt, 3)
    assert len(out) == 3
    assert out[0] == int(torch.argmax(P.forward_logits(cfg, w, prompt)[-1]))
    assert out[1] == int(torch.argmax(P.forward_logits(cfg, w, prompt + out[:1])[-1]))
