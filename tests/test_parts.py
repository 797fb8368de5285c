"""Each part alone, the run order as data, and a toy mixer with state of its own (GPU)."""
from dataclasses import dataclass
from typing import Any, Dict, Mapping

import numpy as np
import pytest
import torch

from helpers import rel_err
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def dev():
    return torch.device("cuda:0")


def tol(dtype):
    return 1e-5 if dtype == torch.float32 else 3e-2


def rt(x, dtype):
    """Round through the storage type: the values the part really gets."""
    return x.to(dtype).float()


def build(family, kind, params, prefix=""):
    from lite_lang_b200.config import PartSpec
    from lite_lang_b200.parts import build_part
    return build_part(family, PartSpec(kind, params, prefix))


def load(part, tensors: Dict[str, torch.Tensor], dtype):
    part.load(lambda rel: tensors.get(rel), dtype, dev())


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    g = torch.Generator().manual_seed(0)
    norm = build("norm", "rms_norm", {"hidden_size": 72, "eps": 2e-5})
    w = 1 + 0.1 * torch.randn(72, generator=g)
    load(norm, {"weight": w.to(torch.bfloat16)}, dtype)
    assert norm.weight.dtype == torch.float32
    x = rt(torch.randn(9, 72, generator=g), dtype)
    y = norm.forward(x.to(dtype).to(dev()))
    assert rel_err(y.float().cpu().numpy(), P.rms_norm(x, rt(w, torch.bfloat16), 2e-5).numpy()) <= tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_position_part(dtype):
    g = torch.Generator().manual_seed(1)
    nh, nkv, hd = 5, 1, 24
    rope = build("position", "rope_half_split", {"rotary_dim": hd, "theta": 777.0, "max_positions": 90})
    rope.prepare(dev())
    assert rope.table.dtype == torch.float32 and tuple(rope.table.shape) == (90, hd)
    qkv = rt(torch.randn(6, (nh + 2 * nkv) * hd, generator=g), dtype)
    pos = torch.tensor([0, 1, 17, 89, 3, 3], dtype=torch.int32)
    buf = qkv.to(dtype).to(dev())
    rope.apply(buf, pos.to(dev()), nh, nkv, hd, 6)
    cos, sin = P.rope_tables(hd, 777.0, pos)
    ref = qkv.clone()
    ref[:, :(nh + nkv) * hd] = P.apply_rope(qkv[:, :(nh + nkv) * hd].view(6, nh + nkv, hd), cos, sin).reshape(6, -1)
    assert rel_err(buf.float().cpu().numpy(), ref.numpy()) <= tol(dtype)       # v is untouched, q and k rotated


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    g = torch.Generator().manual_seed(2)
    ffn = build("feed_forward", "gated_mlp", {"hidden_size": 40, "intermediate_size": 104, "activation": "silu"})
    t = {"gate_proj.weight": 0.2 * torch.randn(104, 40, generator=g), "up_proj.weight": 0.2 * torch.randn(104, 40, generator=g),
         "down_proj.weight": 0.2 * torch.randn(40, 104, generator=g)}
    load(ffn, t, dtype)
    x = rt(torch.randn(7, 40, generator=g), dtype)
    y = ffn.forward(x.to(dtype).to(dev()), None)
    ref = P.gated_mlp(x, rt(t["gate_proj.weight"], dtype), rt(t["up_proj.weight"], dtype), rt(t["down_proj.weight"], dtype))
    assert rel_err(y.float().cpu().numpy(), ref.numpy()) <= tol(dtype)
    with pytest.raises(ValueError, match="activation"):
        build("feed_forward", "gated_mlp", {"hidden_size": 8, "intermediate_size": 8, "activation": "relu"})


# ---------------------------------------------------------------------------
# a model from a hand-made spec: the run order names a layer twice and shares a cache plane
# ---------------------------------------------------------------------------

def _attention_spec(prefix, hidden, nh, nkv, hd, window=None):
    from lite_lang_b200.config import PartSpec
    return PartSpec("gqa_attention", {
        "hidden_size": hidden, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qkv_bias": True,
        "scale": hd ** -0.5, "window": window,
        "position": PartSpec("rope_half_split", {"rotary_dim": hd, "theta": 10000.0, "max_positions": 256}),
    }, prefix + "self_attn.")


def _spec(order, mixers=None, hidden=48, layers=2, ffns=None):
    from lite_lang_b200.config import LayerSpec, ModelSpec, PartSpec
    norm = {"hidden_size": hidden, "eps": 1e-6}
    ls = []
    for i in range(layers):
        p = f"model.layers.{i}."
        mixer = mixers[i](p) if mixers else _attention_spec(p, hidden, 4, 2, 16)
        ffn = ffns[i](p) if ffns else PartSpec("gated_mlp", {"hidden_size": hidden, "intermediate_size": 80}, p + "mlp.")
        ls.append(LayerSpec("pre_norm", {"mixer": mixer, "feed_forward": ffn,
                                         "mixer_norm": PartSpec("rms_norm", norm, p + "input_layernorm."),
                                         "feed_forward_norm": PartSpec("rms_norm", norm, p + "post_attention_layernorm.")}))
    return ModelSpec("Test", hidden, 97, 256,
                     PartSpec("token_embedding", {"vocab_size": 97, "hidden_size": hidden}, "model.embed_tokens."),
                     tuple(ls), tuple(order), PartSpec("rms_norm", norm, "model.norm."),
                     PartSpec("lm_head", {"vocab_size": 97, "hidden_size": hidden, "tied_to": None}, "lm_head."))


def _build_runner(spec, dtype, seed=3, page_size=4, num_pages=40, graphs=False):
    from lite_lang_b200.cache import CacheManager
    from lite_lang_b200.engine.model import CausalLM
    from lite_lang_b200.engine.runner import ModelRunner
    from lite_lang_b200.weights import draw_tensor
    model = CausalLM(spec)
    scales = {"matrix": 0.15, "bias": 0.1, "norm": 0.1}
    tensors = {n: draw_tensor(n, d, seed, scales, torch.bfloat16) for n, d in model.declared_tensors().items()}
    model.load(lambda n: tensors.get(n), dtype, dev())
    n_paged = sum(1 for g in model.cache_groups if g.kind == "paged")
    mgr = CacheManager(model.cache_groups, [num_pages] * n_paged, page_size, 4, 128)
    return model, mgr, ModelRunner(model, mgr, dev(), 128, cuda_graphs=graphs), {k: v.float() for k, v in tensors.items()}


def _plain_layer(h, w, layer, window=None, kv_from=None):
    """One pre-norm layer with the plain functions; returns h and this layer's rotated k and v inputs."""
    cfg = {"num_attention_heads": 4, "num_key_value_heads": 2, "hidden_size": 48, "head_dim": 16,
           "rope_theta": 10000.0, "rms_norm_eps": 1e-6}
    return P.decoder_layer(h, torch.arange(h.shape[0]), w, layer, cfg)


def _run_whole_and_cut(runner, mgr, toks):
    from lite_lang_b200.engine.batch import StepEntry
    s = mgr.open()
    assert runner.reserve(s, len(toks))
    whole = runner.step([StepEntry(s, toks, tuple(range(len(toks))))]).float().cpu().numpy().copy()
    mgr.close(s)
    s = mgr.open()
    rows, t = [], 0
    for c in [5, 2, 1, 9, 1, 1, 3, 100]:
        c = min(c, len(toks) - t)
        if c == 0:
            break
        assert runner.reserve(s, c)
        rows.append(runner.step([StepEntry(s, toks[t:t + c], tuple(range(c)))]).float().cpu().numpy().copy())
        t += c
    mgr.close(s)
    runner.check_status()
    return whole, np.concatenate(rows)


@pytest.mark.parametrize("dtype", DTYPES)
def test_run_order_may_name_a_layer_twice(dtype):
    from lite_lang_b200.config import RunStep
    spec = _spec([RunStep(0), RunStep(1), RunStep(0)])
    model, mgr, runner, w = _build_runner(spec, dtype)
    assert [(p.layer, p.plane, p.writable) for p in model.plan] == [(0, 0, True), (1, 1, True), (0, 2, True)]
    assert model.cache_groups[0].planes == 3
    toks = [int(t) for t in np.random.default_rng(0).integers(0, 97, 30)]
    h = P.embedding(w["model.embed_tokens.weight"], torch.tensor(toks))
    for layer in (0, 1, 0):
        h = _plain_layer(h, w, layer)
    ref = P.linear(P.rms_norm(h, w["model.norm.weight"], 1e-6), w["lm_head.weight"]).numpy()
    whole, cut = _run_whole_and_cut(runner, mgr, toks)
    assert rel_err(whole, ref) <= tol(dtype) and rel_err(cut, ref) <= tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_run_step_may_read_another_ones_cache(dtype):
    """Layer 1 attends with its own queries over the keys and values that layer 0 wrote."""
    from lite_lang_b200.config import RunStep
    spec = _spec([RunStep(0), RunStep(1, cache=0)])
    model, mgr, runner, w = _build_runner(spec, dtype)
    assert [(p.plane, p.writable) for p in model.plan] == [(0, True), (0, False)]
    assert model.cache_groups[0].planes == 1
    toks = [int(t) for t in np.random.default_rng(1).integers(0, 97, 26)]
    T = len(toks)
    cfg = {"num_attention_heads": 4, "num_key_value_heads": 2, "hidden_size": 48, "head_dim": 16,
           "rope_theta": 10000.0, "rms_norm_eps": 1e-6}
    pos = torch.arange(T)
    cos, sin = P.rope_tables(16, 10000.0, pos)
    h = P.embedding(w["model.embed_tokens.weight"], torch.tensor(toks))
    # layer 0, keeping its k and v
    p0 = "model.layers.0."
    x = P.rms_norm(h, w[p0 + "input_layernorm.weight"], 1e-6)
    k0 = P.apply_rope(P.linear(x, w[p0 + "self_attn.k_proj.weight"], w[p0 + "self_attn.k_proj.bias"]).view(T, 2, 16), cos, sin)
    v0 = P.linear(x, w[p0 + "self_attn.v_proj.weight"], w[p0 + "self_attn.v_proj.bias"]).view(T, 2, 16)
    if dtype == torch.bfloat16:
        k0, v0 = rt(k0, dtype), rt(v0, dtype)
    h = P.decoder_layer(h, pos, w, 0, cfg)
    # layer 1 with layer 0's keys and values
    p1 = "model.layers.1."
    x = P.rms_norm(h, w[p1 + "input_layernorm.weight"], 1e-6)
    q1 = P.apply_rope(P.linear(x, w[p1 + "self_attn.q_proj.weight"], w[p1 + "self_attn.q_proj.bias"]).view(T, 4, 16), cos, sin)
    o = P.attention(q1, k0, v0)
    h = h + P.linear(o.reshape(T, 64), w[p1 + "self_attn.o_proj.weight"])
    x = P.rms_norm(h, w[p1 + "post_attention_layernorm.weight"], 1e-6)
    h = h + P.gated_mlp(x, w[p1 + "mlp.gate_proj.weight"], w[p1 + "mlp.up_proj.weight"], w[p1 + "mlp.down_proj.weight"])
    ref = P.linear(P.rms_norm(h, w["model.norm.weight"], 1e-6), w["lm_head.weight"]).numpy()
    whole, cut = _run_whole_and_cut(runner, mgr, toks)
    assert rel_err(whole, ref) <= tol(dtype) and rel_err(cut, ref) <= tol(dtype)


def test_layers_of_one_model_may_differ():
    """Different windows give different cache groups; a bad order is refused."""
    from lite_lang_b200.config import RunStep
    from lite_lang_b200.engine.model import CausalLM
    mixers = [lambda p: _attention_spec(p, 48, 4, 2, 16), lambda p: _attention_spec(p, 48, 2, 1, 32, window=8)]
    model = CausalLM(_spec([RunStep(0), RunStep(1)], mixers))
    assert len(model.cache_groups) == 2 and model.cache_groups[1].window == 8 and model.cache_groups[1].head_dim == 32
    with pytest.raises(ValueError, match="needs differ"):
        CausalLM(_spec([RunStep(0), RunStep(1, cache=0)], mixers))
    with pytest.raises(ValueError, match="not earlier"):
        CausalLM(_spec([RunStep(0, cache=1), RunStep(1)]))
    with pytest.raises(ValueError, match="does not exist"):
        CausalLM(_spec([RunStep(0), RunStep(5)]))


# ---------------------------------------------------------------------------
# a toy mixer with state of its own, defined here, registered, built and stepped
# ---------------------------------------------------------------------------

def test_toy_mixer_with_state_needs_no_change_to_the_framework():
    from lite_lang_b200.config import ModelConfig, PartSpec, RunStep, config_from_dict, register_architecture
    from lite_lang_b200.engine.batch import StepEntry
    from lite_lang_b200.parts import Mixer, StateNeed, TensorDecl, register_part

    class DecayMixer(Mixer):
        """y_t = s_t W, s_t = decay * s_{t-1} + x_t: a running sum kept in the request's state record."""

        def __init__(self, spec):
            super().__init__(spec)
            self.hidden = int(spec.params["hidden_size"])
            self.decay = float(spec.params["decay"])

        def tensors(self):
            return {"mix.weight": TensorDecl((self.hidden, self.hidden))}

        def load(self, fetch, dtype, device):
            self.w = fetch("mix.weight").to(dtype).to(device)

        def cache_need(self):
            return StateNeed((self.hidden,), "float32")

        def forward(self, x, step, cache):
            if step.num_single == step.num_entries:
                # single tokens only: from the step's device arrays alone, so that the step may be captured
                # and replayed (token i belongs to entry i; a slot of -1 marks a padding entry)
                slot = step.req_slot.long()
                live = (slot >= 0).unsqueeze(1)
                idx = slot.clamp(min=0)
                s_old = cache.state[idx]
                s_new = self.decay * s_old + x.float()
                cache.state.index_add_(0, idx, torch.where(live, s_new - s_old, torch.zeros_like(s_new)))
                return torch.where(live, s_new @ self.w.float().t(), torch.zeros_like(s_new)).to(x.dtype)
            out = torch.empty_like(x)
            t = 0
            for e in step.entries:                      # portions of a request arrive in order
                s = cache.state[e.slot]
                for _ in range(len(e.tokens)):
                    s.mul_(self.decay).add_(x[t].float())
                    out[t] = (s @ self.w.float().t()).to(x.dtype)
                    t += 1
            return out

    register_part("mixer", "toy_decay", DecayMixer)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        hidden: int = 48
        architecture = "ToyDecayForCausalLM"

        @classmethod
        def from_dict(cls, d):
            return cls(hidden=int(d["hidden"]))

        def model_spec(self):
            mixers = [lambda p: PartSpec("toy_decay", {"hidden_size": self.hidden, "decay": 0.75}, p + "toy."),
                      lambda p: _attention_spec(p, self.hidden, 4, 2, 16)]
            return _spec([RunStep(0), RunStep(1)], mixers, self.hidden)

    register_architecture("ToyDecayForCausalLM", ToyConfig)
    cfg = config_from_dict({"architectures": ["ToyDecayForCausalLM"], "hidden": 48})
    model, mgr, runner, w = _build_runner(cfg.model_spec(), torch.float32)
    kinds = [g.kind for g in model.cache_groups]
    assert kinds == ["state", "paged"] and model.cache_groups[0].shape == (48,)

    toks = [int(t) for t in np.random.default_rng(2).integers(0, 97, 21)]
    T = len(toks)
    cfgd = {"num_attention_heads": 4, "num_key_value_heads": 2, "hidden_size": 48, "head_dim": 16,
            "rope_theta": 10000.0, "rms_norm_eps": 1e-6}
    h = P.embedding(w["model.embed_tokens.weight"], torch.tensor(toks))
    p0 = "model.layers.0."
    x = P.rms_norm(h, w[p0 + "input_layernorm.weight"], 1e-6)
    s, ys = torch.zeros(48), []
    for t in range(T):
        s = 0.75 * s + x[t]
        ys.append(s @ w[p0 + "toy.mix.weight"].t())
    h = h + torch.stack(ys)
    x = P.rms_norm(h, w[p0 + "post_attention_layernorm.weight"], 1e-6)
    h = h + P.gated_mlp(x, w[p0 + "mlp.gate_proj.weight"], w[p0 + "mlp.up_proj.weight"], w[p0 + "mlp.down_proj.weight"])
    h = P.decoder_layer(h, torch.arange(T), w, 1, cfgd)
    ref = P.linear(P.rms_norm(h, w["model.norm.weight"], 1e-6), w["lm_head.weight"]).numpy()

    whole, cut = _run_whole_and_cut(runner, mgr, toks)
    assert rel_err(whole, ref) <= 1e-4 and rel_err(cut, ref) <= 1e-4
    # a slot that is opened again starts from a zeroed record: the same request twice gives the same logits
    again, _ = _run_whole_and_cut(runner, mgr, toks)
    assert rel_err(again, ref) <= 1e-4
    # two requests side by side keep their records apart
    a, b = mgr.open(), mgr.open()
    assert runner.reserve(a, 10) and runner.reserve(b, T)
    out = runner.step([StepEntry(a, toks[:10], (9,)), StepEntry(b, toks, (T - 1,))]).float().cpu().numpy()
    assert rel_err(out, ref[[9, T - 1]]) <= 1e-4

    # the same model with captured decode steps: a portion each, then single tokens side by side, replayed
    # from CUDA graphs, in which the mixer sees the device arrays only (padding entries included: 3 entries
    # in a bucket of 4 at first, then 2 and 1 as requests end)
    model, mgr, runner, w = _build_runner(cfg.model_spec(), torch.float32, graphs=True)
    slots = [mgr.open() for _ in range(3)]
    starts = [9, 4, 14]
    assert all(runner.reserve(s, n) for s, n in zip(slots, starts))
    runner.step([StepEntry(s, toks[:n], ()) for s, n in zip(slots, starts)])
    at = list(starts)
    while any(n < T for n in at):
        live = [i for i in range(3) if at[i] < T]
        assert all(runner.reserve(slots[i], 1) for i in live)
        out = runner.step([StepEntry(slots[i], [toks[at[i]]], (0,)) for i in live]).float().cpu().numpy()
        assert rel_err(out, ref[[at[i] for i in live]]) <= 1e-4, at
        for i in live:
            at[i] += 1
    runner.check_status()
    assert runner.graph_replays >= T - 4 and sorted({bucket for bucket, _ in runner._graphs}) == [1, 2, 4]


# ---------------------------------------------------------------------------
# a toy feed-forward with routing and a toy position encoding, defined here
# ---------------------------------------------------------------------------

def test_toy_routed_feed_forward_and_another_position_encoding_need_no_change_to_the_framework():
    """Layer 0 keeps the stock parts; layer 1 gets a feed-forward that routes every token to two of four
    small experts and an attention whose position encoding rotates neighbouring pairs (2i, 2i+1) of only the
    first half of each head.  Both parts live in this file; the framework builds, loads and steps them."""
    from lite_lang_b200.config import PartSpec, RunStep
    from lite_lang_b200.parts import FeedForward, PositionEncoding, TensorDecl, register_part

    E, TOPK, INNER, H, HD, ROT = 4, 2, 24, 48, 16, 8

    class ToyRoutedFFN(FeedForward):
        def __init__(self, spec):
            super().__init__(spec)
            self.h, self.e, self.inner, self.k = (int(spec.params[n]) for n in ("hidden_size", "experts", "inner", "top_k"))

        def tensors(self):
            return {"router.weight": TensorDecl((self.e, self.h)),
                    "experts.w_in": TensorDecl((self.e, self.inner, self.h)),       # stacked along the expert axis
                    "experts.w_out": TensorDecl((self.e, self.h, self.inner))}

        def load(self, fetch, dtype, device):
            self.router = fetch("router.weight").float().to(device)                  # router in float32
            self.w_in = fetch("experts.w_in").to(dtype).to(device)
            self.w_out = fetch("experts.w_out").to(dtype).to(device)

        def forward(self, x, step):
            logits = x.float() @ self.router.t()                                     # [T, E] float32
            top, idx = torch.topk(logits, self.k, dim=-1)
            gate = torch.softmax(top, dim=-1)                                        # renormalised over the chosen
            out = torch.zeros_like(x, dtype=torch.float32)
            for e in range(self.e):                                                  # tokens of expert e, gathered
                rows, slot = (idx == e).nonzero(as_tuple=True)
                if rows.numel() == 0:
                    continue
                hcur = torch.relu(x[rows].float() @ self.w_in[e].float().t())
                out.index_add_(0, rows, (hcur @ self.w_out[e].float().t()) * gate[rows, slot].unsqueeze(1))
            return out.to(x.dtype)

    class PairRotary(PositionEncoding):
        """Rotates the pairs (2i, 2i+1) of the first `rot` dimensions of every q and k head."""
        fuses_with_store = False

        def __init__(self, spec):
            super().__init__(spec)
            self.rot, self.theta = int(spec.params["rot"]), float(spec.params["theta"])

        def apply(self, qkv, positions, num_heads, num_kv_heads, head_dim, num_tokens):
            half = self.rot // 2
            inv = self.theta ** (-torch.arange(half, device=qkv.device, dtype=torch.float32) * 2 / self.rot)
            ang = positions[:num_tokens].float().unsqueeze(1) * inv                  # [T, half]
            cos, sin = torch.cos(ang).unsqueeze(1), torch.sin(ang).unsqueeze(1)
            heads = qkv[:num_tokens, :(num_heads + num_kv_heads) * head_dim].view(num_tokens, -1, head_dim)
            part = heads[..., :self.rot].float().reshape(num_tokens, -1, half, 2)
            a, b = part[..., 0], part[..., 1]
            rotated = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).reshape(num_tokens, -1, self.rot)
            heads[..., :self.rot] = rotated.to(qkv.dtype)

    register_part("feed_forward", "toy_routed", ToyRoutedFFN)
    register_part("position", "toy_pair_rotary", PairRotary)

    def toy_attention(p):
        return PartSpec("gqa_attention", {
            "hidden_size": H, "num_heads": 4, "num_kv_heads": 2, "head_dim": HD, "qkv_bias": True,
            "scale": HD ** -0.5, "window": None,
            "position": PartSpec("toy_pair_rotary", {"rot": ROT, "theta": 100.0})}, p + "self_attn.")

    mixers = [lambda p: _attention_spec(p, H, 4, 2, HD), toy_attention]
    ffns = [lambda p: PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": 80}, p + "mlp."),
            lambda p: PartSpec("toy_routed", {"hidden_size": H, "experts": E, "inner": INNER, "top_k": TOPK}, p + "moe.")]
    model, mgr, runner, w = _build_runner(_spec([RunStep(0), RunStep(1)], mixers, H, ffns=ffns), torch.float32)
    assert "model.layers.1.moe.experts.w_in" in model.declared_tensors()

    toks = [int(t) for t in np.random.default_rng(4).integers(0, 97, 23)]
    T = len(toks)
    h = P.embedding(w["model.embed_tokens.weight"], torch.tensor(toks))
    h = _plain_layer(h, w, 0)
    # layer 1 by hand: attention with the pair rotation, then the routed feed-forward
    p1 = "model.layers.1."
    x = P.rms_norm(h, w[p1 + "input_layernorm.weight"], 1e-6)
    pos = torch.arange(T)

    def proj(name, heads):
        y = P.linear(x, w[p1 + f"self_attn.{name}_proj.weight"], w[p1 + f"self_attn.{name}_proj.bias"])
        return y.view(T, heads, HD)

    def pair_rotate(t):
        half = ROT // 2
        inv = 100.0 ** (-torch.arange(half, dtype=torch.float64) * 2 / ROT)
        ang = pos.double().unsqueeze(1) * inv
        cos, sin = torch.cos(ang).unsqueeze(1), torch.sin(ang).unsqueeze(1)
        t = t.double().clone()
        a, b = t[..., 0:ROT:2].clone(), t[..., 1:ROT:2].clone()
        t[..., 0:ROT:2] = a * cos - b * sin
        t[..., 1:ROT:2] = a * sin + b * cos
        return t.float()

    q, k, v = pair_rotate(proj("q", 4)), pair_rotate(proj("k", 2)), proj("v", 2)
    attn = P.attention(q, k, v, None).reshape(T, 4 * HD)
    h = h + P.linear(attn, w[p1 + "self_attn.o_proj.weight"])
    x = P.rms_norm(h, w[p1 + "post_attention_layernorm.weight"], 1e-6)
    logits = x.double() @ w[p1 + "moe.router.weight"].double().t()
    top, idx = torch.topk(logits, TOPK, dim=-1)
    gate = torch.softmax(top, dim=-1)
    y = torch.zeros(T, H, dtype=torch.float64)
    for t in range(T):
        for j in range(TOPK):
            e = int(idx[t, j])
            hid = torch.relu(w[p1 + "moe.experts.w_in"][e].double() @ x[t].double())
            y[t] += gate[t, j] * (w[p1 + "moe.experts.w_out"][e].double() @ hid)
    h = h + y.float()
    ref = P.linear(P.rms_norm(h, w["model.norm.weight"], 1e-6), w["lm_head.weight"]).numpy()

    whole, cut = _run_whole_and_cut(runner, mgr, toks)
    assert rel_err(whole, ref) <= 1e-4 and rel_err(cut, ref) <= 1e-4
    assert len({int(e) for e in idx.flatten()}) >= 3          # the routing really spreads the tokens


# ---------------------------------------------------------------------------
# a toy block with a norm after its mixer, and a toy mixer whose values are half as wide as its keys
# ---------------------------------------------------------------------------

def test_toy_block_with_a_third_norm_and_toy_mixer_with_narrow_values_need_no_change_to_the_framework():
    """Layer 0 is arranged by a block kind of this file that has five parts (a norm after the mixer as well as
    before it); layer 1's mixer, also of this file, keeps keys of 16 and values of 8 numbers a head in pages
    of its own.  The framework builds both from the spec, gives the mixer a cache group with planes of those
    widths, and steps them."""
    from lite_lang_b200.config import LayerSpec, ModelSpec, PartSpec, RunStep
    from lite_lang_b200.parts import Block, Mixer, PagedKVNeed, TensorDecl, register_part, whole_output

    H, NH, NKV, HK, HV = 48, 4, 2, 16, 8

    class SandwichBlock(Block):
        """h += post_norm(mixer(norm(h))); h += feed_forward(norm(h))."""
        roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm",
                 "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

        def forward(self, h, delta, step, caches):
            x = self.mixer_norm.add_forward(h, delta)
            a = whole_output(self.mixer.forward(x, step, caches["mixer"]), h.dtype)
            a = self.mixer_post_norm.forward(a)
            x = self.feed_forward_norm.add_forward(h, a)
            return h, self.feed_forward.forward(x, step)

    class NarrowValueAttention(Mixer):
        """Causal attention without position encoding; keys HK wide, values HV wide, in the paged cache."""

        def tensors(self):
            return {"q.weight": TensorDecl((NH * HK, H)), "k.weight": TensorDecl((NKV * HK, H)),
                    "v.weight": TensorDecl((NKV * HV, H)), "o.weight": TensorDecl((H, NH * HV))}

        def load(self, fetch, dtype, device):
            self.w = {n: fetch(n + ".weight").to(dtype).to(device) for n in "qkvo"}

        def cache_need(self):
            return PagedKVNeed(NKV, HK, None, value_head_dim=HV)

        def forward(self, x, step, cache):
            T, ps = x.shape[0], cache.page_size
            q = (x @ self.w["q"].t()).view(T, NH, HK)
            k = (x @ self.w["k"].t()).view(T, NKV, HK)
            v = (x @ self.w["v"].t()).view(T, NKV, HV)
            where = cache.slot_map.long()
            cache.k[where // ps, :, where % ps] = k          # pages are [page, kv head, place, width]
            cache.v[where // ps, :, where % ps] = v
            out = torch.empty(T, NH * HV, dtype=x.dtype, device=x.device)
            t = 0
            for e, ctx in zip(step.entries, step.entry_ctx):
                n, total = len(e.tokens), ctx + len(e.tokens)
                pages = cache.block_table[e.slot, :(total + ps - 1) // ps].long()
                keys = cache.k[pages].transpose(1, 2).reshape(-1, NKV, HK)[:total].float()
                vals = cache.v[pages].transpose(1, 2).reshape(-1, NKV, HV)[:total].float()
                for a in range(NH):
                    g = a // (NH // NKV)
                    sc = (q[t:t + n, a].float() @ keys[:, g].t()) * HK ** -0.5
                    seen = torch.arange(total, device=x.device)[None, :] <= (ctx + torch.arange(n, device=x.device))[:, None]
                    pr = torch.softmax(sc.masked_fill(~seen, float("-inf")), dim=-1)
                    out[t:t + n, a * HV:(a + 1) * HV] = (pr @ vals[:, g]).to(x.dtype)
                t += n
            return out @ self.w["o"].t()

    register_part("block", "toy_sandwich", SandwichBlock)
    register_part("mixer", "toy_narrow_values", NarrowValueAttention)

    norm = {"hidden_size": H, "eps": 1e-6}
    p0, p1 = "model.layers.0.", "model.layers.1."
    layers = (
        LayerSpec("toy_sandwich", {
            "mixer": _attention_spec(p0, H, 4, 2, 16), "mixer_norm": PartSpec("rms_norm", norm, p0 + "input_layernorm."),
            "mixer_post_norm": PartSpec("rms_norm", norm, p0 + "post_mixer_layernorm."),
            "feed_forward_norm": PartSpec("rms_norm", norm, p0 + "post_attention_layernorm."),
            "feed_forward": PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": 80}, p0 + "mlp.")}),
        LayerSpec("pre_norm", {
            "mixer": PartSpec("toy_narrow_values", {}, p1 + "narrow."),
            "mixer_norm": PartSpec("rms_norm", norm, p1 + "input_layernorm."),
            "feed_forward_norm": PartSpec("rms_norm", norm, p1 + "post_attention_layernorm."),
            "feed_forward": PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": 80}, p1 + "mlp.")}),
    )
    base = _spec([RunStep(0), RunStep(1)], hidden=H)
    spec = ModelSpec("Test", H, 97, 256, base.embedding, layers, (RunStep(0), RunStep(1)), base.final_norm, base.head)
    model, mgr, runner, w = _build_runner(spec, torch.float32)
    assert "model.layers.0.post_mixer_layernorm.weight" in model.declared_tensors()
    narrow = model.cache_groups[1]
    assert (narrow.head_dim, narrow.value_dim) == (HK, HV)
    assert runner.storage.k[1].shape[-1] == HK and runner.storage.v[1].shape[-1] == HV
    with pytest.raises(ValueError, match="missing \\['mixer_post_norm'\\]"):
        from lite_lang_b200.engine.model import CausalLM
        CausalLM(ModelSpec("Test", H, 97, 256, base.embedding,
                           (LayerSpec("toy_sandwich", dict(layers[1].parts)),), (RunStep(0),), base.final_norm, base.head))

    toks = [int(t) for t in np.random.default_rng(6).integers(0, 97, 27)]
    T = len(toks)
    cfgd = {"num_attention_heads": 4, "num_key_value_heads": 2, "hidden_size": H, "head_dim": 16,
            "rope_theta": 10000.0, "rms_norm_eps": 1e-6}
    h = P.embedding(w["model.embed_tokens.weight"], torch.tensor(toks))
    x = P.rms_norm(h, w[p0 + "input_layernorm.weight"], 1e-6)
    a = P.attention_block(x, torch.arange(T), w, p0 + "self_attn.", cfgd, None)
    h = h + P.rms_norm(a, w[p0 + "post_mixer_layernorm.weight"], 1e-6)
    x = P.rms_norm(h, w[p0 + "post_attention_layernorm.weight"], 1e-6)
    h = h + P.gated_mlp(x, w[p0 + "mlp.gate_proj.weight"], w[p0 + "mlp.up_proj.weight"], w[p0 + "mlp.down_proj.weight"])
    x = P.rms_norm(h, w[p1 + "input_layernorm.weight"], 1e-6)
    q = P.linear(x, w[p1 + "narrow.q.weight"]).view(T, NH, HK)
    k = P.linear(x, w[p1 + "narrow.k.weight"]).view(T, NKV, HK)
    v = P.linear(x, w[p1 + "narrow.v.weight"]).view(T, NKV, HV)
    o = torch.zeros(T, NH, HV)
    causal = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    for a_ in range(NH):
        g = a_ // (NH // NKV)
        sc = (q[:, a_].double() @ k[:, g].double().t()) * HK ** -0.5
        o[:, a_] = (torch.softmax(sc.masked_fill(~causal, float("-inf")), dim=-1) @ v[:, g].double()).float()
    h = h + P.linear(o.reshape(T, NH * HV), w[p1 + "narrow.o.weight"])
    x = P.rms_norm(h, w[p1 + "post_attention_layernorm.weight"], 1e-6)
    h = h + P.gated_mlp(x, w[p1 + "mlp.gate_proj.weight"], w[p1 + "mlp.up_proj.weight"], w[p1 + "mlp.down_proj.weight"])
    ref = P.linear(P.rms_norm(h, w["model.norm.weight"], 1e-6), w["lm_head.weight"]).numpy()

    whole, cut = _run_whole_and_cut(runner, mgr, toks)
    assert rel_err(whole, ref) <= 1e-4 and rel_err(cut, ref) <= 1e-4
