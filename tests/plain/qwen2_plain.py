"""Plain, slow Qwen2 forward pass used as the oracle of the test-suite.

Whole sequences, no cache, one function for each part; float32 tensors, with the
sums of the matrix products and of the softmax taken in float64 and rounded
once, so that the oracle's own summation order stays out of the comparison.  It shares no code with ``lite_lang_b200``: it reads ``config.json``
and ``model.safetensors`` itself and works on ordinary torch tensors on the CPU
(or on whatever device the caller moves the weights to).

Source of the formulas.  The model code of ppppppppig/lite_lang cannot be
imported on a machine without a GPU (``litelang/kernel/develop_rmsnorm/
rms_norm.py:6-8`` asks for ``cuda:0`` at import time and every layer calls
``.cuda()``), so the whole-model output rests on the formulas of that code as
cited at each function below.  Its pure-torch per-op helpers do run on the CPU;
``tests/golden/make_op_anchors.py`` compares the functions of this file with
them once and the outputs are committed beside that script.

Where the reference hard-codes a constant that ``config.json`` gives
(``rope_theta`` in ``pre_layer.py:22``, the norm eps in
``transformer_layer.py:41`` and ``post_layer.py:12``), this file takes the value
from ``config.json``: that is the behaviour of a Qwen2 model built from its own
configuration, which is what the engine has to equal.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open


# --------------------------------------------------------------------------
# reading a model folder
# --------------------------------------------------------------------------

def read_model_folder(model_dir: str, device: str = "cpu"):
    """config.json as a dict and every tensor of model.safetensors in float32.

    Reference: ``litelang/models/qwen2/model.py:61-97`` (reads every tensor of
    the checkpoint by name into a dict) and ``model.py:9-21`` (config keys).
    """
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as fh:
        for name in fh.keys():
            tensors[name] = fh.get_tensor(name).to(torch.float32).to(device)
    return cfg, tensors


def layer_window(cfg: dict, layer: int) -> Optional[int]:
    """Sliding window of a layer, or None.

    The reference has no windowed attention at all.  The keys are those of the
    architecture's config.json: with ``use_sliding_window`` true, layers with an
    index of at least ``max_window_layers`` look at the last ``sliding_window``
    positions only (the position itself included).
    """
    if not cfg.get("use_sliding_window", False):
        return None
    w = cfg.get("sliding_window")
    if w is None:
        return None
    if layer >= int(cfg.get("max_window_layers", 0)):
        return int(w)
    return None


# --------------------------------------------------------------------------
# one function for each part
# --------------------------------------------------------------------------

def embedding(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """h[t] = E[token[t]].  Reference: ``qwen2/layer/pre_layer.py:15-19``."""
    return table[tokens.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w, row by row, in float32.

    Reference: ``kernel/develop_rmsnorm/rms_norm.py:11-17`` (torch_rmsnorm) and
    the kernel at ``rms_norm.py:43-53``.
    """
    x = x.to(torch.float32)
    variance = torch.sum(x * x, dim=-1, keepdim=True) / x.shape[-1]
    return x / torch.sqrt(variance + eps) * weight.to(torch.float32)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x @ W^T (+ b) with W stored [out, in] as in the checkpoint.

    Reference: ``transformer_layer.py:95-109`` (addmm with the transposed
    weight and the bias) and ``load_weights.py:15-37`` (the transpose).
    Computed in float64 and rounded once so that the oracle's own summation
    order does not enter the comparison.
    """
    y = x.to(torch.float64) @ weight.to(torch.float64).t()
    if bias is not None:
        y = y + bias.to(torch.float64)
    return y.to(torch.float32)


def rope_tables(head_dim: int, theta: float, positions: torch.Tensor):
    """cos and sin of position * theta^(-2i/head_dim), i < head_dim/2, float32.

    Reference: ``qwen2/layer/pre_layer.py:21-30`` and
    ``kernel/develop_rope/rope.py:202-216``.
    """
    freqs = 1.0 / theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim)
    angle = positions.to(torch.float32)[:, None] * freqs[None, :].to(positions.device)
    return torch.cos(angle), torch.sin(angle)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split rotation of x [T, heads, head_dim]: pairs are (i, i + d/2).

    Reference: ``kernel/develop_rope/rope.py:225-234`` (torch_rotary_emb) and
    the kernel at ``rope.py:81-82,136-137``.
    """
    d = x.shape[-1]
    x0, x1 = x[..., : d // 2], x[..., d // 2:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((x0 * c - x1 * s, x0 * s + x1 * c), dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.

    q [T, nh, hd]; k, v [T, nkv, hd].  Query head a uses kv head
    a // (nh / nkv); score = q.k / sqrt(hd); keys j <= t only (and
    j > t - window when a window is given); softmax in float32.

    Reference: ``kernel/develop_flash_attn/flash_attn_v2.py:356-389``
    (standard_attention_no_pad), ``transformer_layer.py:39-42`` (group and
    scale) and ``flash_attn_v2.py:428,475-478`` (head mapping and mask).
    """
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    pos = torch.arange(T, device=q.device)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed = allowed & (pos[None, :] > pos[:, None] - window)
    out = torch.zeros_like(q)
    for a in range(nh):
        g = a // group
        scores = (q[:, a, :].to(torch.float64) @ k[:, g, :].to(torch.float64).t()) * scale
        scores = torch.where(allowed, scores, torch.full_like(scores, -float("inf")))
        weights = torch.softmax(scores, dim=-1)
        out[:, a, :] = (weights @ v[:, g, :].to(torch.float64)).to(torch.float32)
    return out


def silu_and_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up.  Reference: ``kernel/develop_silu_and_mul/silu_and_mul.py:80-84``."""
    return gate / (1.0 + torch.exp(-gate)) * up


def gated_mlp(x, w_gate, w_up, w_down):
    """down(silu(gate(x)) * up(x)), no biases.  Reference: ``transformer_layer.py:79-83``."""
    return linear(silu_and_mul(linear(x, w_gate), linear(x, w_up)), w_down)


def attention_block(x, positions, w: Dict[str, torch.Tensor], prefix: str, cfg: dict, window: Optional[int]):
    """q/k/v projections with bias, rotation of q and k, attention, output projection.

    Reference: ``transformer_layer.py:94-116`` (_QkvCompute) and ``:140-194``
    (_ComputeAttnScore; the output projection has no bias, ``:193``).
    """
    nh = cfg["num_attention_heads"]
    nkv = cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    T = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"], w.get(prefix + "q_proj.bias")).view(T, nh, hd)
    k = linear(x, w[prefix + "k_proj.weight"], w.get(prefix + "k_proj.bias")).view(T, nkv, hd)
    v = linear(x, w[prefix + "v_proj.weight"], w.get(prefix + "v_proj.bias")).view(T, nkv, hd)
    cos, sin = rope_tables(hd, float(cfg.get("rope_theta", 10000.0)), positions)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = attention(q, k, v, window)
    return linear(o.reshape(T, nh * hd), w[prefix + "o_proj.weight"])


def decoder_layer(h, positions, w, layer: int, cfg: dict):
    """Pre-norm block: h += attn(norm(h)); h += mlp(norm(h)).

    Reference: ``transformer_layer.py:46-77`` (Forward).
    """
    p = f"model.layers.{layer}."
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    x = rms_norm(h, w[p + "input_layernorm.weight"], eps)
    h = h + attention_block(x, positions, w, p + "self_attn.", cfg, layer_window(cfg, layer))
    x = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
    h = h + gated_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return h


def forward_logits(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence.

    Reference: ``qwen2/model.py:48-59`` (embedding, the layers in order, post
    layer) and ``qwen2/layer/post_layer.py:14-24,43-45`` (final norm, lm_head,
    which is the embedding table when ``tie_word_embeddings``,
    ``post_layer_weights.py:10-15``).
    """
    tok = torch.as_tensor(list(tokens), dtype=torch.long, device=w["model.embed_tokens.weight"].device)
    positions = torch.arange(tok.shape[0], device=tok.device)
    h = embedding(w["model.embed_tokens.weight"], tok)
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, positions, w, layer, cfg)
    y = rms_norm(h, w["model.norm.weight"], float(cfg.get("rms_norm_eps", 1e-6)))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(y, head)


def greedy_generate(cfg: dict, w, prompt: Sequence[int], n_new: int) -> List[int]:
    """n_new tokens by argmax, recomputing the whole sequence at every token.

    Reference: ``qwen2/layer/post_layer.py:75-77`` (argmax of the logits).
    """
    seq = list(prompt)
    out: List[int] = []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward_logits(cfg, w, seq)[-1]).item())
        out.append(nxt)
        seq.append(nxt)
    return out


def temperature_probs(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """softmax(logits / temperature) in float64.

    Reference: the disabled sampler at ``qwen2/layer/post_layer.py:47-50``
    (divide by temperature, softmax).
    """
    return torch.softmax(logits.to(torch.float64) / temperature, dim=-1)
