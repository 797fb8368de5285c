"""Weights by name, error reporting, random-weights mode (no GPU)."""
import json
import os
import tempfile

import pytest
import torch
from safetensors.torch import load_file, save_file

from helpers import TINY, make_model_folder
from lite_lang_b200.config import config_from_dict, load_config
from lite_lang_b200.engine.model import CausalLM
from lite_lang_b200.weights import Checkpoint, WeightError, load_weights, write_random_model


def _model(name):
    return CausalLM(config_from_dict(TINY[name]["config"]).model_spec())


def test_declared_names_are_the_checkpoint_names():
    names = set(_model("A").declared_tensors())
    assert "model.embed_tokens.weight" in names and "model.norm.weight" in names
    assert "model.layers.1.self_attn.k_proj.bias" in names
    assert "model.layers.0.mlp.gate_proj.weight" in names
    assert "model.layers.1.post_attention_layernorm.weight" in names
    assert "lm_head.weight" in names and _model("A").declared_tensors()["lm_head.weight"].optional
    assert not _model("B").declared_tensors()["lm_head.weight"].optional


def test_random_folder_is_seeded_and_complete():
    with tempfile.TemporaryDirectory() as d1, tempfile.TemporaryDirectory() as d2:
        make_model_folder("B", d1)
        make_model_folder("B", d2)
        a, b = load_file(os.path.join(d1, "model.safetensors")), load_file(os.path.join(d2, "model.safetensors"))
        assert set(a) == set(b)
        for k in a:
            assert a[k].dtype == torch.bfloat16
            assert torch.equal(a[k], b[k])
        assert "lm_head.weight" in a
        norm = a["model.layers.0.input_layernorm.weight"].float()
        assert abs(norm.mean().item() - 1.0) < 0.1
        cfg = load_config(d1)
        assert cfg.num_attention_heads == 3
    with tempfile.TemporaryDirectory() as d3:
        make_model_folder("A", d3)
        assert "lm_head.weight" not in load_file(os.path.join(d3, "model.safetensors"))   # tied


def test_load_on_cpu_fuses_and_keeps_dtypes():
    with tempfile.TemporaryDirectory() as d:
        make_model_folder("A", d)
        raw = load_file(os.path.join(d, "model.safetensors"))
        m = _model("A")
        load_weights(m, d, torch.bfloat16, torch.device("cpu"))
        att = m.blocks[0].mixer
        assert att.w_qkv.shape == (64 + 2 * 32, 64) and att.w_qkv.dtype == torch.bfloat16
        assert torch.equal(att.w_qkv[:64], raw["model.layers.0.self_attn.q_proj.weight"])
        assert torch.equal(att.w_qkv[64:96], raw["model.layers.0.self_attn.k_proj.weight"])
        assert att.b_qkv.dtype == torch.float32           # biases and norm weights: float32, exact
        assert torch.equal(att.b_qkv[96:], raw["model.layers.0.self_attn.v_proj.bias"].float())
        ffn = m.blocks[1].feed_forward
        assert ffn.w_gate_up.shape == (256, 64)
        assert torch.equal(ffn.w_gate_up[128:], raw["model.layers.1.mlp.up_proj.weight"])
        assert m.blocks[0].mixer_norm.weight.dtype == torch.float32
        assert m.head.weight is m.embedding.weight         # tied: one buffer
        m32 = _model("A")
        load_weights(m32, d, torch.float32, torch.device("cpu"))
        assert m32.blocks[0].mixer.w_qkv.dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    with tempfile.TemporaryDirectory() as d:
        make_model_folder("B", d)
        path = os.path.join(d, "model.safetensors")
        t = load_file(path)
        del t["model.layers.2.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
        t["model.layers.1.self_attn.q_proj.weight"] = torch.zeros(96, 95, dtype=torch.bfloat16)
        save_file(t, path)
        with pytest.raises(WeightError) as ei:
            load_weights(_model("B"), d, torch.bfloat16, torch.device("cpu"))
        msg = str(ei.value)
        assert "missing (2)" in msg and "model.layers.2.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
        assert "unexpected (1)" in msg and "rotary_emb.inv_freq" in msg
        assert "wrong shape (1)" in msg and "expected [96, 96] found [96, 95]" in msg


def test_untied_model_needs_lm_head_and_tied_may_repeat_it():
    with tempfile.TemporaryDirectory() as d:
        make_model_folder("B", d)
        path = os.path.join(d, "model.safetensors")
        t = load_file(path)
        del t["lm_head.weight"]
        save_file(t, path)
        with pytest.raises(WeightError, match="lm_head.weight"):
            load_weights(_model("B"), d, torch.bfloat16, torch.device("cpu"))
    with tempfile.TemporaryDirectory() as d:
        make_model_folder("A", d)
        path = os.path.join(d, "model.safetensors")
        t = load_file(path)
        t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
        save_file(t, path)
        m = _model("A")
        load_weights(m, d, torch.bfloat16, torch.device("cpu"))     # accepted, the table is used
        assert m.head.weight is m.embedding.weight


def test_sharded_checkpoint_with_index():
    with tempfile.TemporaryDirectory() as d:
        make_model_folder("A", d)
        path = os.path.join(d, "model.safetensors")
        t = load_file(path)
        names = sorted(t)
        half = len(names) // 2
        save_file({k: t[k] for k in names[:half]}, os.path.join(d, "model-00001-of-00002.safetensors"))
        save_file({k: t[k] for k in names[half:]}, os.path.join(d, "model-00002-of-00002.safetensors"))
        os.remove(path)
        wm = {k: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
              for i, k in enumerate(names)}
        with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
            json.dump({"weight_map": wm}, fh)
        ck = Checkpoint(d)
        assert ck.names() == names
        m = _model("A")
        load_weights(m, d, torch.float32, torch.device("cpu"))
        assert torch.equal(m.embedding.weight, t["model.embed_tokens.weight"].float())


def test_missing_files():
    with tempfile.TemporaryDirectory() as d:
        with pytest.raises(WeightError, match="model.safetensors"):
            Checkpoint(d)
