"""Shared pieces of the tests: tiny configurations, model folders, trace replay, comparisons."""

from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Three tiny Qwen2 configurations that differ in every size and option.
TINY = {
    # GQA group 2, head 16, tied head, theta 1e4, eps 1e-6, page 4
    "A": dict(
        config=dict(architectures=["Qwen2ForCausalLM"], hidden_size=64, num_hidden_layers=2,
                    num_attention_heads=4, num_key_value_heads=2, intermediate_size=128, vocab_size=256,
                    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                    max_position_embeddings=128, use_sliding_window=False, torch_dtype="bfloat16"),
        scales=dict(matrix=0.02, bias=0.02, norm=0.05), page_size=4, seed=11, sharpen=8.0),
    # MQA group 3 (no power of two), hidden 96, head 32, untied head, theta 1e6, eps 1e-5, page 8
    "B": dict(
        config=dict(architectures=["Qwen2ForCausalLM"], hidden_size=96, num_hidden_layers=3,
                    num_attention_heads=3, num_key_value_heads=1, intermediate_size=320, vocab_size=384,
                    rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                    max_position_embeddings=256, use_sliding_window=False, torch_dtype="bfloat16"),
        scales=dict(matrix=0.03, bias=0.03, norm=0.1), page_size=8, seed=12, sharpen=4.0),
    # heads of 64 (the tensor-core attention kernels), group 4, a window on layers 1.., page 16,
    # head_dim given explicitly and different from hidden / heads, vocabulary no multiple of 8
    "C": dict(
        config=dict(architectures=["Qwen2ForCausalLM"], hidden_size=160, num_hidden_layers=4,
                    num_attention_heads=8, num_key_value_heads=2, head_dim=64, intermediate_size=208,
                    vocab_size=331, rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
                    max_position_embeddings=512, use_sliding_window=True, sliding_window=40,
                    max_window_layers=1, torch_dtype="bfloat16"),
        scales=dict(matrix=0.05, bias=0.05, norm=0.1), page_size=16, seed=13, sharpen=2.0),
}

# "sharpen" is the factor on the q and k projections that makes the attention scores of a
# configuration spread by about 1.5 (softmax peaked on few keys, so a wrong key shows in the
# logits) without making the logits ill-conditioned: beyond it float32 and bfloat16 errors
# grow together, which says nothing about the engine.

# Relative error of a row of logits: max|ours - ref| / max|ref|.
TOL = {"float32": 1e-4, "bfloat16": 5e-2}


def make_model_folder(name: str, folder: Optional[str] = None, scales: Optional[dict] = None,
                      overrides: Optional[dict] = None, sharpen: float = 1.0) -> str:
    """Write a tiny random model.  ``sharpen`` multiplies the q and k projections so that the
    attention is peaked on few keys and a wrong key would show in the logits."""
    from lite_lang_b200.config import config_from_dict
    from lite_lang_b200.weights import write_random_model

    spec = TINY[name]
    cfg_d = dict(spec["config"])
    if overrides:
        cfg_d.update(overrides)
    cfg = config_from_dict(cfg_d)
    folder = folder or tempfile.mkdtemp(prefix=f"ll_tiny_{name}_")
    sc = dict(spec["scales"])
    if scales:
        sc.update(scales)
    write_random_model(folder, cfg, spec["seed"], sc)
    if sharpen != 1.0:
        from safetensors.torch import load_file, save_file
        path = os.path.join(folder, "model.safetensors")
        t = load_file(path)
        for k in list(t):
            if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
                t[k] = (t[k].float() * sharpen).to(t[k].dtype)
        save_file(t, path, metadata={"format": "pt"})
    return folder


def rel_err(ours: np.ndarray, ref: np.ndarray) -> float:
    ours = np.asarray(ours, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert ours.shape == ref.shape, (ours.shape, ref.shape)
    denom = np.abs(ref).max(axis=-1, keepdims=True)
    return float((np.abs(ours - ref) / denom).max())


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=n)]


class TraceRun:
    """Drives bin/trace_run as a user would: a process, steps on stdin, logits in files."""

    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, extra=(),
                 cache_fill: Optional[str] = None):
        self.out = tempfile.mkdtemp(prefix="ll_trace_")
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
               "--out", self.out, "--max-tokens", str(max_tokens), "--page-size", str(page_size), *extra]
        self.err_path = os.path.join(self.out, "stderr.txt")
        self._err = open(self.err_path, "w")
        env = dict(os.environ)
        if cache_fill is not None:            # what the cache pools hold before anything is written to them
            env["LITE_LANG_B200_CACHE_FILL"] = cache_fill
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=self._err,
                                     text=True, bufsize=1, env=env)
        self.step_no = 0
        self.vocab = json.load(open(os.path.join(model_dir, "config.json")))["vocab_size"]

    def step(self, entries: Sequence[dict], end: Sequence[str] = ()) -> Optional[np.ndarray]:
        """entries: [{"id", "tokens", "want"}].  Returns the wanted logits [wanted, vocab] or None."""
        n = self.step_no
        self.step_no += 1
        self.proc.stdin.write(json.dumps({"step": n, "entries": list(entries), "end": list(end)}) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {n}":
            rest = self.proc.stdout.read()
            self._err.flush()
            raise RuntimeError(f"trace_run answered {line!r} {rest!r} (exit {self.proc.poll()}):\n"
                               + open(self.err_path).read()[-3000:])
        wanted = sum(len(e.get("want", [])) for e in entries)
        if wanted == 0:
            return None
        arr = np.fromfile(os.path.join(self.out, f"{n}.f32"), dtype="<f4")
        return arr.reshape(wanted, self.vocab)

    def close(self) -> int:
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=120)
        self._err.close()
        return rc

    def pages_reused(self) -> int:
        """Pages handed out a second time, from the summary trace_run prints when its input ends."""
        import re
        m = re.search(r"pages reused (\d+)", open(self.err_path).read())
        return int(m.group(1)) if m else -1
