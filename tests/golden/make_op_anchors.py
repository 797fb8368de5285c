"""Makes op_anchors.npz: outputs of the reference's own pure-torch per-op helpers on small seeded inputs.

    python tests/golden/make_op_anchors.py <path to a checkout of ppppppppig/lite_lang>

The reference's model code cannot be imported without a GPU, but these helpers
run on the CPU (float32):

  torch_rotary_emb          litelang/kernel/develop_rope/rope.py:225-234
  compute_rotary_emb        litelang/kernel/develop_rope/rope.py:202-222
  torch_silu_and_mul        litelang/kernel/develop_silu_and_mul/silu_and_mul.py:80-84
  standard_attention_no_pad litelang/kernel/develop_flash_attn/flash_attn_v2.py:356-389
  gqa_reference_impl        litelang/kernel/develop_flash_attn/attn_decode_v2.py:392-415
  torch_rmsnorm             litelang/kernel/develop_rmsnorm/rms_norm.py:11-17
                            (cut out of its file with ast: the module asks for cuda:0 at import)

tests/test_plain.py compares the plain implementation with the stored outputs;
the stored file is all it needs.
"""
import ast
import os
import sys

import numpy as np
import torch


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from litelang.kernel.develop_rope.rope import compute_rotary_emb, torch_rotary_emb
    from litelang.kernel.develop_silu_and_mul.silu_and_mul import torch_silu_and_mul
    from litelang.kernel.develop_flash_attn.flash_attn_v2 import standard_attention_no_pad
    from litelang.kernel.develop_flash_attn.attn_decode_v2 import gqa_reference_impl

    src = open(os.path.join(ref_root, "litelang/kernel/develop_rmsnorm/rms_norm.py")).read()
    fn = [n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "torch_rmsnorm"][0]
    ns = {"torch": torch}
    exec(compile(ast.Module([fn], []), "rms_norm.py", "exec"), ns)
    torch_rmsnorm = ns["torch_rmsnorm"]

    g = torch.Generator().manual_seed(20240607)
    out = {}

    x = torch.randn(9, 3, 16, generator=g)
    ang = torch.rand(9, 8, generator=g) * 6.0
    out["rope_x"], out["rope_cos"], out["rope_sin"] = x, torch.cos(ang), torch.sin(ang)
    out["rope_y"] = torch_rotary_emb(x, torch.cos(ang), torch.sin(ang))
    out["rope_theta_y"] = compute_rotary_emb(x, theta=10000)

    gu = torch.randn(5, 24, generator=g)
    out["silu_in"], out["silu_out"] = gu, torch_silu_and_mul(gu)

    xr, gam = torch.randn(6, 40, generator=g), 1 + 0.1 * torch.randn(40, generator=g)
    out["rms_x"], out["rms_w"] = xr, gam
    out["rms_y"] = torch_rmsnorm(xr, gam, 1e-5)

    lens = [5, 9]
    T = sum(lens)
    q, k, v = torch.randn(T, 6, 16, generator=g), torch.randn(T, 2, 16, generator=g), torch.randn(T, 2, 16, generator=g)
    out["att_q"], out["att_k"], out["att_v"] = q, k, v
    out["att_lens"] = torch.tensor(lens)
    out["att_o"] = standard_attention_no_pad(q, k, v, torch.tensor([0, 5]), torch.tensor(lens), 3, 16 ** -0.5)

    qd = torch.randn(2, 6, 16, generator=g)
    out["dec_q"] = qd
    out["dec_o"] = gqa_reference_impl(qd, k, v, torch.tensor([0, 5]), torch.tensor(lens), 16 ** -0.5, 3)

    here = os.path.dirname(os.path.abspath(__file__))
    np.savez(os.path.join(here, "op_anchors.npz"), **{k: np.asarray(v) for k, v in out.items()})
    print("wrote", os.path.join(here, "op_anchors.npz"), {k: tuple(np.asarray(v).shape) for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
