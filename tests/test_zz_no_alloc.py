"""ll_attn_mma_static: attention whose scratch memory is part of the library (GPU).

Some users of these kernels cannot allocate device memory once they are running: a server
that handed all free memory to its own pools at start-up, or a plug-in inside a runtime
whose allocator it cannot use.  For them the library exports one C entry point that takes
its scratch memory from a fixed array inside the library.  This test calls that entry point
through its exported C symbol, twice in a row, and compares each result with the ordinary
entry point, which is given scratch memory by the caller, and with the plain attention formula.
That nothing is allocated is read from the driver (cudaMemGetInfo: the free memory of the device
is the same before and after a call), not from torch's own allocator, which cannot see what a
library loaded beside it does.  It also checks that a launch that would not fit the built-in array
is refused with a message, and that nothing else changed.

The file sorts last so that a run that stops at the first failure has run everything else.
"""
import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import pytest
import torch

from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

TOO_LARGE = 100001


def _case(seed, nh, nkv, hd, ps, lens, q_lens, with_plain=True):
    """Cached keys and values in scattered pages and the step's queries (all bfloat16)."""
    d = torch.device("cuda:0")
    g = torch.Generator().manual_seed(seed)
    n = len(lens)
    max_blocks = max((l + ps - 1) // ps for l in lens) + 1
    num_pages = sum((l + ps - 1) // ps for l in lens) + 2
    perm = torch.randperm(num_pages, generator=g).tolist()
    bt = torch.full((n, max_blocks), -1, dtype=torch.int32)
    for i, l in enumerate(lens):
        for lp in range((l + ps - 1) // ps):
            bt[i, lp] = perm.pop()
    kc = torch.randn(num_pages, nkv, ps, hd, generator=g).to(torch.bfloat16).to(d)
    vc = torch.randn(num_pages, nkv, ps, hd, generator=g).to(torch.bfloat16).to(d)
    q = torch.randn(sum(q_lens), nh * hd, generator=g).to(torch.bfloat16).to(d)
    cu = [0]
    for ql in q_lens:
        cu.append(cu[-1] + ql)
    # the plain formula on each request's keys and values, gathered from its pages
    ref, row = [], 0
    for i, (l, ql) in enumerate(zip(lens, q_lens) if with_plain else ()):
        pages = [int(x) for x in bt[i, :(l + ps - 1) // ps]]
        k = torch.cat([kc[pg].float().cpu().transpose(0, 1) for pg in pages])[:l]      # [l, nkv, hd]
        v = torch.cat([vc[pg].float().cpu().transpose(0, 1) for pg in pages])[:l]
        qq = torch.zeros(l, nh, hd)
        qq[l - ql:] = q[row:row + ql].float().cpu().view(ql, nh, hd)
        ref.append(P.attention(qq, k, v)[l - ql:].reshape(ql, nh * hd))
        row += ql
    return dict(q=q, kc=kc, vc=vc, bt=bt.to(d), cu_q=torch.tensor(cu, dtype=torch.int32, device=d),
                plain=torch.cat(ref) if ref else None,
                ctx=torch.tensor([l - ql for l, ql in zip(lens, q_lens)], dtype=torch.int32, device=d),
                slots=torch.arange(n, dtype=torch.int32, device=d),
                blocks=sum((ql * (nh // nkv) + 15) // 16 for ql in q_lens))


def _call_static(lib, c, out, nh, nkv, hd, ps, nsplit):
    fn = lib.ll_attn_mma_static
    fn.restype = c_int
    p = lambda t: c_void_p(t.data_ptr())
    return fn(p(out), c_long(out.stride(0)), p(c["q"]), c_long(c["q"].stride(0)), p(c["kc"]), p(c["vc"]), p(c["bt"]),
              c_int(c["bt"].stride(0)), p(c["cu_q"]), p(c["ctx"]), p(c["slots"]), c_int(c["slots"].numel()),
              c_int(c["blocks"]), c_int(nh), c_int(nkv), c_int(hd), c_int(ps), c_int(c["kc"].shape[0]), c_int(0),
              c_float(hd ** -0.5), c_int(nsplit), c_void_p(0), c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_point_equals_the_ordinary_one():
    from lite_lang_b200 import ops
    from lite_lang_b200.csrc.build import build_library

    lib = ctypes.CDLL(build_library("attn_mma_static"))
    lib.ll_attn_mma_static_error.restype = ctypes.c_char_p
    nh, nkv, hd, ps = 12, 2, 128, 16
    # two different launches in a row: the second finds the array as the first left it
    for seed, lens, q_lens, nsplit in [(31, [900, 40, 333], [1, 1, 1], 6), (32, [257, 64], [20, 1], 3)]:
        c = _case(seed, nh, nkv, hd, ps, lens, q_lens)
        want = torch.zeros_like(c["q"])
        scratch = torch.empty(ops.attn_mma_scratch_floats(c["blocks"], nkv, nsplit, hd), device=c["q"].device)
        counters = torch.zeros(c["blocks"] * nkv, dtype=torch.int32, device=c["q"].device)
        ops.attn_mma(want, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], c["cu_q"], c["ctx"], c["slots"],
                     len(lens), c["blocks"], nh, nkv, hd, ps, None, hd ** -0.5, nsplit, scratch, counters, None)
        outs = [torch.full_like(c["q"], 5.0) for _ in range(3)]
        # (the first call may load the kernel's code and look up the array's address: it is not measured)
        assert _call_static(lib, c, outs[0], nh, nkv, hd, ps, nsplit) == 0, lib.ll_attn_mma_static_error()
        torch.cuda.synchronize()
        for attempt in (1, 2):
            got = outs[attempt]
            free_before, _ = torch.cuda.mem_get_info()
            rc = _call_static(lib, c, got, nh, nkv, hd, ps, nsplit)
            assert rc == 0, lib.ll_attn_mma_static_error()
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before, "the device's free memory changed during the call"
            scale = float(want.float().abs().max())
            err = float((got.float() - want.float()).abs().max()) / scale
            assert err <= 1.6e-2, (seed, attempt, err)       # the tolerance of the kernel tests for bfloat16
            plain = c["plain"]
            err = float((got.float().cpu() - plain).abs().max()) / float(plain.abs().max())
            assert err <= 1.6e-2, (seed, attempt, err)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from lite_lang_b200.csrc.build import build_library

    lib = ctypes.CDLL(build_library("attn_mma_static"))
    lib.ll_attn_mma_static_error.restype = ctypes.c_char_p
    nh, nkv, hd, ps = 12, 2, 128, 16
    c = _case(33, nh, nkv, hd, ps, [4000] * 8, [1] * 8, with_plain=False)
    out = torch.full_like(c["q"], 5.0)
    rc = _call_static(lib, c, out, nh, nkv, hd, ps, 64)       # 8 * 2 * 64 * 16 * 130 floats > 8 MiB
    assert rc == TOO_LARGE
    msg = lib.ll_attn_mma_static_error().decode()
    assert "scratch floats" in msg and "2097152" in msg
    torch.cuda.synchronize()
    assert float((out.float() - 5.0).abs().max()) == 0.0      # nothing was launched
    assert _call_static(lib, c, out, nh, nkv, hd, ps, 4) == 0  # the same step with fewer splits fits
    torch.cuda.synchronize()
