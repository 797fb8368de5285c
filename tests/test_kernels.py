"""Each CUDA kernel alone against its plain float32 formula, at sizes other than the engine tests' (GPU)."""
import math

import numpy as np
import pytest
import torch

from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def dev():
    return torch.device("cuda:0")


def tol(dtype):
    return 2e-6 if dtype == torch.float32 else 1.6e-2     # bfloat16: two roundings of 2^-8 relative


def assert_close(got, ref, dtype, what=""):
    got, ref = got.float().cpu(), ref.float().cpu()
    scale = float(ref.abs().max()) or 1.0
    err = float((got - ref).abs().max()) / scale
    assert err <= tol(dtype), f"{what}: {err:.3e} > {tol(dtype):.1e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(72, 101), (1536, 333), (50, 7)])
def test_embedding(dtype, hidden, vocab):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, hidden, generator=g).to(dtype).to(dev())
    ids = torch.randint(0, vocab, (37,), generator=g, dtype=torch.int32).to(dev())
    out = torch.empty(37, hidden, dtype=dtype, device=dev())
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.embed_gather(out, table, ids, status)
    assert torch.equal(out.cpu(), P.embedding(table.cpu(), ids.cpu()))
    assert status.item() == 0
    bad = ids.clone()
    bad[3] = vocab
    ops.embed_gather(out, table, bad, status)
    assert status.item() == 1 and float(out[3].float().abs().max()) == 0.0     # refused, not read out of bounds


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden,eps", [(5, 96, 1e-5), (33, 1536, 1e-6), (2, 250, 1e-3), (1, 8192, 1e-6),
                                             # many rows: the warp-a-row kernel of the bfloat16 path, each width class
                                             (1100, 1536, 1e-6), (1024, 160, 1e-5), (1030, 896, 1e-6), (1500, 2048, 1e-6),
                                             (1200, 3584, 1e-6)])
def test_rmsnorm_alone_and_fused(dtype, rows, hidden, eps):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(1)
    x = (3 * torch.randn(rows, hidden, generator=g)).to(dtype)
    d = torch.randn(rows, hidden, generator=g).to(dtype)
    w = (1 + 0.2 * torch.randn(hidden, generator=g))
    xd, dd, wd = x.to(dev()), d.to(dev()), w.to(dev())
    out = torch.empty_like(xd)
    ops.rmsnorm(out, xd, wd, eps)
    assert_close(out, P.rms_norm(x.float(), w, eps), dtype, "rmsnorm")
    # fused with the residual sum: the residual is replaced by the rounded sum
    res = xd.clone()
    ops.add_rmsnorm(out, res, dd, wd, eps)
    s = (x.float() + d.float()).to(dtype)
    assert torch.equal(res.cpu(), s)
    assert_close(out, P.rms_norm(s.float(), w, eps), dtype, "add_rmsnorm")
    # selected rows only, nothing written back
    rows_idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=dev())
    res2 = xd.clone()
    out2 = torch.empty(2, hidden, dtype=dtype, device=dev())
    ops.add_rmsnorm(out2, res2, dd, wd, eps, rows_idx)
    assert torch.equal(res2, xd)
    assert_close(out2, P.rms_norm(s.float(), w, eps)[[rows - 1, 0]], dtype, "add_rmsnorm rows")
    if rows >= 1024:    # many selected rows, and the plain norm of many rows (no delta: nothing written back)
        many = torch.arange(rows - 1, -1, -1, dtype=torch.int32, device=dev())
        res3 = xd.clone()
        out3 = torch.empty(rows, hidden, dtype=dtype, device=dev())
        ops.add_rmsnorm(out3, res3, dd, wd, eps, many)
        assert torch.equal(res3, xd)
        assert_close(out3, P.rms_norm(s.float(), w, eps).flip(0), dtype, "add_rmsnorm of many selected rows")
        res4 = xd.clone()
        ops.add_rmsnorm(out3, res4, None, wd, eps)
        assert torch.equal(res4, xd)
        assert_close(out3, P.rms_norm(x.float(), w, eps), dtype, "norm of many rows without a delta")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [8, 40, 203, 8960])
def test_silu_mul(dtype, inter):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(2)
    gu = (2 * torch.randn(7, 2 * inter, generator=g)).to(dtype)
    out = torch.empty(7, inter, dtype=dtype, device=dev())
    ops.silu_mul(out, gu.to(dev()))
    assert_close(out, P.silu_and_mul(gu[:, :inter].float(), gu[:, inter:].float()), dtype, "silu_mul")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rot,ps", [(6, 2, 48, 48, 4), (3, 1, 128, 128, 16), (4, 4, 80, 32, 8)])
def test_bias_rope_store(dtype, nh, nkv, hd, rot, ps):
    from lite_lang_b200 import ops
    from lite_lang_b200.parts.rope import rope_table
    g = torch.Generator().manual_seed(3)
    T, max_pos, num_pages = 11, 300, 9
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, width, generator=g).to(dtype)
    bias = 0.5 * torch.randn(width, generator=g)
    pos = torch.randint(0, max_pos, (T,), generator=g, dtype=torch.int32)
    slots = torch.randperm(num_pages * ps, generator=g)[:T].to(torch.int32)
    slots[4] = -1                                             # a token whose k/v are not stored
    table = rope_table(rot, 12345.0, max_pos)
    kc = torch.zeros(num_pages, nkv, ps, hd, dtype=dtype, device=dev())
    vc = torch.zeros_like(kc)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    q_dev = qkv.to(dev()).clone()
    ops.bias_rope_store(q_dev, bias.to(dev()), pos.to(dev()), table.to(dev()), nh, nkv, hd, slots.to(dev()), kc, vc,
                        ps, status)
    assert status.item() == 0
    x = qkv.float() + bias
    q = x[:, :nh * hd].view(T, nh, hd)
    k = x[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    v = x[:, (nh + nkv) * hd:].view(T, nkv, hd)
    cos, sin = P.rope_tables(rot, 12345.0, pos)
    q_ref = torch.cat((P.apply_rope(q[..., :rot], cos, sin), q[..., rot:]), dim=-1)
    k_ref = torch.cat((P.apply_rope(k[..., :rot], cos, sin), k[..., rot:]), dim=-1)
    assert_close(q_dev[:, :nh * hd].view(T, nh, hd), q_ref, dtype, "q")
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        page, off = divmod(s, ps)
        assert_close(kc[page, :, off, :], k_ref[t], dtype, f"k of token {t}")
        assert_close(vc[page, :, off, :], v[t], dtype, f"v of token {t}")
    used = {int(s) for s in slots if s >= 0}
    for s in range(num_pages * ps):                            # nothing else was touched
        if s not in used:
            page, off = divmod(s, ps)
            assert float(kc[page, :, off, :].float().abs().max()) == 0.0


def _paged_case(dtype, nh, nkv, hd, ps, lens, q_lens, window, seed, peak=None):
    """Requests with `lens` cached tokens each, the last `q_lens` of which are this step's queries.
    Pages are scattered over the pool in a random order.  Returns kernel inputs and the plain result."""
    g = torch.Generator().manual_seed(seed)
    n = len(lens)
    max_blocks = max((l + ps - 1) // ps for l in lens) + 1
    num_pages = sum((l + ps - 1) // ps for l in lens) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    bt = torch.full((n + 2, max_blocks), -1, dtype=torch.int32)
    kc = torch.zeros(num_pages, nkv, ps, hd)
    vc = torch.zeros(num_pages, nkv, ps, hd)
    slots_of_req = [1 + i for i in range(n)]                   # request slots differ from entry indices
    q_rows, token_req, positions, ref_rows = [], [], [], []
    for i, (l, ql) in enumerate(zip(lens, q_lens)):
        k = torch.randn(l, nkv, hd, generator=g)
        v = torch.randn(l, nkv, hd, generator=g)
        q = torch.randn(l, nh, hd, generator=g)
        if peak is not None:                                   # one far key dominates the last query
            far = peak(l)
            k[far] *= 0.0
            k[far, :, 0] = 30.0
            q[l - 1] *= 0.1
            q[l - 1, :, 0] = 30.0 / math.sqrt(hd) * 4
            v[far] = 5.0
        k, v, q = k.to(dtype).float(), v.to(dtype).float(), q.to(dtype).float()
        for lp in range((l + ps - 1) // ps):
            page = perm.pop()
            bt[slots_of_req[i], lp] = page
            m = min(ps, l - lp * ps)
            kc[page, :, :m] = k[lp * ps:lp * ps + m].transpose(0, 1)
            vc[page, :, :m] = v[lp * ps:lp * ps + m].transpose(0, 1)
        o = P.attention(q, k, v, window)
        for t in range(l - ql, l):
            q_rows.append(q[t].reshape(-1))
            token_req.append(i)
            positions.append(t)
            ref_rows.append(o[t].reshape(-1))
    d = dev()
    return dict(q=torch.stack(q_rows).to(dtype).to(d), kc=kc.to(dtype).to(d), vc=vc.to(dtype).to(d), bt=bt.to(d),
                token_req=torch.tensor(token_req, dtype=torch.int32, device=d),
                req_slot=torch.tensor(slots_of_req, dtype=torch.int32, device=d),
                positions=torch.tensor(positions, dtype=torch.int32, device=d),
                ref=torch.stack(ref_rows), lens=lens, q_lens=q_lens)


GENERIC_SHAPES = [
    # nh, nkv, hd, page, lens, q_lens, window
    (6, 2, 48, 4, [70, 1, 33], [70, 1, 5], None),
    (10, 1, 80, 16, [300, 45], [1, 45], None),             # group 10 > 8 heads a block
    (3, 3, 256, 8, [40, 129], [3, 1], None),
    (4, 2, 32, 32, [200, 64, 65], [10, 64, 1], 33),
    (8, 2, 128, 16, [700], [1], None),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,ps,lens,q_lens,window", GENERIC_SHAPES)
def test_paged_attention_generic(dtype, nh, nkv, hd, ps, lens, q_lens, window):
    from lite_lang_b200 import ops
    c = _paged_case(dtype, nh, nkv, hd, ps, lens, q_lens, window, seed=5)
    out = torch.empty_like(c["q"])
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.paged_attention_generic(out, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], c["token_req"],
                                c["req_slot"], c["positions"], c["q"].shape[0], nh, nkv, hd, ps, window,
                                hd ** -0.5, status)
    assert status.item() == 0
    assert_close(out, c["ref"], dtype, "generic attention")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("where", ["first", "page_edge", "window_in", "window_out"])
def test_generic_attention_finds_one_far_key(dtype, where):
    """A single key carries nearly all the weight: a kernel that misses it (a page's first slot, the
    window's first position) or reads it although the window excludes it gives a very different row."""
    from lite_lang_b200 import ops
    nh, nkv, hd, ps, L, window = 4, 2, 64, 16, 400, None
    if where == "first":
        peak = lambda l: 0
    elif where == "page_edge":
        peak = lambda l: 16 * 7
    else:
        window = 100
        peak = (lambda l: l - 100) if where == "window_in" else (lambda l: l - 101)
    c = _paged_case(dtype, nh, nkv, hd, ps, [L], [1], window, seed=6, peak=peak)
    out = torch.empty_like(c["q"])
    ops.paged_attention_generic(out, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], c["token_req"],
                                c["req_slot"], c["positions"], 1, nh, nkv, hd, ps, window, hd ** -0.5, None)
    assert_close(out, c["ref"], dtype, where)
    mean_v = float(c["ref"].mean())
    assert (mean_v > 4.5) == (where != "window_out")          # the case does what it is meant to do


MMA_SHAPES = [
    # nh, nkv, hd, page, lens, q_lens, window, nsplit
    (12, 2, 128, 16, [700, 33, 1], [1, 1, 1], None, 1),          # decode, group 6
    (12, 2, 128, 16, [700, 33, 1], [1, 1, 1], None, 7),          # the same, keys split over CTAs
    (8, 2, 64, 16, [130, 64, 65, 17], [130, 1, 20, 17], None, 1),  # whole prompts and portions
    (8, 2, 64, 32, [300, 90], [37, 90], None, 3),                # portions with splits, page 32
    (3, 1, 128, 64, [257], [100], None, 2),                      # group 3, page 64
    (40, 2, 64, 16, [99, 50], [2, 1], None, 4),                  # group 20: a token's heads span row blocks
    (4, 4, 128, 16, [200, 77], [5, 1], 50, 2),                   # window
    (8, 2, 64, 16, [160], [160], 33, 1),                         # window inside a whole prompt
    (12, 2, 128, 16, [2100, 33, 1, 640], [1, 1, 1, 1], None, 8),  # decode, splits of 2, 4, 8, 16 also as clusters
    (12, 2, 128, 16, [4000, 700], [1, 1], None, 16),
    (8, 2, 64, 16, [3000], [1], None, 16),
    (8, 2, 64, 16, [500, 90], [1, 30], None, 4),
    (3, 1, 128, 32, [257, 300], [100, 1], 120, 2),
    (12, 2, 128, 16, [4500, 60], [1, 1], None, 1),               # more tiles than the block table's shared-memory copy holds
]


def _run_mma(c, nh, nkv, hd, ps, window, nsplit, cluster=False, warps=4):
    from lite_lang_b200 import ops
    d = dev()
    lens, q_lens = c["lens"], c["q_lens"]
    group = nh // nkv
    cu = [0]
    for ql in q_lens:
        cu.append(cu[-1] + ql)
    cu_q = torch.tensor(cu, dtype=torch.int32, device=d)
    ctx = torch.tensor([l - ql for l, ql in zip(lens, q_lens)], dtype=torch.int32, device=d)
    blocks = sum((ql * group + 15) // 16 for ql in q_lens)
    scratch = counters = None
    if nsplit > 1 and not cluster:
        scratch = torch.full((ops.attn_mma_scratch_floats(blocks, nkv, nsplit, hd),), float("nan"), device=d)
        counters = torch.zeros(blocks * nkv, dtype=torch.int32, device=d)
    out = torch.full_like(c["q"], 3.0)
    status = torch.zeros(1, dtype=torch.int32, device=d)
    single = all(ql == 1 for ql in q_lens) and group <= 16     # the decode fast path when it applies
    for _ in range(2):          # twice: the counters must come back to zero
        ops.attn_mma(out, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], cu_q, ctx, c["req_slot"], len(lens),
                     blocks, nh, nkv, hd, ps, window, hd ** -0.5, nsplit, scratch, counters, status, single, cluster,
                     warps)
    assert status.item() == 0
    if counters is not None:
        assert int(counters.abs().sum()) == 0
    return out


@pytest.mark.parametrize("nh,nkv,hd,ps,lens,q_lens,window,nsplit", MMA_SHAPES)
def test_attn_mma(nh, nkv, hd, ps, lens, q_lens, window, nsplit):
    c = _paged_case(torch.bfloat16, nh, nkv, hd, ps, lens, q_lens, window, seed=15)
    out = _run_mma(c, nh, nkv, hd, ps, window, nsplit)
    assert_close(out, c["ref"], torch.bfloat16, "attn_mma")
    if nsplit in (2, 4, 8, 16):     # the same splits as one thread-block cluster, merged through shared memory
        out = _run_mma(c, nh, nkv, hd, ps, window, nsplit, cluster=True)
        assert_close(out, c["ref"], torch.bfloat16, "attn_mma as clusters")
        out = _run_mma(c, nh, nkv, hd, ps, window, nsplit, cluster=True, warps=8)
        assert_close(out, c["ref"], torch.bfloat16, "attn_mma as clusters of 8-warp CTAs")
    out = _run_mma(c, nh, nkv, hd, ps, window, nsplit, warps=8)
    assert_close(out, c["ref"], torch.bfloat16, "attn_mma with 8 warps")


DECODE_SHAPES = [
    # nh, nkv, hd, page, lens, window
    (12, 2, 128, 16, [700, 33, 1, 2100], None),      # group 6
    (8, 1, 64, 16, [130, 64, 65, 17, 1000], None),   # group 8: every MMA column used
    (3, 3, 128, 32, [257, 16, 15], None),            # group 1
    (14, 2, 64, 64, [300, 900], None),               # group 7, page 64
    (12, 2, 128, 16, [500, 77, 3000], 120),          # window
    (12, 2, 128, 16, [4700, 100], None),             # more tiles a split than the block table's shared-memory copy holds
]


@pytest.mark.parametrize("nsplit", [1, 2, 4, 8])
@pytest.mark.parametrize("nh,nkv,hd,ps,lens,window", DECODE_SHAPES)
def test_attn_decode(nh, nkv, hd, ps, lens, window, nsplit):
    from lite_lang_b200 import ops
    c = _paged_case(torch.bfloat16, nh, nkv, hd, ps, lens, [1] * len(lens), window, seed=27)
    d = dev()
    ctx = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=d)
    status = torch.zeros(1, dtype=torch.int32, device=d)
    # 4 or 8 warps a CTA, rings of 2 to 4 tiles a warp (0: the kernel's choice): more or fewer tiles than the ring holds
    for warps, depth in ((4, 0), (4, 2), (4, 4), (8, 0), (8, 3)):
        out = torch.full_like(c["q"], 3.0)
        ops.attn_decode(out, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], ctx, c["req_slot"], len(lens), nh, nkv,
                        hd, ps, window, hd ** -0.5, nsplit, status, warps=warps, depth=depth)
        assert status.item() == 0
        assert_close(out, c["ref"], torch.bfloat16, f"attn_decode with {warps} warps, rings of {depth}")


@pytest.mark.parametrize("nsplit,nouter,warps", [(8, 4, 8), (2, 7, 8), (4, 16, 8), (8, 2, 8)])
@pytest.mark.parametrize("nh,nkv,hd,ps,lens,window", [(12, 2, 128, 16, [9000, 33, 1, 2100], None),
                                                      (8, 1, 64, 32, [5000, 700], None),
                                                      (14, 2, 64, 16, [3000, 6100], 2500)])
def test_attn_decode_with_several_clusters_a_request(nh, nkv, hd, ps, lens, window, nsplit, nouter, warps):
    """Few requests with long contexts: `nouter` clusters a (entry, kv head) that meet through scratch memory (also
    requests so short that most clusters have no keys); twice, so that the counters must have come back to zero."""
    from lite_lang_b200 import ops
    c = _paged_case(torch.bfloat16, nh, nkv, hd, ps, lens, [1] * len(lens), window, seed=33)
    d = dev()
    ctx = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=d)
    status = torch.zeros(1, dtype=torch.int32, device=d)
    for _ in range(2):
        out = torch.full_like(c["q"], 3.0)
        ops.attn_decode(out, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], ctx, c["req_slot"], len(lens), nh, nkv,
                        hd, ps, window, hd ** -0.5, nsplit, status, warps=warps, depth=2, nouter=nouter)
        assert status.item() == 0
        assert_close(out, c["ref"], torch.bfloat16, f"attn_decode, {nouter} clusters of {nsplit}")


@pytest.mark.parametrize("nsplit", [1, 8])
@pytest.mark.parametrize("where", ["first", "page_edge", "last_of_page", "window_in", "window_out"])
def test_attn_decode_finds_one_far_key(where, nsplit):
    from lite_lang_b200 import ops
    nh, nkv, hd, ps, L, window = 12, 2, 128, 16, 1000, None
    if where == "first":
        peak = lambda l: 0
    elif where == "page_edge":
        peak = lambda l: 16 * 31
    elif where == "last_of_page":
        peak = lambda l: 16 * 31 + 15
    else:
        window = 300
        peak = (lambda l: l - 300) if where == "window_in" else (lambda l: l - 301)
    c = _paged_case(torch.bfloat16, nh, nkv, hd, ps, [L], [1], window, seed=28, peak=peak)
    ctx = torch.tensor([L - 1], dtype=torch.int32, device=dev())
    out = torch.full_like(c["q"], 3.0)
    ops.attn_decode(out, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], ctx, c["req_slot"], 1, nh, nkv, hd, ps,
                    window, hd ** -0.5, nsplit, None)
    assert_close(out, c["ref"], torch.bfloat16, where)
    assert (float(c["ref"].mean()) > 4.5) == (where != "window_out")


def test_attn_decode_padding_and_refusals():
    from lite_lang_b200 import ops
    c = _paged_case(torch.bfloat16, 8, 2, 64, 16, [50], [1], None, seed=29)
    d = dev()
    q = torch.cat([c["q"], c["q"], c["q"]])
    ctx = torch.tensor([49, 0, 0], dtype=torch.int32, device=d)
    req_slot = torch.tensor([int(c["req_slot"][0]), -1, -1], dtype=torch.int32, device=d)
    out = torch.full_like(q, 9.0)
    ops.attn_decode(out, q, q.stride(0), c["kc"], c["vc"], c["bt"], ctx, req_slot, 3, 8, 2, 64, 16, None, 64 ** -0.5, 4,
                    None)
    assert_close(out[:1], c["ref"], torch.bfloat16)
    assert float(out[1:].float().abs().max()) == 0.0
    with pytest.raises(ValueError, match="groups of at most 8"):
        ops.attn_decode(out, q, q.stride(0), c["kc"], c["vc"], c["bt"], ctx, req_slot, 3, 32, 2, 64, 16, None, 1.0, 1,
                        None)


PREFILL_SHAPES = [
    # nh, nkv, hd, page, lens, q_lens, window
    (12, 2, 128, 16, [300], [300], None),                       # a whole prompt, group 6
    (12, 2, 128, 16, [700, 33, 1, 129], [150, 33, 1, 2], None),   # portions behind a context, short entries
    (8, 2, 64, 16, [130, 64, 65, 17], [130, 1, 20, 17], None),
    (8, 2, 64, 32, [300, 90], [37, 90], None),
    (3, 1, 128, 64, [257], [100], None),
    (40, 2, 64, 16, [99, 50], [7, 3], None),                    # group 20
    (4, 4, 128, 16, [200, 77], [120, 1], 50),                   # window
    (8, 2, 64, 16, [400], [400], 33),
    (12, 2, 128, 16, [1500], [1500], None),                     # many stages, many row blocks
]


@pytest.mark.parametrize("nh,nkv,hd,ps,lens,q_lens,window", PREFILL_SHAPES)
def test_attn_prefill(nh, nkv, hd, ps, lens, q_lens, window):
    from lite_lang_b200 import ops
    c = _paged_case(torch.bfloat16, nh, nkv, hd, ps, lens, q_lens, window, seed=18)
    d = dev()
    group = nh // nkv
    cu = [0]
    for ql in q_lens:
        cu.append(cu[-1] + ql)
    cu_q = torch.tensor(cu, dtype=torch.int32, device=d)
    ctx = torch.tensor([l - ql for l, ql in zip(lens, q_lens)], dtype=torch.int32, device=d)
    blocks = sum((ql * group + 127) // 128 for ql in q_lens)
    out = torch.full_like(c["q"], 3.0)
    status = torch.zeros(1, dtype=torch.int32, device=d)
    ops.attn_prefill(out, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], cu_q, ctx, c["req_slot"], len(lens),
                     blocks, nh, nkv, hd, ps, window, hd ** -0.5, status)
    assert status.item() == 0
    assert_close(out, c["ref"], torch.bfloat16, "attn_prefill")


@pytest.mark.parametrize("where", ["first", "stage_edge", "last_of_stage", "window_in", "window_out"])
def test_attn_prefill_finds_one_far_key(where):
    from lite_lang_b200 import ops
    nh, nkv, hd, ps, L, window = 12, 2, 128, 16, 1000, None
    if where == "first":
        peak = lambda l: 0
    elif where == "stage_edge":
        peak = lambda l: 64 * 7
    elif where == "last_of_stage":
        peak = lambda l: 64 * 7 + 63
    else:
        window = 300
        peak = (lambda l: l - 300) if where == "window_in" else (lambda l: l - 301)
    c = _paged_case(torch.bfloat16, nh, nkv, hd, ps, [L], [40], window, seed=19, peak=peak)
    d = dev()
    cu_q = torch.tensor([0, 40], dtype=torch.int32, device=d)
    ctx = torch.tensor([L - 40], dtype=torch.int32, device=d)
    out = torch.full_like(c["q"], 3.0)
    ops.attn_prefill(out, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], cu_q, ctx, c["req_slot"], 1,
                     (40 * 6 + 127) // 128, nh, nkv, hd, ps, window, hd ** -0.5, None)
    assert_close(out, c["ref"], torch.bfloat16, where)
    assert (float(c["ref"][-1].mean()) > 4.5) == (where != "window_out")


def _run_prefill_tc(c, nh, nkv, hd, ps, lens, q_lens, window, status=None, nsplit=None):
    from lite_lang_b200 import ops
    d = dev()
    cu = [0]
    for ql in q_lens:
        cu.append(cu[-1] + ql)
    cu_q = torch.tensor(cu, dtype=torch.int32, device=d)
    ctx = torch.tensor([l - ql for l, ql in zip(lens, q_lens)], dtype=torch.int32, device=d)
    out = torch.full_like(c["q"], 3.0)
    ops.attn_prefill_tc(out, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], cu_q, ctx, c["req_slot"], len(lens),
                        ops.attn_prefill_tc_blocks(q_lens, nh // nkv), nh, nkv, hd, ps, window, hd ** -0.5, status,
                        nsplit)
    return out


@pytest.mark.parametrize("nh,nkv,hd,ps,lens,q_lens,window", PREFILL_SHAPES + [
    (14, 2, 64, 8, [90, 200], [90, 64], None),                  # group 7, pages of 8
    (2, 2, 128, 128, [600], [333], 100),                        # group 1: 128 tokens a CTA; pages larger than a block
])
def test_attn_prefill_tc(nh, nkv, hd, ps, lens, q_lens, window):
    c = _paged_case(torch.bfloat16, nh, nkv, hd, ps, lens, q_lens, window, seed=18)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    for nsplit in (1, None, 4, 8):      # unsplit, as the engine would, and with the keys split over 4 and 8 CTAs
        out = _run_prefill_tc(c, nh, nkv, hd, ps, lens, q_lens, window, status, nsplit)
        assert status.item() == 0
        assert_close(out, c["ref"], torch.bfloat16, f"attn_prefill_tc nsplit {nsplit}")


@pytest.mark.parametrize("where", ["first", "block_edge", "last_of_block", "window_in", "window_out"])
def test_attn_prefill_tc_finds_one_far_key(where):
    nh, nkv, hd, ps, L, window = 12, 2, 128, 16, 1000, None
    if where == "first":
        peak = lambda l: 0
    elif where == "block_edge":
        peak = lambda l: 64 * 7
    elif where == "last_of_block":
        peak = lambda l: 64 * 7 + 63
    else:
        window = 300
        peak = (lambda l: l - 300) if where == "window_in" else (lambda l: l - 301)
    c = _paged_case(torch.bfloat16, nh, nkv, hd, ps, [L], [40], window, seed=19, peak=peak)
    for nsplit in (1, 8):
        out = _run_prefill_tc(c, nh, nkv, hd, ps, [L], [40], window, nsplit=nsplit)
        assert_close(out, c["ref"], torch.bfloat16, where)
    assert (float(c["ref"][-1].mean()) > 4.5) == (where != "window_out")


@pytest.mark.parametrize("nsplit,cluster", [(1, False), (5, False), (8, True), (32, False)])
@pytest.mark.parametrize("where", ["first", "page_edge", "last_of_page", "window_in", "window_out"])
def test_attn_mma_finds_one_far_key(where, nsplit, cluster):
    nh, nkv, hd, ps, L, window = 12, 2, 128, 16, 1000, None
    if nsplit == 32:       # (the plan of one or two requests with very long contexts: 32 parts, 8 warps)
        L = 9000
    if where == "first":
        peak = lambda l: 0
    elif where == "page_edge":
        peak = lambda l: 16 * 31
    elif where == "last_of_page":
        peak = lambda l: 16 * 31 + 15
    else:
        window = 300
        peak = (lambda l: l - 300) if where == "window_in" else (lambda l: l - 301)
    c = _paged_case(torch.bfloat16, nh, nkv, hd, ps, [L], [1], window, seed=16, peak=peak)
    out = _run_mma(c, nh, nkv, hd, ps, window, nsplit, cluster, warps=8 if nsplit == 32 else 4)
    assert_close(out, c["ref"], torch.bfloat16, where)
    assert (float(c["ref"].mean()) > 4.5) == (where != "window_out")


def test_attn_mma_padding_entries_and_refusals():
    from lite_lang_b200 import ops
    c = _paged_case(torch.bfloat16, 8, 2, 64, 16, [50], [1], None, seed=17)
    d = dev()
    q = torch.cat([c["q"], c["q"], c["q"]])
    cu_q = torch.tensor([0, 1, 2, 3], dtype=torch.int32, device=d)
    ctx = torch.tensor([49, 0, 0], dtype=torch.int32, device=d)
    req_slot = torch.tensor([int(c["req_slot"][0]), -1, -1], dtype=torch.int32, device=d)
    out = torch.full_like(q, 9.0)
    scratch = torch.zeros(ops.attn_mma_scratch_floats(3, 2, 4, 64), device=d)
    counters = torch.zeros(6, dtype=torch.int32, device=d)
    ops.attn_mma(out, q, q.stride(0), c["kc"], c["vc"], c["bt"], cu_q, ctx, req_slot, 3, 3, 8, 2, 64, 16, None,
                 64 ** -0.5, 4, scratch, counters, None)
    assert_close(out[:1], c["ref"], torch.bfloat16)
    assert float(out[1:].float().abs().max()) == 0.0 and int(counters.abs().sum()) == 0
    assert not ops.attn_mma_supported(torch.float32, 64, 16, 512)
    assert not ops.attn_mma_supported(torch.bfloat16, 96, 16, 512)
    assert not ops.attn_mma_supported(torch.bfloat16, 64, 8, 512)
    with pytest.raises(ValueError, match="attn_mma takes"):
        ops.attn_mma(out, q, q.stride(0), c["kc"], c["vc"], c["bt"], cu_q, ctx, req_slot, 3, 3, 8, 2, 96, 16, None,
                     1.0, 1, None, None, None)


def _poison_what_no_query_may_see(c, ps, window):
    """Inf and NaN in every place of the pools that no query of the case may read: pages nobody owns (page 0
    among them: the kernels read it in place of a page that is not there), the unwritten ends of last pages,
    and pages that lie wholly before every query's window, which are also taken out of the block table, as
    the cache manager does.  That is what an earlier owner with broken weights may have left behind."""
    bt = c["bt"].cpu().clone()
    kc, vc = c["kc"].clone(), c["vc"].clone()
    num_pages = kc.shape[0]
    owned = set(int(x) for x in bt.flatten().tolist() if x >= 0)
    if 0 in owned:                                  # page 0 becomes nobody's
        spare = next(pg for pg in range(num_pages) if pg not in owned)
        kc[spare], vc[spare] = kc[0], vc[0]
        bt[bt == 0] = spare
        owned.discard(0)
        owned.add(spare)
    bad = torch.tensor([float("nan"), float("inf"), -float("inf")], device=kc.device).to(kc.dtype)

    def spoil(t):
        t.copy_(bad[torch.randint(0, 3, t.shape, device=t.device)])

    for pg in range(num_pages):
        if pg not in owned:
            spoil(kc[pg])
            spoil(vc[pg])
    for i, (l, ql) in enumerate(zip(c["lens"], c["q_lens"])):
        row = bt[int(c["req_slot"][i])]
        last = (l - 1) // ps
        if l % ps:
            spoil(kc[int(row[last]), :, l % ps:])
            spoil(vc[int(row[last]), :, l % ps:])
        if window is not None:
            first_needed = max(0, (l - ql) - window + 1)
            for lp in range(first_needed // ps):
                spoil(kc[int(row[lp])])
                spoil(vc[int(row[lp])])
                row[lp] = -1
    return dict(c, kc=kc, vc=vc, bt=bt.to(c["bt"].device))


@pytest.mark.parametrize("kernel", ["generic32", "generic", "mma", "mma_split", "decode", "decode_split", "prefill",
                                    "prefill_tc"])
@pytest.mark.parametrize("window", [None, 70])
def test_attention_kernels_are_blind_to_what_freed_pages_hold(kernel, window):
    """0 x NaN is NaN: a key that is masked must not enter the products with whatever its page holds."""
    from lite_lang_b200 import ops
    d = dev()
    dtype = torch.float32 if kernel == "generic32" else torch.bfloat16
    nh, nkv, hd, ps = 12, 2, 128, 16
    lens = [333, 90, 1, 203]                                  # no length is a multiple of the page size
    decode = kernel.startswith("decode") or kernel.startswith("mma")
    q_lens = [1, 1, 1, 1] if decode else [150, 90, 1, 2]
    c = _paged_case(dtype, nh, nkv, hd, ps, lens, q_lens, window, seed=41)
    c = _poison_what_no_query_may_see(c, ps, window)
    status = torch.zeros(1, dtype=torch.int32, device=d)
    out = torch.full_like(c["q"], 3.0)
    cu = [0]
    for ql in q_lens:
        cu.append(cu[-1] + ql)
    cu_q = torch.tensor(cu, dtype=torch.int32, device=d)
    ctx = torch.tensor([l - ql for l, ql in zip(lens, q_lens)], dtype=torch.int32, device=d)
    group = nh // nkv
    if kernel.startswith("generic"):
        ops.paged_attention_generic(out, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], c["token_req"],
                                    c["req_slot"], c["positions"], c["q"].shape[0], nh, nkv, hd, ps, window,
                                    hd ** -0.5, status)
    elif kernel.startswith("mma"):
        out = _run_mma(c, nh, nkv, hd, ps, window, 4 if kernel == "mma_split" else 1, cluster=kernel == "mma_split")
    elif kernel.startswith("decode"):
        ops.attn_decode(out, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], ctx, c["req_slot"], len(lens), nh,
                        nkv, hd, ps, window, hd ** -0.5, 4 if kernel == "decode_split" else 1, status)
    elif kernel == "prefill":
        blocks = sum((ql * group + 127) // 128 for ql in q_lens)
        ops.attn_prefill(out, c["q"], c["q"].stride(0), c["kc"], c["vc"], c["bt"], cu_q, ctx, c["req_slot"], len(lens),
                         blocks, nh, nkv, hd, ps, window, hd ** -0.5, status)
    else:
        for nsplit in (1, 4):
            out = _run_prefill_tc(c, nh, nkv, hd, ps, lens, q_lens, window, status, nsplit)
            assert torch.isfinite(out.float()).all(), nsplit
            assert_close(out, c["ref"], dtype, f"{kernel} nsplit {nsplit}")
    assert status.item() == 0
    assert torch.isfinite(out.float()).all()
    assert_close(out, c["ref"], dtype, kernel)


def test_attn_prefill_tc_reports_a_table_entry_outside_the_pool():
    """A key that a row sees and whose table entry names no page of the pool sets the status word (3) instead
    of being read from somewhere."""
    nh, nkv, hd, ps = 8, 2, 64, 16
    c = _paged_case(torch.bfloat16, nh, nkv, hd, ps, [200], [100], None, seed=42)
    for bad in (c["kc"].shape[0] + 5, -1):
        bt = c["bt"].clone()
        bt[int(c["req_slot"][0]), 3] = bad
        status = torch.zeros(1, dtype=torch.int32, device=dev())
        _run_prefill_tc(dict(c, bt=bt), nh, nkv, hd, ps, [200], [100], None, status, 1)
        assert status.item() == 3, bad


def test_padding_entries_write_zeros_and_read_nothing():
    from lite_lang_b200 import ops
    c = _paged_case(torch.float32, 4, 2, 32, 8, [20], [1], None, seed=8)
    q = torch.cat([c["q"], c["q"]])
    token_req = torch.tensor([0, 1], dtype=torch.int32, device=dev())
    req_slot = torch.tensor([int(c["req_slot"][0]), -1], dtype=torch.int32, device=dev())
    positions = torch.tensor([19, 0], dtype=torch.int32, device=dev())
    out = torch.full_like(q, 7.0)
    ops.paged_attention_generic(out, q, q.stride(0), c["kc"], c["vc"], c["bt"], token_req, req_slot, positions, 2,
                                4, 2, 32, 8, None, 32 ** -0.5, None)
    assert_close(out[:1], c["ref"], torch.float32)
    assert float(out[1].abs().max()) == 0.0


@pytest.mark.parametrize("vocab", [7, 1000, 151936, 50257])
def test_greedy_is_argmax_with_lowest_index_on_ties(vocab):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(4)
    logits = torch.randn(5, vocab, generator=g)
    logits[1, vocab // 2] = logits[1, vocab - 1] = 50.0        # a tie
    logits[2, 0] = 60.0
    logits[3, vocab - 1] = 60.0
    out = torch.zeros(5, dtype=torch.int32, device=dev())
    ops.sample(logits.to(dev()), out)
    assert out.cpu().tolist() == torch.argmax(logits, dim=-1).tolist()
    assert out[1].item() == vocab // 2


@pytest.mark.parametrize("vocab", [13, 2048, 151936])
def test_temperature_sampling_walks_the_cdf(vocab):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(9)
    rows = 40
    logits = 3 * torch.randn(rows, vocab, generator=g)
    temps = torch.tensor([0.7, 1.0, 0.3, 1.5] * (rows // 4))
    temps[5] = 0.0                                             # greedy row among sampled ones
    u = torch.rand(rows, generator=g)
    out = torch.zeros(rows, dtype=torch.int32, device=dev())
    ops.sample(logits.to(dev()), out, temps.to(dev()), u.to(dev()))
    got = out.cpu().tolist()
    for r in range(rows):
        if temps[r] == 0:
            assert got[r] == int(torch.argmax(logits[r]))
            continue
        p = P.temperature_probs(logits[r], float(temps[r]))
        cdf = torch.cumsum(p, 0)
        i = got[r]
        lo = float(cdf[i - 1]) if i > 0 else 0.0
        hi = float(cdf[i])
        # the token's CDF interval holds u, up to float32 rounding of the sums
        assert lo - 1e-4 <= float(u[r]) <= hi + 1e-4, (r, i, lo, float(u[r]), hi)
    # the distribution is right: many draws of one row
    row = torch.tensor([2.0, 1.0, 0.0, -1.0, 1.5]).repeat(4000, 1)
    uu = torch.rand(4000, generator=g)
    out = torch.zeros(4000, dtype=torch.int32, device=dev())
    ops.sample(row.to(dev()), out, torch.full((4000,), 0.8).to(dev()), uu.to(dev()))
    freq = torch.bincount(out.cpu().long(), minlength=5).double() / 4000
    assert float((freq - P.temperature_probs(row[0], 0.8)).abs().max()) < 0.03


@pytest.mark.parametrize("m,n,k", [(1, 48, 64), (8, 2048, 1536), (5, 1536, 8960), (13, 100, 96), (33, 331, 160),
                                   (64, 272, 1024), (2, 16, 32)])
def test_gemm_smallm(m, n, k):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(21)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    ref = P.linear(x.float(), w.float())
    for dt in (torch.bfloat16, torch.float32):
        out = torch.full((m, n), 7.0, dtype=dt, device=dev())
        ops.gemm_smallm(x.to(dev()), w.to(dev()), out)
        scale = float(ref.abs().max())
        err = float((out.float().cpu() - ref).abs().max()) / scale
        assert err <= (8e-3 if dt == torch.bfloat16 else 2e-5), (dt, err)
    # a view with a row stride (the q part of a fused projection)
    wide = torch.randn(m, k + 64, generator=g).to(torch.bfloat16).to(dev())
    out = torch.empty(m, n, dtype=torch.float32, device=dev())
    ops.gemm_smallm(wide[:, :k], w.to(dev()), out)
    ref2 = P.linear(wide[:, :k].float().cpu(), w.float())
    assert float((out.cpu() - ref2).abs().max()) / float(ref2.abs().max()) <= 2e-5


@pytest.mark.parametrize("m,inter,k", [(1, 128, 64), (8, 8960, 1536), (20, 203, 96), (64, 320, 256)])
def test_gemm_smallm_gated_equals_product_then_activation(m, inter, k):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(22)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev())
    w = (2 * torch.randn(2 * inter, k, generator=g) / k ** 0.5).to(torch.bfloat16).to(dev())
    fused = ops.gemm_smallm(x, w, torch.empty(m, inter, dtype=torch.bfloat16, device=dev()), gated=True)
    gu = torch.mm(x, w.t())
    unfused = torch.empty(m, inter, dtype=torch.bfloat16, device=dev())
    ops.silu_mul(unfused, gu)
    ref = P.silu_and_mul(P.linear(x.float().cpu(), w[:inter].float().cpu()), P.linear(x.float().cpu(), w[inter:].float().cpu()))
    assert_close(fused, ref, torch.bfloat16, "gated")
    # the same roundings as the unfused path: equal up to the order of the float32 sums
    assert float((fused.float() - unfused.float()).abs().max()) <= 2e-2 * float(ref.abs().max())


@pytest.mark.parametrize("mode,m,n,k", [(2, 1, 48, 256), (2, 8, 2048, 1536), (2, 5, 1536, 8960), (2, 13, 100, 512),
                                        (0, 8, 9000, 1536), (0, 3, 331, 128), (0, 32, 151936, 256), (2, 32, 272, 1024),
                                        (0, 16, 64, 384), (2, 16, 17, 768), (2, 33, 1536, 1536), (2, 64, 2048, 512),
                                        (2, 47, 100, 256)])
def test_gemm_stream(mode, m, n, k):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(24)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    for dt in (torch.bfloat16, torch.float32):
        if m > 32 and dt == torch.float32:       # (33 to 64 tokens: two blocks of tokens, to bfloat16 only)
            continue
        out = torch.full((m, n), 7.0, dtype=dt, device=dev())
        for _ in range(2):
            ops.gemm_stream(x.to(dev()), w.to(dev()), out, mode, status)
        err = float((out.double().cpu() - ref).abs().max()) / float(ref.abs().max())
        assert err <= (8e-3 if dt == torch.bfloat16 else 2e-5), (dt, err)
    assert status.item() == 0


@pytest.mark.parametrize("mode,m,n,k,parts", [(2, 8, 1536, 8960, 3), (0, 5, 1536, 8960, 12), (2, 32, 100, 1024, 2),
                                              (2, 1, 1536, 8960, 35)])
def test_gemm_stream_split_over_k_and_summed_by_the_norm(mode, m, n, k, parts):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(26)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    out = torch.full((parts, m, n), float("nan"), dtype=torch.float32, device=dev())
    ops.gemm_stream(x.to(dev()), w.to(dev()), out, mode)
    total = out.double().sum(0).cpu()
    assert float((total - ref).abs().max()) / float(ref.abs().max()) <= 2e-5
    # the fused residual-and-norm kernel takes the partial sums as its delta
    res = torch.randn(m, n, generator=g).to(torch.bfloat16)
    wn = 1 + 0.1 * torch.randn(n, generator=g)
    res_dev = res.to(dev()).clone()
    y = torch.empty(m, n, dtype=torch.bfloat16, device=dev())
    ops.add_rmsnorm(y, res_dev, out, wn.to(dev()), 1e-6)
    s_ref = (res.float() + ref.float().to(torch.bfloat16).float()).to(torch.bfloat16)
    assert float((res_dev.float().cpu() - s_ref.float()).abs().max()) <= 2 ** -6 * float(s_ref.float().abs().max())
    assert_close(y, P.rms_norm(s_ref.float(), wn, 1e-6), torch.bfloat16, "norm of residual + partial sums")
    assert ops.stream_ksplit(1536, 8960, 2, dev()) == 3 and ops.stream_ksplit(2048, 1536, 2, dev()) == 1


@pytest.mark.parametrize("m,hidden,k,inter", [(8, 1536, 1536, 8960), (1, 256, 512, 96), (13, 768, 256, 203),
                                              (32, 2048, 2048, 320), (16, 3584, 3584, 1184), (40, 1536, 1536, 8960),
                                              (64, 1536, 1024, 11008), (33, 768, 512, 640), (24, 1536, 1536, 640), (17, 256, 256, 96)])
def test_norm_split_between_the_product_before_and_the_gated_product_after(m, hidden, k, inter):
    """o projection -> residual sum -> RMS norm -> gated feed-forward product as two kernels: against the plain
    formulas, and the residual rows bit for bit against the three separate kernels."""
    from lite_lang_b200 import ops
    d = dev()
    g = torch.Generator().manual_seed(61)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(d)
    w1 = (torch.randn(hidden, k, generator=g) / k ** 0.5).to(torch.bfloat16).to(d)
    res0 = torch.randn(m, hidden, generator=g).to(torch.bfloat16).to(d)
    wn = (1 + 0.2 * torch.randn(hidden, generator=g)).to(d)
    w2 = (2 * torch.randn(2 * inter, hidden, generator=g) / hidden ** 0.5).to(torch.bfloat16).to(d)
    eps = 1e-5
    status = torch.zeros(1, dtype=torch.int32, device=d)
    # the separate kernels
    res_a = res0.clone()
    delta = ops.gemm_stream(x, w1, torch.empty(m, hidden, dtype=torch.bfloat16, device=d), 2, status)
    xa = torch.empty_like(res_a)
    ops.add_rmsnorm(xa, res_a, delta, wn, eps)
    act_a = ops.gated_linear(xa, w2)      # (the streaming kernel, or from 17 tokens on the tcgen05 one)
    # the two kernels with the norm split between them
    res_b = res0.clone()
    u, sumsq = ops.gemm_stream_into_norm(x, w1, res_b, wn, status)
    act_b = ops.gemm_stream_gated_scaled(u, w2, sumsq, eps, status)
    assert status.item() == 0
    assert torch.equal(res_a, res_b), "the residual rows differ from the separate kernels'"
    total = sumsq[:, :m].sum(0).double().cpu()
    want = (res_b.double() ** 2).sum(1).cpu()
    assert float(((total - want).abs() / want).max()) <= 1e-5
    assert float((u.float() - res_b.float() * wn).abs().max()) <= 2 ** -8 * float((res_b.float() * wn).abs().max())
    # the plain formulas on the rounded residual rows
    h = res_b.float().cpu()
    xn = P.rms_norm(h, wn.cpu(), eps)
    ref = P.silu_and_mul(P.linear(xn, w2[:inter].float().cpu()), P.linear(xn, w2[inter:].float().cpu()))
    assert_close(act_b, ref, torch.bfloat16, "gated product after the split norm")
    assert_close(act_a, ref, torch.bfloat16, "gated product after the norm kernel")
    assert float((act_a.float() - act_b.float()).abs().max()) <= 2e-2 * float(ref.abs().max())


@pytest.mark.parametrize("m,inter,k", [(1, 128, 128), (8, 8960, 1536), (20, 203, 384), (32, 320, 256)])
def test_gemm_stream_gated(m, inter, k):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(25)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev())
    w = (2 * torch.randn(2 * inter, k, generator=g) / k ** 0.5).to(torch.bfloat16).to(dev())
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    fused = ops.gemm_stream(x, w, torch.empty(m, inter, dtype=torch.bfloat16, device=dev()), 1, status)
    gu = torch.mm(x, w.t())
    unfused = torch.empty(m, inter, dtype=torch.bfloat16, device=dev())
    ops.silu_mul(unfused, gu)
    ref = P.silu_and_mul(P.linear(x.float().cpu(), w[:inter].float().cpu()), P.linear(x.float().cpu(), w[inter:].float().cpu()))
    assert_close(fused, ref, torch.bfloat16, "gated")
    assert float((fused.float() - unfused.float()).abs().max()) <= 2e-2 * float(ref.abs().max())
    assert status.item() == 0


@pytest.mark.parametrize("m,n,k", [(64, 128, 64), (33, 256, 128), (128, 128, 192), (7, 100, 64), (100, 331, 448)])
def test_gemm_tc_is_exact_on_small_integers(m, n, k):
    """Integer operands whose products and sums are exact in float32: a wrong swizzle, descriptor or
    tensor-memory lane shows as a wrong integer, not as rounding."""
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(40)
    x = torch.randint(-3, 4, (m, k), generator=g).to(torch.bfloat16)
    w = torch.randint(-3, 4, (n, k), generator=g).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    out = torch.full((m, n), 7.0, dtype=torch.float32, device=dev())
    for _ in range(2):
        ops.gemm_tc(x.to(dev()), w.to(dev()), out, status=status)
    assert status.item() == 0
    assert torch.equal(out.double().cpu(), ref)


@pytest.mark.parametrize("m,n,k", [(64, 1536, 1536), (48, 2048, 1536), (128, 1000, 8960), (33, 151936 // 8, 1536)])
def test_gemm_tc(m, n, k):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(41)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    for dt in (torch.bfloat16, torch.float32):
        out = torch.full((m, n), 7.0, dtype=dt, device=dev())
        for _ in range(2):
            ops.gemm_tc(x.to(dev()), w.to(dev()), out, status=status)
        err = float((out.double().cpu() - ref).abs().max()) / float(ref.abs().max())
        assert err <= (8e-3 if dt == torch.bfloat16 else 2e-5), (dt, err)
    assert status.item() == 0


@pytest.mark.parametrize("m,n,k,parts", [(64, 1536, 8960, 12), (40, 1536, 1536, 6), (128, 200, 1024, 4)])
def test_gemm_tc_split_over_k(m, n, k, parts):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(42)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    out = torch.full((parts, m, n), float("nan"), dtype=torch.float32, device=dev())
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.gemm_tc(x.to(dev()), w.to(dev()), out, status=status)
    assert status.item() == 0
    total = out.double().sum(0).cpu()
    assert float((total - ref).abs().max()) / float(ref.abs().max()) <= 2e-5
    assert ops.tc_ksplit(1536, 8960, dev()) >= 2 and ops.tc_ksplit(17920, 1536, dev()) == 1


@pytest.mark.parametrize("m,inter,k", [(64, 8960, 1536), (33, 203, 384), (128, 320, 256), (100, 1024, 128)])
def test_gemm_tc_gated(m, inter, k):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(43)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev())
    w = (2 * torch.randn(2 * inter, k, generator=g) / k ** 0.5).to(torch.bfloat16).to(dev())
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    fused = ops.gemm_tc(x, w, torch.empty(m, inter, dtype=torch.bfloat16, device=dev()), gated=True, status=status)
    ref = P.silu_and_mul(P.linear(x.float().cpu(), w[:inter].float().cpu()), P.linear(x.float().cpu(), w[inter:].float().cpu()))
    assert_close(fused, ref, torch.bfloat16, "gated")
    assert status.item() == 0


def test_gemm_tc_refuses_what_it_cannot_do():
    from lite_lang_b200 import ops
    x = torch.zeros(129, 64, dtype=torch.bfloat16, device=dev())
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device=dev())
    with pytest.raises((RuntimeError, ValueError)):
        ops.gemm_tc(x, w, torch.empty(129, 128, dtype=torch.bfloat16, device=dev()))
    with pytest.raises((RuntimeError, ValueError)):
        ops.gemm_tc(x[:8, :32], w[:, :32].contiguous(), torch.empty(8, 128, dtype=torch.bfloat16, device=dev()))


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (512, 512, 448), (300, 331, 200), (1, 40, 8), (700, 1100, 1096)])
def test_gemm_pair_is_exact_on_small_integers(m, n, k):
    """The two-SM tcgen05 product on integer operands whose sums are exact in float32 and in bfloat16
    (|sum| <= 256): a wrong half of the pair, descriptor, swizzle or tensor-memory lane is a wrong integer."""
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(44)
    x = torch.randint(-1, 2, (m, k), generator=g).to(torch.bfloat16)
    w = torch.randint(-1, 2, (n, k), generator=g).to(torch.bfloat16)
    w[:, k // 4:] *= (torch.rand(n, k - k // 4, generator=g) < 128.0 / k).to(torch.bfloat16)   # keep |sum| small
    ref = x.double() @ w.double().t()
    assert float(ref.abs().max()) <= 256
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    out = torch.full((m + 1, n + 8), 7.0, dtype=torch.bfloat16, device=dev())
    for _ in range(2):
        ops.gemm_pair(x.to(dev()), w.to(dev()), out[:m, :n], status=status)
    assert status.item() == 0
    assert torch.equal(out[:m, :n].double().cpu(), ref)
    assert bool((out[m:] == 7).all()) and bool((out[:, n:] == 7).all())     # nothing written outside


@pytest.mark.parametrize("m,inter,k", [(2048, 8960, 1536), (512, 203, 384), (777, 1000, 264), (256, 128, 64)])
def test_gemm_pair_gated(m, inter, k):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(45)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev())
    w = (2 * torch.randn(2 * inter, k, generator=g) / k ** 0.5).to(torch.bfloat16).to(dev())
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    fused = torch.full((m, inter), 7.0, dtype=torch.bfloat16, device=dev())
    for _ in range(2):
        ops.gemm_pair(x, w, fused, gated=True, status=status)
    assert status.item() == 0
    rows = torch.arange(0, m, max(1, m // 97))          # a sample of rows keeps the float64 reference quick
    xs = x[rows].double().cpu()
    gate = (xs @ w[:inter].double().cpu().t()).to(torch.bfloat16).double()
    up = (xs @ w[inter:].double().cpu().t()).to(torch.bfloat16).double()
    ref = gate / (1 + torch.exp(-gate)) * up
    err = float((fused[rows].double().cpu() - ref).abs().max()) / float(ref.abs().max())
    assert err <= 1.5e-2, err
    # and against the unfused path it replaces, everywhere
    unfused = torch.empty(m, inter, dtype=torch.bfloat16, device=dev())
    ops.silu_mul(unfused, torch.mm(x, w.t()))
    assert float((fused.float() - unfused.float()).abs().max()) <= 2e-2 * float(ref.abs().max())


def test_gemm_pair_refuses_what_it_cannot_do():
    from lite_lang_b200 import ops
    x = torch.zeros(256, 68, dtype=torch.bfloat16, device=dev())
    w = torch.zeros(128, 68, dtype=torch.bfloat16, device=dev())
    with pytest.raises((RuntimeError, ValueError)):
        ops.gemm_pair(x, w, torch.empty(256, 128, dtype=torch.bfloat16, device=dev()))      # K % 8
    with pytest.raises((RuntimeError, ValueError)):
        ops.gemm_pair(x[:, :64], w[:, :64].contiguous(), torch.empty(256, 128, dtype=torch.float32, device=dev()))


def _assert_qkv_equals_the_plain_formulas(x, w, bias, pos, slots, q, kc, vc, nh, nkv, hd, ps, theta):
    """q, and the cache rows of the tokens that have a slot, against projection with bias (P.linear) and
    half-split rotation of q and k (P.rope_tables, P.apply_rope) in float32."""
    m = x.shape[0]
    qkv = P.linear(x.float().cpu(), w.float().cpu(), None if bias is None else bias.float().cpu())
    cos, sin = P.rope_tables(hd, theta, pos.cpu())
    q_ref = P.apply_rope(qkv[:, :nh * hd].reshape(m, nh, hd), cos, sin).reshape(m, nh * hd)
    k_ref = P.apply_rope(qkv[:, nh * hd:(nh + nkv) * hd].reshape(m, nkv, hd), cos, sin)
    v_ref = qkv[:, (nh + nkv) * hd:].reshape(m, nkv, hd)
    scale = float(qkv.abs().max())
    assert float((q.float().cpu() - q_ref).abs().max()) / scale <= tol(torch.bfloat16), "q against the plain formulas"
    if kc is None:
        return
    sl = slots.cpu().long()
    has = sl >= 0
    k_got = kc.float().cpu()[sl[has] // ps, :, sl[has] % ps]          # [tokens with a slot, nkv, hd]
    v_got = vc.float().cpu()[sl[has] // ps, :, sl[has] % ps]
    assert float((k_got - k_ref[has]).abs().max()) / scale <= tol(torch.bfloat16), "cached keys against the plain formulas"
    assert float((v_got - v_ref[has]).abs().max()) / scale <= tol(torch.bfloat16), "cached values against the plain formulas"


@pytest.mark.parametrize("m,hidden,nh,nkv,hd,ps", [(8, 1536, 12, 2, 128, 16), (1, 256, 3, 1, 64, 32), (19, 512, 4, 4, 32, 16),
                                                   (32, 768, 6, 2, 128, 64), (50, 1536, 12, 2, 128, 16), (64, 512, 4, 2, 64, 16),
                                                   (33, 256, 2, 2, 128, 32)])
def test_gemm_stream_qkv_rope_equals_the_plain_formulas_and_the_three_kernels_it_replaces(m, hidden, nh, nkv, hd, ps):
    from lite_lang_b200 import ops
    from lite_lang_b200.parts.rope import rope_table
    g = torch.Generator().manual_seed(30)
    d = dev()
    width = (nh + 2 * nkv) * hd
    x = torch.randn(m, hidden, generator=g).to(torch.bfloat16).to(d)
    w = (torch.randn(width, hidden, generator=g) / hidden ** 0.5).to(torch.bfloat16).to(d)
    bias = (0.5 * torch.randn(width, generator=g)).to(d)
    max_pos, num_pages = 500, 12
    pos = torch.randint(0, max_pos, (m,), generator=g, dtype=torch.int32).to(d)
    slots = torch.randperm(num_pages * ps, generator=g)[:m].to(torch.int32)
    if m > 2:
        slots[2] = -1
    slots = slots.to(d)
    table = rope_table(hd, 10000.0, max_pos).to(d)
    status = torch.zeros(1, dtype=torch.int32, device=d)
    # the unfused path: library product, then bias + rotation + store
    ref_qkv = torch.mm(x, w.t())
    kc_ref = torch.zeros(num_pages, nkv, ps, hd, dtype=torch.bfloat16, device=d)
    vc_ref = torch.zeros_like(kc_ref)
    ops.bias_rope_store(ref_qkv, bias, pos, table, nh, nkv, hd, slots, kc_ref, vc_ref, ps, status)
    # fused
    q = torch.full((m, nh * hd), 7.0, dtype=torch.bfloat16, device=d)
    kc, vc = torch.zeros_like(kc_ref), torch.zeros_like(kc_ref)
    ops.gemm_stream_qkv_rope(q, x, w, bias, pos, table, nh, nkv, hd, slots, kc, vc, ps, status)
    assert status.item() == 0
    scale = float(ref_qkv.float().abs().max())
    for got, want, what in ((q, ref_qkv[:, :nh * hd], "q"), (kc, kc_ref, "k cache"), (vc, vc_ref, "v cache")):
        err = float((got.float() - want.float()).abs().max()) / scale
        assert err <= 1.6e-2, (what, err)       # same roundings; only the order of the float32 sums differs
    assert float((kc.float().abs().sum(dim=(1, 3)) > 0).sum()) == float((kc_ref.float().abs().sum(dim=(1, 3)) > 0).sum())
    _assert_qkv_equals_the_plain_formulas(x, w, bias, pos, slots, q, kc, vc, nh, nkv, hd, ps, 10000.0)


@pytest.mark.parametrize("m,hidden,nh,nkv,hd,ps", [(2048, 1536, 12, 2, 128, 16), (300, 264, 3, 1, 64, 32),
                                                   (257, 512, 5, 5, 64, 16), (520, 328, 2, 1, 256, 64), (1, 64, 1, 1, 128, 16)])
def test_gemm_pair_qkv_rope_equals_the_plain_formulas_and_the_two_kernels_it_replaces(m, hidden, nh, nkv, hd, ps):
    from lite_lang_b200 import ops
    from lite_lang_b200.parts.rope import rope_table
    g = torch.Generator().manual_seed(31)
    d = dev()
    width = (nh + 2 * nkv) * hd
    x = torch.randn(m, hidden, generator=g).to(torch.bfloat16).to(d)
    w = (torch.randn(width, hidden, generator=g) / hidden ** 0.5).to(torch.bfloat16).to(d)
    bias = (0.5 * torch.randn(width, generator=g)).to(d)
    max_pos = 3000
    num_pages = (m + ps - 1) // ps + 3
    pos = torch.randint(0, max_pos, (m,), generator=g, dtype=torch.int32).to(d)
    slots = torch.randperm(num_pages * ps, generator=g)[:m].to(torch.int32)
    if m > 2:
        slots[2] = -1
    slots = slots.to(d)
    table = rope_table(hd, 10000.0, max_pos).to(d)
    status = torch.zeros(1, dtype=torch.int32, device=d)
    ref_qkv = torch.mm(x, w.t())
    kc_ref = torch.zeros(num_pages, nkv, ps, hd, dtype=torch.bfloat16, device=d)
    vc_ref = torch.zeros_like(kc_ref)
    ops.bias_rope_store(ref_qkv, bias, pos, table, nh, nkv, hd, slots, kc_ref, vc_ref, ps, status)
    q = torch.full((m + 1, nh * hd + 8), 7.0, dtype=torch.bfloat16, device=d)
    kc, vc = torch.zeros_like(kc_ref), torch.zeros_like(kc_ref)
    for _ in range(2):
        ops.gemm_pair_qkv_rope(q[:m, :nh * hd], x, w, bias, pos, table, nh, nkv, hd, slots, kc, vc, ps, status)
    assert status.item() == 0
    scale = float(ref_qkv.float().abs().max())
    for got, want, what in ((q[:m, :nh * hd], ref_qkv[:, :nh * hd], "q"), (kc, kc_ref, "k cache"), (vc, vc_ref, "v cache")):
        err = float((got.float() - want.float()).abs().max()) / scale
        assert err <= 1.6e-2, (what, err)       # same roundings; only the order of the float32 sums differs
    assert bool((q[m:] == 7).all()) and bool((q[:, nh * hd:] == 7).all())
    written = lambda c: c.float().abs().sum(dim=(1, 3)) > 0
    assert bool((written(kc) == written(kc_ref)).all()) and bool((written(vc) == written(vc_ref)).all())
    _assert_qkv_equals_the_plain_formulas(x, w, bias, pos, slots, q[:m, :nh * hd], kc, vc, nh, nkv, hd, ps, 10000.0)
    # no bias, no cache write: q only
    q2 = torch.empty(m, nh * hd, dtype=torch.bfloat16, device=d)
    ops.gemm_pair_qkv_rope(q2, x, w, None, pos, table, nh, nkv, hd, None, None, None, ps, status)
    ref2 = torch.mm(x, w.t())
    ops.bias_rope_store(ref2, None, pos, table, nh, nkv, hd, None, None, None, ps, status)
    assert float((q2.float() - ref2[:, :nh * hd].float()).abs().max()) / scale <= 1.6e-2
    _assert_qkv_equals_the_plain_formulas(x, w, None, pos, None, q2, None, None, nh, nkv, hd, ps, 10000.0)
    # a position outside the table is reported
    bad = pos.clone()
    bad[0] = max_pos
    ops.gemm_pair_qkv_rope(q2, x, w, None, bad, table, nh, nkv, hd, None, None, None, ps, status)
    assert status.item() == 4


def test_linear_picks_the_library_for_other_shapes():
    from lite_lang_b200 import ops
    ops.configure_matmul_precision()
    g = torch.Generator().manual_seed(23)
    for m, n, k, dt in [(65, 40, 64, torch.bfloat16), (4, 40, 50, torch.bfloat16), (4, 40, 64, torch.float32)]:
        x = torch.randn(m, k, generator=g).to(dt).to(dev())
        w = torch.randn(n, k, generator=g).to(dt).to(dev())
        assert not ops.smallm_preferred(x, w)
        y = ops.linear(x, w)
        assert_close(y, P.linear(x.float().cpu(), w.float().cpu()), dt if dt == torch.bfloat16 else torch.float32)
    x = torch.randn(3, 64, generator=g).to(torch.bfloat16).to(dev())
    w = torch.randn(40, 64, generator=g).to(torch.bfloat16).to(dev())
    y = ops.linear(x, w, out_dtype=torch.float32)
    assert y.dtype == torch.float32
    assert_close(y, P.linear(x.float().cpu(), w.float().cpu()), torch.float32, "float32 logits from bfloat16 operands")


def test_kernels_refuse_what_they_do_not_take():
    from lite_lang_b200 import ops
    x = torch.zeros(2, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.rmsnorm(torch.empty_like(x), x, torch.ones(8), 1e-6)       # CPU tensors: no fallback
    d = dev()
    with pytest.raises(TypeError):
        ops.rmsnorm(torch.empty(2, 8, dtype=torch.float16, device=d), torch.zeros(2, 8, dtype=torch.float16, device=d),
                    torch.ones(8, device=d), 1e-6)
    with pytest.raises(ValueError, match="head_dim"):
        c = _paged_case(torch.float32, 2, 1, 32, 8, [9], [1], None, seed=1)
        ops.paged_attention_generic(torch.empty(1, 2 * 320, device=d), c["q"], 640, c["kc"], c["vc"], c["bt"],
                                    c["token_req"], c["req_slot"], c["positions"], 1, 2, 1, 320, 8, None, 1.0, None)
