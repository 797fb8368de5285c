"""Typed Python entry points of the hand-written CUDA kernels.

Every function takes torch CUDA tensors, checks what the kernel assumes
(device, dtype, contiguity, sizes) and launches on torch's current stream.
There is no CPU or library fallback: a tensor that is not on a CUDA device, or
a missing kernel library, raises.

Matrix products are the exception: like the reference, which calls cuBLAS
through ``torch.mm`` / ``torch.addmm`` (``litelang/models/qwen2/layer/
transformer_layer.py:79-109,193``), ``linear`` is a library product.  On the
float32 path TF32 is switched off so that it is a true 32-bit product.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from .csrc.build import load_library

_DT = {torch.float32: 0, torch.bfloat16: 1}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}") from None


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream's handle.  (``torch.cuda.current_stream()`` builds a Python object through
    several layers, 15 us a call, with well over a hundred launches in a step that is not captured.)"""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("lite_lang_b200 kernels run on CUDA tensors only; there is no CPU path")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _i32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None:
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")


def _f32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None:
        _need(t.dtype == torch.float32 and t.is_contiguous(), f"{name} must be a contiguous float32 tensor")


def core():
    return load_library("core")


def configure_matmul_precision() -> None:
    """True float32 products (no TF32) and float32 accumulation for bfloat16 ones."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    try:
        torch.set_float32_matmul_precision("highest")
    except Exception:  # pragma: no cover
        pass


# --------------------------------------------------------------------------
def embed_gather(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, status: Optional[torch.Tensor]) -> None:
    _need_cuda(out, table, ids)
    _i32(ids, "ids")
    _need(out.dtype == table.dtype and out.is_contiguous() and table.is_contiguous(), "embed: dtype/contiguity")
    n, hidden = ids.numel(), table.shape[1]
    _need(out.shape[0] >= n and out.shape[1] == hidden, "embed: out has the wrong shape")
    core().call("ll_embed_gather", c_int(_dtype_code(out)), _ptr(out), _ptr(table), _ptr(ids), c_int(n),
                c_int(hidden), c_int(table.shape[0]), _ptr(status), _stream())


def feed_tokens(ids: torch.Tensor, feed: torch.Tensor, results: torch.Tensor) -> None:
    """ids[i] = results[feed[i]] where feed[i] >= 0: token ids sampled by the step before, taken on the device."""
    _need_cuda(ids, feed, results)
    for t, nm in ((ids, "ids"), (feed, "feed"), (results, "results")):
        _i32(t, nm)
    _need(feed.numel() >= ids.numel(), "feed_tokens: one feed index per token id")
    core().call("ll_feed_tokens", _ptr(ids), _ptr(feed), _ptr(results), c_int(ids.numel()), c_int(results.numel()),
                _stream())


def rmsnorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    _need_cuda(out, x, weight)
    _f32(weight, "norm weight")
    _need(x.dim() == 2 and out.shape == x.shape and out.dtype == x.dtype, "rmsnorm: shapes")
    _need(x.stride(1) == 1 and out.stride(1) == 1, "rmsnorm: rows must be contiguous")
    _need(weight.numel() == x.shape[1], "rmsnorm: weight size")
    core().call("ll_rmsnorm", c_int(_dtype_code(x)), _ptr(out), _ptr(x), _ptr(weight), c_float(eps),
                c_int(x.shape[0]), c_int(x.shape[1]), c_long(x.stride(0)), c_long(out.stride(0)), _stream())


def add_rmsnorm(out: torch.Tensor, residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None, write_residual: bool = True) -> None:
    """out[i] = norm(residual[r] + delta[r]); r = rows[i] if rows is given, else i.

    Without ``rows`` the rounded sum is written back into ``residual``.
    """
    _need_cuda(out, residual, delta, weight, rows)
    _f32(weight, "norm weight")
    _i32(rows, "rows")
    hidden = residual.shape[1]
    _need(residual.is_contiguous() and out.is_contiguous() and out.dtype == residual.dtype, "add_rmsnorm: layout")
    if delta is not None and delta.dim() == 2:
        _need(delta.is_contiguous() and delta.dtype == residual.dtype and delta.shape[1] == hidden,
              "add_rmsnorm: delta layout")
    n_out = rows.numel() if rows is not None else residual.shape[0]
    _need(out.shape[0] >= n_out and out.shape[1] == hidden, "add_rmsnorm: out shape")
    wr = 1 if (write_residual and rows is None and delta is not None) else 0
    partial, parts, part_stride = None, 0, 0
    if delta is not None and delta.dim() == 3:      # float32 partial sums [parts, tokens, hidden]
        _need(delta.dtype == torch.float32 and delta.is_contiguous() and delta.shape[2] == hidden,
              "add_rmsnorm: partial sums must be contiguous float32 [parts, tokens, hidden]")
        partial, parts, part_stride, delta = delta, delta.shape[0], delta.shape[1] * hidden, None
    core().call("ll_add_rmsnorm", c_int(_dtype_code(residual)), _ptr(out), _ptr(residual), _ptr(delta),
                _ptr(partial), c_int(parts), c_long(part_stride), _ptr(weight), c_float(eps), c_int(n_out),
                c_int(hidden), _ptr(rows), c_int(wr), _stream())


def bias_rope_store(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: Optional[torch.Tensor],
                    cos_sin: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                    slot_map: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                    v_cache: Optional[torch.Tensor], page_size: int, status: Optional[torch.Tensor],
                    num_tokens: Optional[int] = None) -> None:
    """Bias, half-split rotation of q and k, and the store of k and v into a cache plane.

    Each of the three is skipped when its argument is None.  ``cos_sin`` is the
    float32 table [max_positions, rot_dim] (cos half, then sin half).
    """
    _need_cuda(qkv, bias, positions, cos_sin, slot_map, k_cache, v_cache)
    _f32(bias, "bias")
    _f32(cos_sin, "cos_sin")
    _i32(positions, "positions")
    _i32(slot_map, "slot_map")
    width = (num_heads + 2 * num_kv_heads) * head_dim
    _need(qkv.dim() == 2 and qkv.shape[1] == width and qkv.stride(1) == 1, "qkv must be [tokens, (nh+2nkv)*hd]")
    n = qkv.shape[0] if num_tokens is None else num_tokens
    if bias is not None:
        _need(bias.numel() == width, "bias size")
    rot_dim, max_pos = 0, 0
    if cos_sin is not None:
        _need(positions is not None, "rotation needs positions")
        max_pos, rot_dim = cos_sin.shape
    num_slots = 0
    if slot_map is not None:
        _need(k_cache is not None and v_cache is not None, "store needs the cache plane")
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype, "cache dtype differs from activations")
        _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
        _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane shape")
        num_slots = k_cache.shape[0] * page_size
    core().call("ll_bias_rope_store", c_int(_dtype_code(qkv)), _ptr(qkv), c_long(qkv.stride(0)), _ptr(bias),
                _ptr(positions), _ptr(cos_sin), c_int(max_pos), c_int(rot_dim), c_int(num_heads),
                c_int(num_kv_heads), c_int(head_dim), _ptr(slot_map), _ptr(k_cache), _ptr(v_cache),
                c_int(page_size), c_long(num_slots), c_int(n), _ptr(status), _stream())


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor) -> None:
    _need_cuda(out, gate_up)
    _need(gate_up.is_contiguous() and out.is_contiguous() and out.dtype == gate_up.dtype, "silu_mul: layout")
    n, two_i = gate_up.shape
    _need(two_i % 2 == 0 and out.shape[0] == n and out.shape[1] == two_i // 2, "silu_mul: shapes")
    core().call("ll_silu_mul", c_int(_dtype_code(out)), _ptr(out), _ptr(gate_up), c_int(n), c_int(two_i // 2),
                _stream())


def paged_attention_generic(out: torch.Tensor, q: torch.Tensor, q_stride: int, k_cache: torch.Tensor,
                            v_cache: torch.Tensor, block_table: torch.Tensor, token_req: torch.Tensor,
                            req_slot: torch.Tensor, positions: torch.Tensor, num_tokens: int, num_heads: int,
                            num_kv_heads: int, head_dim: int, page_size: int, window: Optional[int], scale: float,
                            status: Optional[torch.Tensor]) -> None:
    """Attention of every new token over its request's cached keys (any sizes, both dtypes).

    ``q`` points at the first query head of the first token; head h of token t
    is at ``q + t*q_stride + h*head_dim`` (elements).
    """
    _need_cuda(out, q, k_cache, v_cache, block_table, token_req, req_slot, positions)
    for t, nm in ((block_table, "block_table"), (token_req, "token_req"), (req_slot, "req_slot"),
                  (positions, "positions")):
        _i32(t, nm)
    _need(head_dim <= 256, f"head_dim {head_dim} is larger than the generic attention kernel takes (256)")
    _need(num_heads % num_kv_heads == 0, "num_heads must be a multiple of num_kv_heads")
    _need(out.dtype == q.dtype == k_cache.dtype == v_cache.dtype, "attention: dtypes differ")
    _need(out.stride(1) == 1 and out.shape[1] == num_heads * head_dim, "attention: out shape")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane shape")
    core().call("ll_paged_attention_generic", c_int(_dtype_code(out)), _ptr(out), c_long(out.stride(0)), _ptr(q),
                c_long(q_stride), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), c_int(block_table.stride(0)),
                _ptr(token_req), _ptr(req_slot), _ptr(positions), c_int(num_tokens), c_int(num_heads),
                c_int(num_kv_heads), c_int(head_dim), c_int(page_size), c_int(k_cache.shape[0]),
                c_int(window or 0), c_float(scale), _ptr(status), _stream())


def attn_mma_supported(dtype: torch.dtype, head_dim: int, page_size: int, q_stride: int) -> bool:
    """Shapes the tensor-core attention kernel takes; everything else goes to the generic kernel."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 16 == 0 and q_stride % 8 == 0


def attn_mma_scratch_floats(row_blocks: int, num_kv_heads: int, nsplit: int, head_dim: int) -> int:
    return row_blocks * num_kv_heads * nsplit * 16 * (head_dim + 2)


def attn_mma(out: torch.Tensor, q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
             block_table: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor, req_slot: torch.Tensor,
             num_entries: int, row_blocks: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
             window: Optional[int], scale: float, nsplit: int, scratch: Optional[torch.Tensor],
             counters: Optional[torch.Tensor], status: Optional[torch.Tensor], all_single: bool = False,
             cluster: bool = False, warps: int = 4) -> None:
    """Tensor-core paged attention (bfloat16) of the step's entries: decode and prompt portions.

    ``row_blocks`` is the sum over entries of ceil(q_len * group / 16).  With ``nsplit`` > 1 the
    keys of every row block are split over that many CTAs, which park partial results in
    ``scratch`` (float32, ``attn_mma_scratch_floats`` elements); ``counters`` (int32
    [row_blocks * num_kv_heads]) must be zero and are left zero.  ``all_single`` promises that
    every entry brings exactly one token (a decode step).  ``cluster`` (nsplit 2, 4 or 8) makes the
    splits of a row block one thread-block cluster that merges through distributed shared memory;
    scratch and counters are then not needed.  ``warps``: 4 or 8 warps a CTA (8 pays when the step
    has few row blocks).
    """
    _need_cuda(out, q, k_cache, v_cache, block_table, cu_q, ctx_len, req_slot, scratch, counters)
    for t, nm in ((block_table, "block_table"), (cu_q, "cu_q"), (ctx_len, "ctx_len"), (req_slot, "req_slot"),
                  (counters, "counters")):
        _i32(t, nm)
    _f32(scratch, "scratch")
    _need(attn_mma_supported(q.dtype, head_dim, page_size, q_stride),
          f"attn_mma takes bfloat16, head_dim 64 or 128 and pages of a multiple of 16 tokens, "
          f"not {q.dtype}, {head_dim}, {page_size}")
    _need(out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16,
          "attn_mma: dtypes differ")
    _need(out.stride(1) == 1 and out.shape[1] == num_heads * head_dim and out.stride(0) % 2 == 0, "attn_mma: out")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane shape")
    _need(cu_q.numel() >= num_entries + 1 and ctx_len.numel() >= num_entries and req_slot.numel() >= num_entries,
          "attn_mma: entry arrays too short")
    if cluster:
        _need(nsplit in (2, 4, 8, 16), "attn_mma: a cluster has 2, 4, 8 or 16 splits")
    if nsplit > 1 and not cluster:
        _need(scratch is not None and counters is not None, "attn_mma: splits need scratch and counters")
        _need(scratch.numel() >= attn_mma_scratch_floats(row_blocks, num_kv_heads, nsplit, head_dim),
              "attn_mma: scratch too small")
        _need(counters.numel() >= row_blocks * num_kv_heads, "attn_mma: counters too small")
    load_library("attn_mma").call(
        "ll_attn_mma_ex", _ptr(out), c_long(out.stride(0)), _ptr(q), c_long(q_stride), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), c_int(block_table.stride(0)), _ptr(cu_q), _ptr(ctx_len), _ptr(req_slot),
        c_int(num_entries), c_int(row_blocks), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(page_size), c_int(k_cache.shape[0]), c_int(window or 0), c_float(scale), c_int(nsplit),
        c_int(1 if all_single else 0), c_int(1 if cluster else 0), c_int(warps), _ptr(scratch), _ptr(counters),
        _ptr(status), _stream())


_attn_decode_scratch = {}   # per device: (partial results, counters) of attn_decode's clusters that meet through memory
_DECODE_SCRATCH_FLOATS = 1 << 19    # 2 MB; a plan's need is (CTAs / 4) * 8 * (head size + 2 splits) floats: far less
_DECODE_SCRATCH_COUNTERS = 4096


def _decode_scratch(device, floats: int, counters: int):
    """One buffer a device, of a fixed size and never replaced: captured steps keep its address."""
    _need(floats <= _DECODE_SCRATCH_FLOATS and counters <= _DECODE_SCRATCH_COUNTERS,
          "attn_decode: too many clusters for the scratch memory of their partial results")
    have = _attn_decode_scratch.get(device)
    if have is None:
        have = (torch.empty(_DECODE_SCRATCH_FLOATS, dtype=torch.float32, device=device),
                torch.zeros(_DECODE_SCRATCH_COUNTERS, dtype=torch.int32, device=device))
        _attn_decode_scratch[device] = have
    return have


def attn_decode(out: torch.Tensor, q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                block_table: torch.Tensor, ctx_len: torch.Tensor, req_slot: torch.Tensor, num_entries: int,
                num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: Optional[int],
                scale: float, nsplit: int, status: Optional[torch.Tensor], warps: int = 4, depth: int = 0,
                nouter: int = 1) -> None:
    """Tensor-core decode attention (bfloat16), transposed product: one new token per entry, groups of at
    most 8 query heads.  ``nsplit`` in (1, 2, 4, 8) CTAs per (entry, kv head) form a cluster; ``warps`` (4 or 8)
    a CTA take the split's tiles in turn through rings of ``depth`` tiles a warp (0: the kernel's choice; 2 to 4
    for 4 warps, 2 or 3 for 8).  ``nouter`` > 1 (few requests, very long contexts; needs nsplit >= 2): that many
    clusters a (entry, kv head), each with a range of the keys, which meet through scratch memory kept by this
    module."""
    _need_cuda(out, q, k_cache, v_cache, block_table, ctx_len, req_slot)
    for t, nm in ((block_table, "block_table"), (ctx_len, "ctx_len"), (req_slot, "req_slot")):
        _i32(t, nm)
    _need(attn_mma_supported(q.dtype, head_dim, page_size, q_stride) and num_heads // num_kv_heads <= 8,
          "attn_decode takes bfloat16, head_dim 64 or 128, pages of a multiple of 16 tokens, groups of at most 8")
    _need(nsplit in (1, 2, 4, 8), "attn_decode: 1, 2, 4 or 8 splits")
    _need(warps in (4, 8), "attn_decode: 4 or 8 warps")
    _need(out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16,
          "attn_decode: dtypes differ")
    _need(out.stride(1) == 1 and out.shape[1] == num_heads * head_dim and out.stride(0) % 2 == 0, "attn_decode: out")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane shape")
    _need(ctx_len.numel() >= num_entries and req_slot.numel() >= num_entries, "attn_decode: entry arrays too short")
    scratch = counters = None
    if nouter > 1:
        _need(nsplit >= 2 and 1 < nouter <= 64 and warps == 8 and depth in (0, 2),
              "attn_decode: several clusters a (entry, kv head) need nsplit >= 2, 8 warps and rings of two tiles")
        depth = 2
        scratch, counters = _decode_scratch(q.device, num_entries * num_kv_heads * nouter * 8 * (head_dim + 2 * nsplit),
                                            num_entries * num_kv_heads * nsplit)
    load_library("attn_mma").call(
        "ll_attn_decode", _ptr(out), c_long(out.stride(0)), _ptr(q), c_long(q_stride), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), c_int(block_table.stride(0)), _ptr(ctx_len), _ptr(req_slot), c_int(num_entries),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page_size), c_int(k_cache.shape[0]),
        c_int(window or 0), c_float(scale), c_int(nsplit), c_int(warps), c_int(depth), c_int(nouter), _ptr(scratch),
        _ptr(counters), _ptr(status), _stream())


def attn_prefill(out: torch.Tensor, q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 block_table: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor, req_slot: torch.Tensor,
                 num_entries: int, row_blocks: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 page_size: int, window: Optional[int], scale: float, status: Optional[torch.Tensor]) -> None:
    """Tensor-core paged attention (bfloat16) for portions of prompts: 128 query rows a CTA share the
    keys and values through shared memory.  ``row_blocks`` is the sum over the entries of
    ceil(q_len * group / 128).  Same shapes as ``attn_mma``."""
    _need_cuda(out, q, k_cache, v_cache, block_table, cu_q, ctx_len, req_slot)
    for t, nm in ((block_table, "block_table"), (cu_q, "cu_q"), (ctx_len, "ctx_len"), (req_slot, "req_slot")):
        _i32(t, nm)
    _need(attn_mma_supported(q.dtype, head_dim, page_size, q_stride),
          f"attn_prefill takes bfloat16, head_dim 64 or 128 and pages of a multiple of 16 tokens, "
          f"not {q.dtype}, {head_dim}, {page_size}")
    _need(out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16,
          "attn_prefill: dtypes differ")
    _need(out.stride(1) == 1 and out.shape[1] == num_heads * head_dim and out.stride(0) % 8 == 0,
          "attn_prefill: out")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane shape")
    _need(cu_q.numel() >= num_entries + 1 and ctx_len.numel() >= num_entries and req_slot.numel() >= num_entries,
          "attn_prefill: entry arrays too short")
    load_library("attn_mma").call(
        "ll_attn_prefill", _ptr(out), c_long(out.stride(0)), _ptr(q), c_long(q_stride), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), c_int(block_table.stride(0)), _ptr(cu_q), _ptr(ctx_len), _ptr(req_slot),
        c_int(num_entries), c_int(row_blocks), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(page_size), c_int(k_cache.shape[0]), c_int(window or 0), c_float(scale), _ptr(status), _stream())


def attn_prefill_tc_supported(dtype: torch.dtype, head_dim: int, page_size: int, q_stride: int, group: int) -> bool:
    """Whether the tcgen05 prefill attention takes this shape."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and q_stride % 8 == 0 and 1 <= group <= 128
            and (page_size in (8, 16, 32) or (page_size > 0 and page_size % 64 == 0)))


def attn_prefill_tc_blocks(q_lens, group: int) -> int:
    """Row blocks of a step for ``attn_prefill_tc``: a CTA takes floor(128 / group) tokens of one entry."""
    tpb = 128 // group
    return sum((int(n) + tpb - 1) // tpb for n in q_lens)


_attn_tc_scratch = {}


def attn_prefill_tc_plan(entries, group: int, window: Optional[int], num_kv_heads: int = 1, slots: int = 0):
    """(row blocks, nsplit, split_len) of a step for ``attn_prefill_tc``.  ``entries``: (cached tokens, new tokens)
    per entry; a row block takes floor(128 / group) tokens and walks n key blocks of 64.

    A CTA's blocks are a chain (scores, softmax, P V: about 1.4 us a block), so a step lasts as long as its
    longest CTA, and a CTA that finds no room on the SMs at once waits for a whole one to end (the hardware hands
    CTAs out in order).  So row blocks are cut into splits of at most ``split_len`` blocks, with the smallest
    ``split_len`` for which all CTAs of the step fit the ``slots`` (two an SM) at once: a whole causal prompt of
    2,048 tokens (row blocks of 1..32 blocks, 2 kv heads) gets 16, i.e. its longer half is cut in two.  Not below
    4 blocks a split or over 8 splits (every split's partial result goes through scratch memory); when the
    unsplit row blocks already exceed the slots, nothing is cut."""
    tpb = 128 // group
    lengths = []
    for ctx, q in entries:
        for first in range(0, q, tpb):
            hi = ctx + min(first + tpb, q) - 1
            lo = max(0, ctx + first - window + 1) if window else 0
            lengths.append(hi // 64 - lo // 64 + 1)
    blocks = len(lengths)
    if not lengths or slots <= 0 or blocks * num_kv_heads > slots:
        return blocks, 1, 1 << 20
    longest = max(lengths)
    best = longest
    for t in range(max(4, (longest + 7) // 8), longest + 1):
        if sum((n + t - 1) // t for n in lengths) * num_kv_heads <= slots:
            best = t
            break
    if best * 5 > longest * 4:      # cutting off less than a fifth of the longest chain does not pay for the merges
        return blocks, 1, 1 << 20   # (four portions of 512 behind 1,536 tokens: 49 us uncut, 52.5 us cut at 29 of 32)
    most = (longest + best - 1) // best
    nsplit = 1 if most <= 1 else 2 if most <= 2 else 4 if most <= 4 else 8
    return blocks, nsplit, best


def attn_prefill_tc_splits(row_blocks: int, num_kv_heads: int, device) -> int:
    """CTAs a row block's keys may be split over when nothing is known about the entries' lengths: as many as
    still fit the SMs (two CTAs each) at once."""
    ctas = row_blocks * num_kv_heads
    slots = 2 * sm_count(device)
    for n in (8, 4, 2):
        if ctas * n <= slots:
            return n
    return 1


def attn_prefill_tc(out: torch.Tensor, q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_table: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor, req_slot: torch.Tensor,
                    num_entries: int, row_blocks: int, num_heads: int, num_kv_heads: int, head_dim: int,
                    page_size: int, window: Optional[int], scale: float, status: Optional[torch.Tensor],
                    nsplit: Optional[int] = None, split_len: int = 8) -> None:
    """Paged attention for portions of prompts on the tcgen05 tensor cores (TMA loads, S and O in tensor
    memory).  ``row_blocks`` from ``attn_prefill_tc_blocks``.  Otherwise as ``attn_prefill``.
    ``nsplit`` (1, 2, 4, 8; default: by the size of the step): the keys of a row block are split over up to that
    many CTAs of about ``split_len`` blocks of 64 keys each (``attn_prefill_tc_plan`` chooses both), which merge
    through scratch memory kept by this module (grown when needed, never shrunk)."""
    _need_cuda(out, q, k_cache, v_cache, block_table, cu_q, ctx_len, req_slot)
    for t, nm in ((block_table, "block_table"), (cu_q, "cu_q"), (ctx_len, "ctx_len"), (req_slot, "req_slot")):
        _i32(t, nm)
    _need(attn_prefill_tc_supported(q.dtype, head_dim, page_size, q_stride, num_heads // num_kv_heads),
          f"attn_prefill_tc takes bfloat16, head_dim 64 or 128 and pages of 8, 16, 32 or a multiple of 64 tokens, "
          f"not {q.dtype}, {head_dim}, {page_size}")
    _need(out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16,
          "attn_prefill_tc: dtypes differ")
    _need(out.stride(1) == 1 and out.shape[1] == num_heads * head_dim and out.stride(0) % 8 == 0,
          "attn_prefill_tc: out")
    _need(q.stride(1) == 1 and q.shape[1] >= num_heads * head_dim and q.stride(0) == q_stride, "attn_prefill_tc: q")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane shape")
    _need(cu_q.numel() >= num_entries + 1 and ctx_len.numel() >= num_entries and req_slot.numel() >= num_entries,
          "attn_prefill_tc: entry arrays too short")
    if nsplit is None:
        nsplit = attn_prefill_tc_splits(row_blocks, num_kv_heads, q.device)
    _need(nsplit in (1, 2, 4, 8), "attn_prefill_tc: nsplit is 1, 2, 4 or 8")
    scratch = counters = None
    if nsplit > 1:
        floats = row_blocks * num_kv_heads * nsplit * 128 * (head_dim + 2)
        have = _attn_tc_scratch.get(q.device)
        if have is None or have[0].numel() < floats or have[1].numel() < row_blocks * num_kv_heads:
            have = (torch.empty(max(floats, have[0].numel() if have else 0), dtype=torch.float32, device=q.device),
                    torch.zeros(max(row_blocks * num_kv_heads, 1024), dtype=torch.int32, device=q.device))
            _attn_tc_scratch[q.device] = have
        scratch, counters = have
    load_library("attn_tc").call(
        "ll_attn_prefill_tc", _ptr(out), c_long(out.stride(0)), _ptr(q), c_long(q_stride), c_int(q.shape[0]),
        _ptr(k_cache), _ptr(v_cache), _ptr(block_table), c_int(block_table.stride(0)), _ptr(cu_q), _ptr(ctx_len),
        _ptr(req_slot), c_int(num_entries), c_int(row_blocks), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(page_size), c_int(k_cache.shape[0]), c_int(window or 0), c_float(scale), c_int(nsplit), c_int(max(1, int(split_len))),
        _ptr(scratch), _ptr(counters), _ptr(status), _stream())


_sample_scratch = {}


def sample_scratch_floats(rows: int, vocab: int) -> int:
    return rows * ((vocab + 2047) // 2048) * 3


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           uniform: Optional[torch.Tensor] = None, rows: Optional[int] = None,
           scratch: Optional[torch.Tensor] = None) -> None:
    """Greedy (temperature None or <= 0) or temperature sampling of each row of float32 logits.

    Two kernels (per-chunk partial results, then one block per row); ``scratch`` holds the partial
    results (float32, ``sample_scratch_floats`` elements) and is taken from a per-device cache if
    not given."""
    _need_cuda(logits, out, temperature, uniform)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "logits must be float32 2-D")
    _i32(out, "out")
    _f32(temperature, "temperature")
    _f32(uniform, "uniform")
    n = logits.shape[0] if rows is None else rows
    _need(out.numel() >= n, "sample: out too small")
    need = sample_scratch_floats(n, logits.shape[1])
    if scratch is None:
        scratch = _sample_scratch.get(logits.device)
        if scratch is None or scratch.numel() < need:
            scratch = torch.empty(max(need, 1024), dtype=torch.float32, device=logits.device)
            _sample_scratch[logits.device] = scratch
    _f32(scratch, "scratch")
    _need(scratch.numel() >= need, "sample: scratch too small")
    core().call("ll_sample", _ptr(logits), c_long(logits.stride(0)), _ptr(temperature), _ptr(uniform), _ptr(out),
                c_int(n), c_int(logits.shape[1]), _ptr(scratch), _stream())


# --------------------------------------------------------------------------
SMALL_M = 64          # the most tokens the weight-streaming kernel takes


def smallm_preferred(x: torch.Tensor, weight: torch.Tensor, gated: bool = False) -> bool:
    """Where the hand-written kernel is used instead of the library product: few tokens and a
    weight matrix small enough that the library's tile shapes leave most SMs idle (measured on
    B200: the q|k|v and output projections; the library wins on the wide feed-forward and
    lm_head products)."""
    if not smallm_supported(x, weight):
        return False
    n, k = weight.shape
    return x.shape[0] <= 16 and n <= 4096 and k <= 2048 and not gated


def smallm_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and 0 < x.shape[0] <= SMALL_M and x.shape[1] % 32 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and weight.is_contiguous() and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_smallm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gated: bool = False) -> torch.Tensor:
    """out = x @ weight.T for up to 64 tokens with the weight-streaming kernel.

    ``gated``: weight holds gate rows then up rows ([2 I, K]); out [M, I] = silu(gate) * up.
    out may be bfloat16 or (not gated) float32.
    """
    _need_cuda(x, weight, out)
    _need(smallm_supported(x, weight), "gemm_smallm: bfloat16, at most 64 tokens, K a multiple of 32")
    m, k = x.shape
    n = weight.shape[0] // 2 if gated else weight.shape[0]
    _need(weight.shape[1] == k and (not gated or weight.shape[0] % 2 == 0), "gemm_smallm: weight shape")
    _need(out.shape[0] == m and out.shape[1] == n and out.stride(1) == 1, "gemm_smallm: out shape")
    _need(out.dtype in (torch.bfloat16, torch.float32) and not (gated and out.dtype != torch.bfloat16),
          "gemm_smallm: out dtype")
    load_library("gemm_smallm").call(
        "ll_gemm_smallm", _ptr(out), c_long(out.stride(0)), c_int(1 if out.dtype == torch.float32 else 0), _ptr(x),
        c_long(x.stride(0)), _ptr(weight), c_int(m), c_int(n), c_int(k), c_int(1 if gated else 0), _stream())
    return out


STREAM_M = 32         # the most tokens the bulk-copy streaming kernel takes
STREAM_M_NARROW = 64  # ... for its units of 16 features (q|k|v, o): the tokens then go in two blocks of 32
_sm_count = {}


def sm_count(device) -> int:
    n = _sm_count.get(device)
    if n is None:
        n = torch.cuda.get_device_properties(device).multi_processor_count
        _sm_count[device] = n
    return n


def stream_mode(x: torch.Tensor, weight: torch.Tensor, gated: bool = False) -> Optional[int]:
    """Work-unit shape of ``gemm_stream`` for this product (0 wide, 1 gated, 2 narrow), or None."""
    if not (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and 0 < x.shape[0] <= STREAM_M_NARROW and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and weight.is_contiguous() and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0):
        return None
    k = x.shape[1]
    if x.shape[0] > STREAM_M:
        # 33 to 64 tokens: only small products with units of 16 features (bfloat16 out, k whole), a unit a CTA in
        # both blocks of tokens at once and k up to 1,536: a CTA re-reads its 32 token rows (twice its weights' bytes)
        # with every unit, which a larger product pays for (Qwen2-7B sizes at batch 64: 4.33 -> 4.85 ms a step;
        # 2.5-3B sizes 3.27 -> 3.43, and 3.32 with the o projection, k = 2,048, alone) and the 1.5B sizes gain from
        # (2.06 -> 2.00)
        units = (weight.shape[0] + 15) // 16
        return 2 if (not gated and k % 256 == 0 and k <= 1536 and 2 * units <= 2 * sm_count(x.device)) else None
    if gated:
        return 1 if k % 128 == 0 else None
    n = weight.shape[0]
    if n >= 8192 and k % 128 == 0:
        return 0
    if k % 256 == 0:
        return 2
    return 0 if k % 128 == 0 else None


def stream_ksplit(n: int, k: int, mode: int, device) -> int:
    """Parts to cut k into so that a product with few output features still has work units for every
    SM (only worth it for a long k).  The kernel needs every part non-empty: the count is normalised."""
    if mode == 1 or k < 4096:
        return 1
    feats, chunk = (64, 128) if mode == 0 else (16, 256)
    units = (n + feats - 1) // feats
    chunks = k // chunk
    want = max(1, min((2 * sm_count(device)) // units, chunks // 4))
    cpp = (chunks + want - 1) // want
    return (chunks + cpp - 1) // cpp


def gemm_stream(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, mode: int,
                status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = x @ weight.T for up to 32 bfloat16 tokens (64 for mode 2 to bfloat16 with k whole) with the TMA
    weight-streaming kernel.

    mode 0: units of 64 output features; 1: SiLU-gated (weight [2 I, K], out [M, I]);
    2: units of 16 features with k split over the warps.  A float32 ``out`` of shape
    [parts, M, N] receives partial sums of a k range cut into ``parts`` (see ``stream_ksplit``).
    """
    _need_cuda(x, weight, out, status)
    m, k = x.shape
    gated = mode == 1
    n = weight.shape[0] // 2 if gated else weight.shape[0]
    _need(stream_mode(x, weight, gated) is not None, "gemm_stream: bfloat16, at most 32 tokens (64 for mode 2), K % 128 == 0")
    _need(mode in (0, 1, 2) and k % (256 if mode == 2 else 128) == 0, "gemm_stream: K does not fit the mode")
    _need(weight.shape[1] == k, "gemm_stream: weight shape")
    ksplit = 1
    if out.dim() == 3:
        ksplit = out.shape[0]
        _need(out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape[1:]) == (m, n) and not gated,
              "gemm_stream: partial sums go to a contiguous float32 [parts, M, N]")
        out_stride = n
    else:
        _need(out.shape[0] == m and out.shape[1] == n and out.stride(1) == 1, "gemm_stream: out shape")
        out_stride = out.stride(0)
    _need(out.dtype == torch.bfloat16 or (out.dtype == torch.float32 and not gated), "gemm_stream: out dtype")
    load_library("gemm_stream").call(
        "ll_gemm_stream", _ptr(out), c_long(out_stride), c_int(1 if out.dtype == torch.float32 else 0), _ptr(x),
        c_long(x.stride(0)), _ptr(weight), c_int(m), c_int(n), c_int(k), c_int(mode), c_int(ksplit),
        c_int(sm_count(x.device)), _ptr(status if status is not None else TIMELINE_STATUS), _stream())
    return out


SUMSQ_ROWS = 64     # rows of a sums-of-squares record (the most tokens ``gemm_stream`` takes)
NORM_SPLIT = os.environ.get("LITE_LANG_B200_NORM_SPLIT", "1") != "0"   # 0: the norm between two streaming products
                                                                        # stays a kernel of its own (for comparisons)


def into_norm_supported(x: torch.Tensor, w_before: torch.Tensor, residual: torch.Tensor) -> bool:
    """Whether ``gemm_stream_into_norm`` takes the product ``x @ w_before.T`` added to ``residual``: a streaming
    product of a decode step with units of 16 features and an unsplit k, bfloat16 residual rows of its shape."""
    n = w_before.shape[0]
    return (NORM_SPLIT and stream_mode(x, w_before) == 2 and n % 16 == 0 and residual.dtype == torch.bfloat16
            and residual.dim() == 2 and tuple(residual.shape) == (x.shape[0], n) and residual.stride(1) == 1)


def gated_scaled_supported(rows: torch.Tensor, w_gate_up: torch.Tensor) -> bool:
    """Whether ``gemm_stream_gated_scaled`` takes rows of this shape: where the streaming gated product runs."""
    if not (NORM_SPLIT and w_gate_up.shape[1] == rows.shape[1] and rows.shape[0] <= SUMSQ_ROWS):
        return False
    if tc_preferred(rows, w_gate_up, gated=True):      # 17 tokens and more: the tcgen05 kernel has the same epilogue
        return True
    return stream_mode(rows, w_gate_up, gated=True) == 1


def gemm_stream_into_norm(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor,
                          status: Optional[torch.Tensor] = None):
    """residual += x @ weight.T (rounded as the separate product and sum would be); returns (u, sumsq): u = the new
    residual rows times ``norm_weight`` (bfloat16), sumsq float32 [out / 16, 64] = the sums of squares of each
    row's 16 values of a unit.  With ``gemm_stream_gated_scaled`` after it, this is the residual sum, the RMS norm
    and the two products around them in two kernels instead of three."""
    _need_cuda(x, weight, residual, norm_weight, status)
    m, k = x.shape
    n = weight.shape[0]
    _need(into_norm_supported(x, weight, residual), "gemm_stream_into_norm: bfloat16, at most 64 tokens, K % 256 == 0, "
                                                    "N % 16 == 0, residual bfloat16 [tokens, N]")
    _need(norm_weight.dtype == torch.float32 and norm_weight.numel() == n and norm_weight.is_contiguous(),
          "gemm_stream_into_norm: the norm's weight is float32 [out]")
    u = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    sumsq = torch.empty((n // 16, SUMSQ_ROWS), dtype=torch.float32, device=x.device)
    load_library("gemm_stream").call(
        "ll_gemm_stream_into_norm", _ptr(u), c_long(u.stride(0)), _ptr(residual), c_long(residual.stride(0)),
        _ptr(norm_weight), _ptr(sumsq), _ptr(x), c_long(x.stride(0)), _ptr(weight), c_int(m), c_int(n), c_int(k),
        c_int(sm_count(x.device)), _ptr(status if status is not None else TIMELINE_STATUS), _stream())
    return u, sumsq


def gemm_stream_gated_scaled(u: torch.Tensor, w_gate_up: torch.Tensor, sumsq: torch.Tensor, eps: float,
                             status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(g) * up of the rows x = u / sqrt(mean of squares + eps), where u is already multiplied by the norm's
    weight and ``sumsq`` [units, 64] holds the rows' sums of squares in parts (``gemm_stream_into_norm``)."""
    _need_cuda(u, w_gate_up, sumsq, status)
    m, k = u.shape
    inter = w_gate_up.shape[0] // 2
    _need(gated_scaled_supported(u, w_gate_up), "gemm_stream_gated_scaled: bfloat16, K % 128 == 0, at most 32 tokens (64 where the tcgen05 kernel takes the product)")
    _need(sumsq.dtype == torch.float32 and sumsq.dim() == 2 and sumsq.shape[1] == SUMSQ_ROWS and sumsq.is_contiguous(),
          "gemm_stream_gated_scaled: sums of squares are float32 [units, 64]")
    act = torch.empty((m, inter), dtype=torch.bfloat16, device=u.device)
    if tc_preferred(u, w_gate_up, gated=True):
        return gemm_tc(u, w_gate_up, act, gated=True, status=status, sumsq=sumsq, eps=eps)
    load_library("gemm_stream").call(
        "ll_gemm_stream_gated_scaled", _ptr(act), c_long(act.stride(0)), _ptr(u), c_long(u.stride(0)), _ptr(w_gate_up),
        c_int(m), c_int(inter), c_int(k), _ptr(sumsq), c_int(sumsq.shape[0]), c_float(eps),
        c_int(sm_count(u.device)), _ptr(status if status is not None else TIMELINE_STATUS), _stream())
    return act


def qkv_rope_supported(x: torch.Tensor, w_qkv: torch.Tensor, head_dim: int, rot_dim: int) -> bool:
    """Whether the fused projection + bias + rotation + cache write kernel takes this step."""
    return (stream_mode(x, w_qkv) is not None and x.shape[1] % 256 == 0 and head_dim % 16 == 0
            and rot_dim == head_dim)


def gemm_stream_qkv_rope(q_out: torch.Tensor, x: torch.Tensor, w_qkv: torch.Tensor, bias: Optional[torch.Tensor],
                         positions: torch.Tensor, cos_sin: torch.Tensor, num_heads: int, num_kv_heads: int,
                         head_dim: int, slot_map: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                         v_cache: Optional[torch.Tensor], page_size: int, status: Optional[torch.Tensor]) -> None:
    """q|k|v projection of up to 32 tokens with what follows it, in one kernel: bias, half-split rotation
    of q and k, q into ``q_out`` [tokens, num_heads * head_dim], k and v into the cache plane."""
    _need_cuda(q_out, x, w_qkv, bias, positions, cos_sin, slot_map, k_cache, v_cache, status)
    _f32(bias, "bias")
    _f32(cos_sin, "cos_sin")
    _i32(positions, "positions")
    _i32(slot_map, "slot_map")
    m, k = x.shape
    width = (num_heads + 2 * num_kv_heads) * head_dim
    _need(qkv_rope_supported(x, w_qkv, head_dim, cos_sin.shape[1]), "gemm_stream_qkv_rope: shapes")
    _need(tuple(w_qkv.shape) == (width, k), "gemm_stream_qkv_rope: weight shape")
    _need(q_out.dtype == torch.bfloat16 and q_out.shape[0] == m and q_out.shape[1] >= num_heads * head_dim
          and q_out.stride(1) == 1, "gemm_stream_qkv_rope: q_out")
    if bias is not None:
        _need(bias.numel() == width, "bias size")
    num_slots = 0
    if slot_map is not None:
        _need(k_cache is not None and v_cache is not None and k_cache.dtype == torch.bfloat16
              and k_cache.is_contiguous() and v_cache.is_contiguous()
              and tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane")
        num_slots = k_cache.shape[0] * page_size
    load_library("gemm_stream").call(
        "ll_gemm_stream_qkv_rope", _ptr(q_out), c_long(q_out.stride(0)), _ptr(x), c_long(x.stride(0)), _ptr(w_qkv),
        c_int(m), c_int(k), _ptr(bias), _ptr(positions), _ptr(cos_sin), c_int(cos_sin.shape[0]), c_int(num_heads),
        c_int(num_kv_heads), c_int(head_dim), _ptr(slot_map), _ptr(k_cache), _ptr(v_cache), c_int(page_size),
        c_long(num_slots), c_int(sm_count(x.device)), _ptr(status), _stream())


# A timeline build (LITE_LANG_B200_TIMELINE=1, see csrc/common.cuh): the kernels stamp the clock behind the status
# word that the runner hands out; those that a caller gives no status word get the runner's.
TIMELINE_KERNELS = ("qkv", "attention", "o", "gated", "down", "logits")
TIMELINE_SLOTS = len(TIMELINE_KERNELS) * 512 * 4
TIMELINE_STATUS = None


def timeline_build() -> bool:
    from .csrc.build import timeline_build as on
    return on()


TC_M = 128          # most tokens the tcgen05 weight-streaming kernel takes
TC_ENABLED = os.environ.get("LITE_LANG_B200_TC", "1") != "0"   # 0: library products instead (for comparisons)


def tc_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether ``gemm_tc`` takes this product: bfloat16, at most 128 tokens, K % 64 == 0, aligned rows."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and 0 < x.shape[0] <= TC_M and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.shape[1] % 64 == 0
            and weight.is_contiguous() and weight.shape[1] == x.shape[1]
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


TC_MIN_M = 17       # from this many tokens on the tcgen05 kernel was measured ahead of gemm_stream's mma.sync tiles


def tc_preferred(x: torch.Tensor, weight: torch.Tensor, gated: bool = False, wide: bool = False) -> bool:
    """Where the tcgen05 kernel was measured ahead on a B200: more tokens than ``gemm_stream`` takes well
    (its mma.sync tiles get slower from 16 tokens up) and few enough that the step is still bound by reading
    the weights.  The gated feed-forward and a wide product (the logits) up to 64 tokens; a product with a
    long k (split over k, partial sums to the norm) up to 128.  Other products of such steps go to
    ``gemm_stream`` (up to 32 tokens) or the library."""
    if not (TC_ENABLED and tc_supported(x, weight) and x.shape[0] >= TC_MIN_M):
        return False
    if gated or wide:
        return x.shape[0] <= 64
    return x.shape[1] >= 4096 and tc_ksplit(weight.shape[0], x.shape[1], x.device) > 1


def tc_ksplit(n: int, k: int, device) -> int:
    """Parts to cut k into so that a product with few output features (units of 128) has a unit for
    every SM; every part keeps at least four 64-wide boxes.  Normalised so that no part is empty."""
    units = (n + 127) // 128
    boxes = k // 64
    want = max(1, min(sm_count(device) // units, boxes // 4))
    per = (boxes + want - 1) // want
    return (boxes + per - 1) // per


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gated: bool = False,
            status: Optional[torch.Tensor] = None, sumsq: Optional[torch.Tensor] = None, eps: float = 0.0) -> torch.Tensor:
    """out = x @ weight.T for up to 128 bfloat16 tokens on the tcgen05 tensor cores (weights streamed
    by TMA, accumulator in tensor memory).  ``gated``: weight is [2 I, K] and out = silu(gate) * up.
    A float32 ``out`` of shape [parts, M, N] receives the partial sums of a k range cut into parts."""
    _need_cuda(x, weight, out, status)
    _need(tc_supported(x, weight), "gemm_tc: bfloat16, at most 128 tokens, K % 64 == 0, 16-byte aligned rows")
    m, k = x.shape
    n = weight.shape[0] // 2 if gated else weight.shape[0]
    ksplit = 1
    if out.dim() == 3:
        ksplit = out.shape[0]
        _need(out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape[1:]) == (m, n) and not gated,
              "gemm_tc: partial sums go to a contiguous float32 [parts, M, N]")
        per = (k // 64 + ksplit - 1) // ksplit
        _need((k // 64 + per - 1) // per == ksplit, "gemm_tc: a part of k would be empty")
        out_stride = n
    else:
        _need(out.shape[0] == m and out.shape[1] == n and out.stride(1) == 1, "gemm_tc: out shape")
        out_stride = out.stride(0)
    _need(out.dtype == torch.bfloat16 or (out.dtype == torch.float32 and not gated), "gemm_tc: out dtype")
    load_library("gemm_tc").call(
        "ll_gemm_tc", _ptr(out), c_long(out_stride), c_int(1 if out.dtype == torch.float32 else 0), _ptr(x),
        c_long(x.stride(0)), _ptr(weight), c_int(m), c_int(n), c_int(k), c_int(1 if gated else 0), c_int(ksplit),
        c_int(sm_count(x.device)), _ptr(sumsq), c_int(0 if sumsq is None else sumsq.shape[0]), c_float(eps),
        _ptr(status if status is not None else TIMELINE_STATUS), _stream())
    return out


PAIR_MIN_M = 65     # from this many tokens on (measured from 129 to 4,096) the two-SM tcgen05 kernel with the
                    # activation in its epilogue is ahead of a library product followed by ``silu_mul``


def pair_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether ``gemm_pair`` takes this product: bfloat16, K % 8 == 0, 16-byte aligned rows."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] > 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.shape[1] % 8 == 0
            and weight.is_contiguous() and weight.shape[1] == x.shape[1]
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_pair(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gated: bool = False,
              status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = x @ weight.T for many bfloat16 tokens on the tcgen05 tensor cores, a pair of SMs a tile of
    256 tokens x 256 columns.  ``gated``: weight is [2 I, K] and out = silu(gate) * up, the activation done
    on the accumulator, so gate and up never go to memory."""
    _need_cuda(x, weight, out, status)
    _need(pair_supported(x, weight), "gemm_pair: bfloat16, K % 8 == 0, 16-byte aligned rows")
    m, k = x.shape
    n = weight.shape[0] // 2 if gated else weight.shape[0]
    _need(out.dtype == torch.bfloat16 and out.dim() == 2 and out.shape[0] == m and out.shape[1] == n
          and out.stride(1) == 1, "gemm_pair: out is bfloat16 [M, N] with unit column stride")
    load_library("gemm_pair").call(
        "ll_gemm_pair", _ptr(out), c_long(out.stride(0)), _ptr(x), c_long(x.stride(0)), _ptr(weight), c_int(m),
        c_int(n), c_int(k), c_int(1 if gated else 0), c_int(sm_count(x.device)), _ptr(status), _stream())
    return out


def pair_qkv_supported(x: torch.Tensor, w_qkv: torch.Tensor, head_dim: int, rot_dim: int) -> bool:
    """Whether the two-SM tcgen05 projection with bias, rotation and cache write in its epilogue takes
    this step: whole heads in a tile of 256 columns, rotation of the whole head."""
    return TC_ENABLED and pair_supported(x, w_qkv) and head_dim in (64, 128, 256) and rot_dim == head_dim


def pair_qkv_preferred(x: torch.Tensor, w_qkv: torch.Tensor) -> bool:
    """Where it was measured ahead of a library product followed by ``bias_rope_store``: when the
    tiles of 256 tokens x 256 columns are enough for a good part of the SM pairs."""
    tiles = ((x.shape[0] + 255) // 256) * ((w_qkv.shape[0] + 255) // 256)
    return tiles * 4 >= sm_count(x.device)


def gemm_pair_qkv_rope(q_out: torch.Tensor, x: torch.Tensor, w_qkv: torch.Tensor, bias: Optional[torch.Tensor],
                       positions: torch.Tensor, cos_sin: torch.Tensor, num_heads: int, num_kv_heads: int,
                       head_dim: int, slot_map: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                       v_cache: Optional[torch.Tensor], page_size: int, status: Optional[torch.Tensor]) -> None:
    """q|k|v projection of many tokens with what follows it, in one kernel: bias, half-split rotation of q
    and k, q into ``q_out`` [tokens, num_heads * head_dim], k and v into the cache plane."""
    _need_cuda(q_out, x, w_qkv, bias, positions, cos_sin, slot_map, k_cache, v_cache, status)
    _f32(bias, "bias")
    _f32(cos_sin, "cos_sin")
    _i32(positions, "positions")
    _i32(slot_map, "slot_map")
    m, k = x.shape
    width = (num_heads + 2 * num_kv_heads) * head_dim
    _need(pair_qkv_supported(x, w_qkv, head_dim, cos_sin.shape[1]), "gemm_pair_qkv_rope: shapes")
    _need(tuple(w_qkv.shape) == (width, k), "gemm_pair_qkv_rope: weight shape")
    _need(q_out.dtype == torch.bfloat16 and q_out.shape[0] == m and q_out.shape[1] >= num_heads * head_dim
          and q_out.stride(1) == 1 and q_out.stride(0) % 8 == 0, "gemm_pair_qkv_rope: q_out")
    _need(cos_sin.is_contiguous() and positions.numel() >= m, "gemm_pair_qkv_rope: table and positions")
    if bias is not None:
        _need(bias.numel() == width and bias.is_contiguous(), "bias size")
    num_slots = 0
    if slot_map is not None:
        _need(k_cache is not None and v_cache is not None and k_cache.dtype == torch.bfloat16
              and k_cache.is_contiguous() and v_cache.is_contiguous() and slot_map.numel() >= m
              and tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane")
        num_slots = k_cache.shape[0] * page_size
    load_library("gemm_pair").call(
        "ll_gemm_pair_qkv_rope", _ptr(q_out), c_long(q_out.stride(0)), _ptr(x), c_long(x.stride(0)), _ptr(w_qkv),
        c_int(m), c_int(k), _ptr(bias), _ptr(positions), _ptr(cos_sin), c_int(cos_sin.shape[0]), c_int(num_heads),
        c_int(num_kv_heads), c_int(head_dim), _ptr(slot_map), _ptr(k_cache), _ptr(v_cache), c_int(page_size),
        c_long(num_slots), c_int(sm_count(x.device)), _ptr(status), _stream())


ACCUMULATE_MIN_M = 129   # more tokens than any of the hand-written plain products takes: library territory


def accumulate_preferred(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether ``linear_accumulate`` should stand for ``linear`` + a later residual sum: when the product
    is a library one anyway (portions of prompts), its epilogue adds the residual for the price of reading it."""
    return x.shape[0] >= ACCUMULATE_MIN_M and x.dtype == weight.dtype


def linear_accumulate(x: torch.Tensor, weight: torch.Tensor, acc: torch.Tensor) -> None:
    """acc += x @ weight.T in place (library product with beta = 1: float32 accumulation, the sum with ``acc``
    in float32, one rounding), so that the norm after it reads the residual stream only."""
    _need_cuda(x, weight, acc)
    _need(acc.dtype == x.dtype and acc.shape[0] == x.shape[0] and acc.shape[1] == weight.shape[0]
          and acc.stride(1) == 1, "linear_accumulate: acc is [tokens, out] of the operands' dtype")
    if x.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("TF32 is on; call ops.configure_matmul_precision() before a float32 product")
    torch.addmm(acc, x, weight.t(), out=acc)


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x @ Wg.T) * (x @ Wu.T) with W = [Wg; Wu]: fused for few tokens, else product + kernel."""
    inter = w_gate_up.shape[0] // 2
    act = torch.empty((x.shape[0], inter), dtype=x.dtype, device=x.device)
    if tc_preferred(x, w_gate_up, gated=True):
        return gemm_tc(x, w_gate_up, act, gated=True)
    if stream_mode(x, w_gate_up, gated=True) is not None:
        return gemm_stream(x, w_gate_up, act, 1)
    if smallm_preferred(x, w_gate_up, gated=True):
        return gemm_smallm(x, w_gate_up, act, gated=True)
    if TC_ENABLED and x.shape[0] >= PAIR_MIN_M and pair_supported(x, w_gate_up):
        return gemm_pair(x, w_gate_up, act, gated=True)
    gu = linear(x, w_gate_up)
    silu_mul(act, gu)
    return act


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, partial_ok: bool = False) -> torch.Tensor:
    """x [n, in] times weight [out, in] transposed.

    Up to 32 bfloat16 tokens (decode) go to the hand-written TMA weight-streaming kernel
    (``gemm_stream``), or to ``gemm_smallm`` for shapes that one does not take.  Everything
    else is a library (cuBLAS) product, as in the reference: float32 operands give a true
    float32 product (TF32 is off); bfloat16 operands accumulate in float32.
    ``out_dtype=torch.float32`` with bfloat16 operands keeps the float32 accumulator as the
    result (the logits).  ``partial_ok``: the caller's consumer (the fused residual-and-norm
    kernel) accepts float32 partial sums [parts, n, out] of a product split over k.
    """
    _need_cuda(x, weight)
    if out is None and partial_ok and out_dtype in (None, x.dtype) and tc_preferred(x, weight):
        parts = tc_ksplit(weight.shape[0], x.shape[1], x.device)
        out = torch.empty((parts, x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        return gemm_tc(x, weight, out)
    if out is None and weight.shape[0] >= 8192 and tc_preferred(x, weight, wide=True):
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype or x.dtype, device=x.device)
        return gemm_tc(x, weight, out)
    mode = stream_mode(x, weight) if (out is None or out.stride(1) == 1) else None
    many = x.shape[0] > STREAM_M       # 33 to 64 tokens: bfloat16 out, k whole
    if mode is not None and many and ((out_dtype or x.dtype) != torch.bfloat16 or (out is not None and out.dtype != torch.bfloat16)):
        mode = None
    if mode is not None:
        dt = out_dtype or x.dtype
        if out is None:
            parts = (stream_ksplit(weight.shape[0], x.shape[1], mode, x.device)
                     if (partial_ok and dt == x.dtype and not many) else 1)
            if parts > 1:
                out = torch.empty((parts, x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
                return gemm_stream(x, weight, out, mode)
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=dt, device=x.device)
        if out.dtype == dt:
            return gemm_stream(x, weight, out, mode)
    if smallm_preferred(x, weight) and (out is None or out.stride(1) == 1):
        dt = out_dtype or x.dtype
        if out is None:
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=dt, device=x.device)
        if out.dtype == dt:
            return gemm_smallm(x, weight, out)
    if x.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("TF32 is on; call ops.configure_matmul_precision() before a float32 product")
    if out_dtype is not None and out_dtype != x.dtype:
        res = torch.mm(x, weight.t(), out_dtype=out_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is not None:
        return torch.mm(x, weight.t(), out=out)
    return torch.mm(x, weight.t())
