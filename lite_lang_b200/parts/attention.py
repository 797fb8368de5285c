"""Grouped-query attention over the paged cache, with q/k/v bias.

Per layer (``litelang/models/qwen2/layer/transformer_layer.py:94-194``):
q|k|v projection with bias, rotation of q and k, k and v written to the
request's cache, attention of each new token over the request's cached keys
(query head a uses kv head a // group, scores scaled by head_dim^-1/2, causal),
output projection without bias.  The reference fuses k and v only
(``layer_weights/load_weights.py:110-116``); here q, k and v are one projection.

Differences that come with this engine: any number of new tokens per request in
one step (portions of prompts beside decoded tokens), pages of ``page_size``
tokens instead of one token (``litelang/models/cache.py:138``), bias added and
rotation done in float32 in one kernel that also writes the cache, and an
optional window of the last ``window`` positions.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import Mixer, NormSplit, PagedKVNeed, TensorDecl, build_part, register_part


class GQAttention(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.out_bias = bool(p.get("out_bias", False))
        self.scale = float(p.get("scale", self.head_dim ** -0.5))
        self.window = p.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("gqa_attention: num_heads must be a multiple of num_kv_heads")
        if self.out_bias:
            raise ValueError("gqa_attention: a bias on the output projection is not built")
        pos = p.get("position")
        self.position = build_part("position", pos) if pos is not None else None
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.w_qkv = None
        self.b_qkv = None
        self.w_o = None

    def tensors(self) -> Dict[str, TensorDecl]:
        h = self.hidden_size
        d = {
            "q_proj.weight": TensorDecl((self.q_width, h)),
            "k_proj.weight": TensorDecl((self.kv_width, h)),
            "v_proj.weight": TensorDecl((self.kv_width, h)),
            "o_proj.weight": TensorDecl((h, self.q_width)),
        }
        if self.qkv_bias:
            d["q_proj.bias"] = TensorDecl((self.q_width,), "bias")
            d["k_proj.bias"] = TensorDecl((self.kv_width,), "bias")
            d["v_proj.bias"] = TensorDecl((self.kv_width,), "bias")
        return d

    def load(self, fetch, dtype, device) -> None:
        w = [fetch(n).to(dtype) for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight")]
        self.w_qkv = torch.cat(w, dim=0).to(device).contiguous()
        if self.qkv_bias:
            b = [fetch(n).to(torch.float32) for n in ("q_proj.bias", "k_proj.bias", "v_proj.bias")]
            self.b_qkv = torch.cat(b, dim=0).to(device).contiguous()
        self.w_o = fetch("o_proj.weight").to(dtype).to(device).contiguous()

    def weight_bytes(self) -> int:
        n = self.w_qkv.numel() * self.w_qkv.element_size() + self.w_o.numel() * self.w_o.element_size()
        if self.b_qkv is not None:
            n += self.b_qkv.numel() * 4
        return n

    def cache_need(self):
        return PagedKVNeed(self.num_kv_heads, self.head_dim, self.window)

    def kernel_libraries(self):
        libs = ["core"]
        if self.w_qkv is not None and self.w_qkv.dtype == torch.bfloat16:
            libs.extend(["gemm_smallm", "gemm_stream", "gemm_tc", "gemm_pair"])
            if self.head_dim in (64, 128):
                libs.extend(["attn_mma", "attn_tc"])
        return libs

    def prepare(self, device, dtype) -> None:
        if self.position is not None:
            self.position.prepare(device)

    # ------------------------------------------------------------------
    accumulates = True
    splits_norm = True

    def _project_out(self, attn, residual, into_norm=None, status=None):
        if residual is not None and ops.accumulate_preferred(attn, self.w_o):
            ops.linear_accumulate(attn, self.w_o, residual)
            return None
        if (residual is not None and into_norm is not None and ops.into_norm_supported(attn, self.w_o, residual)
                and into_norm.accepts(residual)):
            # decode: the o projection adds into the residual stream and leaves the norm after it to the next product
            u, sumsq = ops.gemm_stream_into_norm(attn, self.w_o, residual, into_norm.weight, status)
            return NormSplit(u, sumsq, into_norm.eps)
        return ops.linear(attn, self.w_o, partial_ok=True)

    def forward(self, x, step, cache, residual=None, into_norm=None):
        n = x.shape[0]
        slot_map = cache.slot_map if cache.writable else None
        if (self.position is not None and self.position.fuses_with_store
                and ops.qkv_rope_supported(x, self.w_qkv, self.head_dim, self.position.fused_table().shape[1])):
            # decode: projection, bias, rotation and cache write in one kernel; only q is materialised
            q = torch.empty((n, self.q_width), dtype=x.dtype, device=x.device)
            ops.gemm_stream_qkv_rope(q, x, self.w_qkv, self.b_qkv, step.positions, self.position.fused_table(),
                                     self.num_heads, self.num_kv_heads, self.head_dim, slot_map, cache.k, cache.v,
                                     cache.page_size, step.status)
            attn = torch.empty((n, self.q_width), dtype=x.dtype, device=x.device)
            self.attend(attn, q, step, cache)
            return self._project_out(attn, residual, into_norm, step.status)
        if (self.position is not None and self.position.fuses_with_store
                and ops.pair_qkv_supported(x, self.w_qkv, self.head_dim, self.position.fused_table().shape[1])
                and ops.pair_qkv_preferred(x, self.w_qkv)):
            # portions of prompts: the same fusion on the two-SM tcgen05 kernel
            q = torch.empty((n, self.q_width), dtype=x.dtype, device=x.device)
            ops.gemm_pair_qkv_rope(q, x, self.w_qkv, self.b_qkv, step.positions, self.position.fused_table(),
                                   self.num_heads, self.num_kv_heads, self.head_dim, slot_map, cache.k, cache.v,
                                   cache.page_size, step.status)
            attn = torch.empty((n, self.q_width), dtype=x.dtype, device=x.device)
            self.attend(attn, q, step, cache)
            return self._project_out(attn, residual, into_norm, step.status)
        qkv = ops.linear(x, self.w_qkv)
        if self.position is None or self.position.fuses_with_store:
            table = self.position.fused_table() if self.position is not None else None
            ops.bias_rope_store(qkv, self.b_qkv, step.positions, table, self.num_heads, self.num_kv_heads,
                                self.head_dim, slot_map, cache.k, cache.v, cache.page_size, step.status, n)
        else:
            if self.b_qkv is not None:
                ops.bias_rope_store(qkv, self.b_qkv, None, None, self.num_heads, self.num_kv_heads, self.head_dim,
                                    None, None, None, cache.page_size, step.status, n)
            self.position.apply(qkv, step.positions, self.num_heads, self.num_kv_heads, self.head_dim, n)
            if slot_map is not None:
                ops.bias_rope_store(qkv, None, None, None, self.num_heads, self.num_kv_heads, self.head_dim,
                                    slot_map, cache.k, cache.v, cache.page_size, step.status, n)
        attn = torch.empty((n, self.q_width), dtype=x.dtype, device=x.device)
        self.attend(attn, qkv, step, cache)
        return self._project_out(attn, residual, into_norm, step.status)

    def _plan_mma(self, step, entries, max_kv_len, sms):
        """Row blocks, splits and warps of the decode kernel for ``entries`` single-token entries on a
        device of ``sms`` SMs."""
        group = self.num_heads // self.num_kv_heads
        if self.window:
            max_kv_len = min(max_kv_len, int(self.window) + 16)     # (the keys a token of a windowed layer may see)
        max_tiles = (max_kv_len + 15) // 16
        if group <= 8:
            # attn_decode: one CTA per (entry, kv head, split).  Measured on a B200 (148 SMs; 1.5B sizes, context
            # 2k, batch 1..64): about 7/8 of the SMs in CTAs are best, as splits of 8, 4, 2 or none, with at least 8 tiles
            # (128 keys) a split; 8 warps a CTA, except that many clusters of 8 such CTAs do not find room
            # side by side (batch 8: 4 warps 1.19 ms a step, 8 warps 1.32 ms).  The same choices were the best or
            # within 1 % of it at context 8k (batch 2 and 8).
            base = entries * self.num_kv_heads
            most = (sms * 7) // 8
            # Few requests with long contexts: a cluster takes 8 splits at most, which leaves most SMs without work
            # and every CTA with thousands of keys.  Beyond 8,192 tokens a (entry, kv head) gets several clusters of
            # 4 CTAs instead, each with a range of the keys, which meet through scratch memory: about 7/8 of the
            # SMs in CTAs again, with at least 16 tiles a CTA at 3/4 of the longest context that the plan is for (a
            # captured step's plan serves a class of context lengths).  Kernel alone, batch 1: context 8k 12.2 ->
            # 8.3 us, 16k 20.5 -> 10.8, 32k 37.2 -> 13.5; in a step (CTAs of 128 KB, which the products around
            # them do not sit beside) it pays from about 8k on: batch 1 at 16k 1.37 -> 1.24 ms, at 30k 1.83 -> 1.29.
            if max_tiles > (512 if base <= 4 else 1024):     # (four requests: from 16k on; at 9k 1.24 -> 1.25 ms)
                nouter = 1
                while base * 4 * (2 * nouter) <= most and (max_tiles * 3 // 4) // (4 * 2 * nouter) >= 16:
                    nouter *= 2
                if nouter >= 4:
                    return entries, 4, True, 8, nouter
            nsplit = 1
            for n in (8, 4, 2):
                if base * n <= most and n <= max(1, max_tiles // 8):
                    nsplit = n
                    break
            warps = 4 if (nsplit == 8 and base * nsplit > most // 2) else 8
            return entries, nsplit, True, warps, 1
        blocks = entries * ((group + 15) // 16)
        ctas = blocks * self.num_kv_heads
        # attn_mma: one wave of CTAs at most, and at least 8 tiles (128 keys) a split: with less, merging the
        # splits costs more than the split saves.  The splits of a row block form a thread-block cluster
        # and merge through distributed shared memory: no scratch memory, no counters.
        want = max(1, min((2 * sms) // ctas, max(1, max_tiles // 8)))
        # (clusters of 16, the non-portable size, were measured slower than 8: placement costs more
        # than the shorter key ranges save)
        nsplit = 8 if want >= 8 else 4 if want >= 4 else 2 if want >= 2 else 1
        # 8 warps a CTA when the step has very few row blocks: more warps to hide instruction latency
        # behind.  Not beyond half the SMs: 8-warp CTAs fit one an SM, and clusters of 8 of them then
        # no longer find room in one wave
        warps = 8 if ctas * nsplit <= sms // 2 and max_tiles >= 16 * nsplit else 4
        return blocks, nsplit, group <= 16, warps, 0

    def attend(self, out, qkv, step, cache) -> None:
        """Attention of the step's tokens over the cache plane; picks the kernels by shape.

        Single-token entries come first in a step: they go to the decode kernel (keys split over a
        cluster of CTAs), the portions of prompts after them to a prefill kernel (128 query rows a
        CTA share the keys: the tcgen05 one where it takes the shape, else the mma.sync one)."""
        if ops.attn_mma_supported(qkv.dtype, self.head_dim, cache.page_size, qkv.stride(0)):
            n_single = step.num_single
            n_rest = step.num_entries - n_single
            args = (self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size, self.window, self.scale)
            if n_single > 0:
                key = ("attn_mma", self.num_heads, self.num_kv_heads, self.head_dim)
                plan = step.scratch.get(key)
                if plan is None:
                    plan = step.scratch[key] = self._plan_mma(step, n_single, step.max_kv_len, ops.sm_count(qkv.device))
                blocks, nsplit, single, warps, nouter = plan     # (nouter 0: groups of more than 8 heads, attn_mma)
                if nouter >= 1:
                    # keys on the M side, the group's heads on the N side of the MMA: half the work a tile
                    ops.attn_decode(out, qkv, qkv.stride(0), cache.k, cache.v, cache.block_table, step.ctx_len,
                                    step.req_slot, n_single, *args, nsplit, step.status, warps=warps, nouter=nouter)
                else:
                    ops.attn_mma(out, qkv, qkv.stride(0), cache.k, cache.v, cache.block_table, step.cu_q,
                                 step.ctx_len, step.req_slot, n_single, blocks, *args, nsplit, None, None,
                                 step.status, all_single=single, cluster=nsplit > 1, warps=warps)
            if n_rest > 0:
                group = self.num_heads // self.num_kv_heads
                rest = (step.cu_q[n_single:], step.ctx_len[n_single:], step.req_slot[n_single:], n_rest)
                if ops.TC_ENABLED and ops.attn_prefill_tc_supported(qkv.dtype, self.head_dim, cache.page_size,
                                                                    qkv.stride(0), group):
                    # tcgen05: S and O in tensor memory, K and V page by page through TMA
                    key = ("attn_prefill_tc", group, self.window)
                    plan = step.scratch.get(key)
                    if plan is None:
                        ctxs = getattr(step, "entry_ctx", None)
                        rest_entries = step.entries[n_single:]
                        if ctxs is not None:
                            plan = ops.attn_prefill_tc_plan(
                                [(ctxs[n_single + i], len(e.tokens)) for i, e in enumerate(rest_entries)], group,
                                self.window, self.num_kv_heads, 2 * ops.sm_count(qkv.device))
                        else:
                            blocks = ops.attn_prefill_tc_blocks((len(e.tokens) for e in rest_entries), group)
                            plan = (blocks, ops.attn_prefill_tc_splits(blocks, self.num_kv_heads, qkv.device), 8)
                        step.scratch[key] = plan
                    ops.attn_prefill_tc(out, qkv, qkv.stride(0), cache.k, cache.v, cache.block_table, *rest, plan[0],
                                        *args, step.status, nsplit=plan[1], split_len=plan[2])
                else:
                    key = ("attn_prefill", group)
                    blocks = step.scratch.get(key)
                    if blocks is None:
                        blocks = sum((len(e.tokens) * group + 127) // 128 for e in step.entries[n_single:])
                        step.scratch[key] = blocks
                    ops.attn_prefill(out, qkv, qkv.stride(0), cache.k, cache.v, cache.block_table, *rest, blocks,
                                     *args, step.status)
            return
        ops.paged_attention_generic(out, qkv, qkv.stride(0), cache.k, cache.v, cache.block_table, step.token_req,
                                    step.req_slot, step.positions, qkv.shape[0], self.num_heads, self.num_kv_heads,
                                    self.head_dim, cache.page_size, self.window, self.scale, step.status)


register_part("mixer", "gqa_attention", GQAttention)
