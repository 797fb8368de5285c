"""The step function: runs a batch of (request, next tokens) from the cache.

It takes the place of the reference's ``Qwen2ModelRunner.forward`` together
with the cache allocation that the reference does inside layer 0
(``litelang/models/qwen2/model.py:123-126``, ``qwen2/layer/transformer_layer.py:
53-60``).  Differences: the pages of a step are reserved *before* it is launched
(by the scheduler or the replay tool, through the cache manager), a step may mix
portions of prompts with single decoded tokens, nothing between the upload of
the index arrays and the logits waits for the host, and the result is the
float32 logits at the wanted places, not token ids.

Steps made of single-token entries only are captured in CUDA graphs, one per
batch-size bucket, and replayed; everything a captured step reads (index
arrays, block tables, cache) sits at fixed addresses.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..csrc.build import load_library
from .batch import BatchBuilder, StepBatch, StepEntry
from .model import CausalLM

_STATUS_TEXT = {
    1: "a token id outside the vocabulary",
    2: "a cache slot outside the pool",
    3: "a block-table entry outside the pool",
    4: "a position outside the position table",
    5: "a bounded wait inside a kernel (TMA or tensor-core pipeline) that ran out",
    6: "a shared-memory window that is not aligned as the kernel needs",
    7: "tensor memory of a pair of CTAs that is not at the same columns in both",
}


class KernelStatusError(RuntimeError):
    pass


def _buckets(limit: int) -> List[int]:
    out, b = [], 1
    while b < limit:
        out.append(b)
        b *= 2
    out.append(limit)
    return out


class ModelRunner:
    def __init__(self, model: CausalLM, manager: CacheManager, device: torch.device, max_tokens_per_step: int,
                 cuda_graphs: bool = True):
        if device.type != "cuda":
            raise RuntimeError("lite_lang_b200 runs on a CUDA device only; there is no CPU path")
        self.model = model
        self.manager = manager
        self.device = device
        ops.configure_matmul_precision()
        for lib in model.kernel_libraries():
            load_library(lib)
        self.storage = CacheStorage(manager, model.dtype, device)
        # last element: the kernels' status word; the rest: sampled tokens (see sampling/)
        self.result_buf = torch.zeros(manager.max_requests + 1, dtype=torch.int32, device=device)
        self.status = self.result_buf[manager.max_requests:]
        self._timeline = None
        if ops.timeline_build():
            # a timeline build's kernels write their time stamps behind the status word, which then heads a
            # buffer of its own (kernels that are given no status word find it through ops)
            self._timeline = torch.zeros(4 + 2 * ops.TIMELINE_SLOTS, dtype=torch.int32, device=device)
            self.status = self._timeline[:1]
            ops.TIMELINE_STATUS = self.status
        self.builder = BatchBuilder(manager, max_tokens_per_step, manager.max_requests, device, self.status)
        self.single_builder = BatchBuilder(manager, manager.max_requests, manager.max_requests, device, self.status)
        self.use_graphs = bool(cuda_graphs)
        self._graphs: Dict[tuple, tuple] = {}     # (batch bucket, class of context length) -> (graph, logits)
        self._graph_pool = None
        self.graph_kernel_launches: Dict[int, int] = {}   # hand-written kernels inside each captured step
        self._bucket_list = _buckets(manager.max_requests)
        # A captured step's kernels are planned (splits of the keys, warps) for the longest context that may be
        # replayed through the graph; a plan for tens of thousands of keys does not suit a short context and the
        # other way round, so a batch size has a graph per class of context length: up to 8,192 tokens (where the
        # plans do not differ), up to 16,384, 32,768, ...
        self._context_classes = [c for c in (1 << k for k in range(13, 31)) if c < manager.max_model_len]
        self._context_classes.append(manager.max_model_len)
        self.steps_run = 0
        self.graph_replays = 0

    # ------------------------------------------------------------------
    def reserve(self, slot: int, new_tokens: int) -> bool:
        """Make room for ``new_tokens`` more tokens of the request in ``slot``."""
        return self.manager.reserve(slot, self.manager.length(slot) + new_tokens)

    def step(self, entries: Sequence[StepEntry], allow_graph: bool = True) -> Optional[torch.Tensor]:
        """Run one step.  Pages must have been reserved.  Returns float32 logits
        [wanted, vocab] in the order of the entries and of their ``want`` lists (None if
        nothing is wanted).  The tensor is valid until the next step."""
        entries = list(entries)
        m = self.manager
        self.storage.sync()      # (the batch builder refuses tokens whose pages were not reserved)
        single = all(len(e.tokens) == 1 for e in entries)
        if single and self.use_graphs and allow_graph:
            logits = self._step_graph(entries)
        else:
            batch = self.builder.build(entries)
            if batch.has_feed:
                ops.feed_tokens(batch.token_ids, batch.feed, self.result_buf[:m.max_requests])
            logits = self.model.forward(batch, self.storage)
        for e in entries:
            m.advance(e.slot, m.length(e.slot) + len(e.tokens))
        self.steps_run += 1
        return logits

    # ------------------------------------------------------------------
    def _bucket(self, n: int) -> int:
        for b in self._bucket_list:
            if b >= n:
                return b
        return self._bucket_list[-1]

    def _context_class(self, longest: int) -> int:
        for c in self._context_classes:
            if c >= longest:
                return c
        return self._context_classes[-1]

    def _capture(self, bucket: int, context: Optional[int] = None):
        context = self.manager.max_model_len if context is None else context
        batch = self.single_builder.build([], pad_entries=bucket)
        batch.max_kv_len = context
        batch.captured = True
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        results = self.result_buf[:self.manager.max_requests]
        with torch.cuda.stream(side):
            for _ in range(2):
                ops.feed_tokens(batch.token_ids, batch.feed, results)
                self.model.forward(batch, self.storage)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        from ..csrc import build as _build
        before = _build.LAUNCHES
        with torch.cuda.graph(graph, pool=self._graph_pool):
            # tokens that the host has not seen yet come from the last step's sampled results
            ops.feed_tokens(batch.token_ids, batch.feed, results)
            logits = self.model.forward(batch, self.storage)
        self.graph_kernel_launches[bucket] = _build.LAUNCHES - before
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        self._graphs[(bucket, context)] = (graph, logits)
        return self._graphs[(bucket, context)]

    def capture_all(self) -> None:
        """Capture every bucket and class of context length now (largest first, so that the pool is sized once)."""
        if not self.use_graphs:
            return
        for b in sorted(self._bucket_list, reverse=True):
            for c in sorted(self._context_classes, reverse=True):
                if (b, c) not in self._graphs:
                    self._capture(b, c)

    def _step_graph(self, entries: List[StepEntry]) -> Optional[torch.Tensor]:
        bucket = self._bucket(len(entries))
        m = self.manager
        context = self._context_class(max(m.length(e.slot) for e in entries) + 1)
        got = self._graphs.get((bucket, context))
        if got is None:
            got = self._capture(bucket, context)
        graph, logits = got
        batch = self.single_builder.build(entries, pad_entries=bucket, views=False)
        graph.replay()
        self.graph_replays += 1
        if batch.real_logits == 0:
            return None
        return logits[:batch.real_logits]

    # ------------------------------------------------------------------
    def timeline(self):
        """A timeline build's time stamps of the last layer of the last step, in microseconds from the first
        stamp: {kernel name: float array [CTAs that ran, 4 events]} with the events started, released (the wait
        for the kernel before is over), done, and for the attention the end of its tile loop; 0 where a CTA wrote
        none.  None in an ordinary build."""
        if self._timeline is None:
            return None
        import numpy as np
        raw = self._timeline[4:].cpu().numpy().view(np.uint64).reshape(len(ops.TIMELINE_KERNELS), -1, 4)
        t0 = raw[raw > 0].min() if (raw > 0).any() else 0
        out = {}
        for name, block in zip(ops.TIMELINE_KERNELS, raw):
            ran = block[block[:, 0] > 0]
            if len(ran):
                out[name] = np.where(ran > 0, (ran.astype(np.int64) - np.int64(t0)) / 1000.0, 0.0)
        return out

    def check_status(self) -> None:
        """Raise if a kernel met an index out of range (synchronises)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise KernelStatusError(f"a kernel reported {_STATUS_TEXT.get(code, code)}")
