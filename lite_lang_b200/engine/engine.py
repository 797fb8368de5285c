"""The Python entry point: a model folder (or random weights) to generated tokens.

The reference has no offline entry point; its de-facto API is the benchmark
script ``test/generate_token.py:24-67`` (config, runner, ``init_model``, a batch,
a loop of forwards) and the HTTP manager ``litelang/apis/http_server_manager.py:
12-63``.  ``Engine`` does what those do between a prompt's tokens and its new
tokens: it builds the model chosen by config.json, sizes the cache from free
memory (``mem_usage``, as ``litelang/models/cache.py:218-223``) or from an
explicit page count, and ``generate`` drives the scheduler to completion.
"""

from __future__ import annotations

import os
import time
from typing import Dict, List, Optional, Sequence, Union

import torch

from .. import models as _models  # noqa: F401  (registers the architectures)
from ..cache.manager import CacheManager
from ..cache.sizing import plan_pages
from ..config.base import ModelConfig, load_config
from ..config.engine import EngineConfig
from ..sampling.sampler import Sampler, SamplingParams, uniform_for
from ..weights.loader import load_weights
from ..weights.random_init import random_fetch
from .batch import StepEntry
from .model import CausalLM
from .runner import ModelRunner
from .scheduler import RUNNING, PlannedEntry, Request, Scheduler

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class _Launched:
    """A step that is on the stream: its plan and where its results arrive."""

    __slots__ = ("plan", "rows", "host", "event")

    def __init__(self, plan, rows, host, event):
        self.plan, self.rows, self.host, self.event = plan, rows, host, event


class Engine:
    def __init__(self, model_path: Optional[str] = None, engine_config: Optional[EngineConfig] = None, *,
                 config: Optional[ModelConfig] = None, random_seed: Optional[int] = None,
                 device: str = "cuda:0"):
        """Load ``model_path`` (config.json + safetensors), or build ``config`` with random
        weights drawn on the device from ``random_seed`` (no folder is written)."""
        self.cfg = engine_config or EngineConfig()
        if not torch.cuda.is_available():
            raise RuntimeError("lite_lang_b200 needs a CUDA device (B200, sm_100a); none is visible")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        if model_path is not None:
            self.model_config = load_config(model_path)
        elif config is not None:
            self.model_config = config
        else:
            raise ValueError("give a model_path or a config")
        self.model_path = model_path
        self.dtype = _TORCH_DTYPE[self.cfg.dtype]
        spec = self.model_config.model_spec()
        self.model = CausalLM(spec)
        if model_path is not None and random_seed is None:
            load_weights(self.model, model_path, self.dtype, self.device)
        else:
            seed = 0 if random_seed is None else random_seed
            fetch = random_fetch(self.model, seed, self.model_config.init_scales(), torch.bfloat16,
                                 device=str(self.device))
            self.model.load(fetch, self.dtype, self.device)
        self.max_model_len = min(self.cfg.model_len, spec.max_positions)
        n_paged = sum(1 for g in self.model.cache_groups if g.kind == "paged")
        if self.cfg.num_pages is not None:
            pages = [self.cfg.num_pages] * n_paged
        else:
            # a share of the free memory, less the fixed-size state records, shared out over the groups
            torch.cuda.synchronize(self.device)
            free, _total = torch.cuda.mem_get_info(self.device)
            pages = plan_pages(self.model.cache_groups, int(free * self.cfg.mem_usage), self.cfg.page_size,
                               2 if self.dtype == torch.bfloat16 else 4, self.cfg.max_batch_size, self.max_model_len,
                               self.cfg.max_tokens_per_step)
        self.manager = CacheManager(self.model.cache_groups, pages, self.cfg.page_size,
                                    self.cfg.max_batch_size, self.max_model_len)
        self.runner = ModelRunner(self.model, self.manager, self.device, self.cfg.max_tokens_per_step,
                                  self.cfg.cuda_graphs)
        self.sampler = Sampler(self.device, self.cfg.max_batch_size, out=self.runner.result_buf)
        self.scheduler = Scheduler(self.manager, self.cfg.max_tokens_per_step, self.cfg.max_reqs,
                                   self.cfg.busy_scale, self.cfg.preempt_strategy, self.cfg.max_output_length)
        self._next_id = 0
        self._tokenizer = None
        # results of up to two steps in flight (tokens and the status word), read one step at a time
        self._result_hosts = [torch.zeros(self.cfg.max_batch_size + 1, dtype=torch.int32, pin_memory=True)
                              for _ in range(3)]
        self._result_events = [torch.cuda.Event() for _ in self._result_hosts]
        self._result_turn = 0
        self._ahead: Optional[_Launched] = None
        self.host_wait_s = 0.0          # seconds the host has spent waiting for steps' results
        self._pipeline = os.environ.get("LITE_LANG_B200_PIPELINE", "1") != "0"

    # ------------------------------------------------------------------
    def tokenizer(self):
        """The folder's tokenizer (only needed when prompts are text)."""
        if self._tokenizer is None:
            if self.model_path is None:
                raise RuntimeError("text prompts need a model folder with a tokenizer")
            from transformers import AutoTokenizer
            self._tokenizer = AutoTokenizer.from_pretrained(self.model_path)
        return self._tokenizer

    def add_request(self, prompt: Union[str, Sequence[int]], params: Optional[SamplingParams] = None) -> Request:
        params = params or SamplingParams()
        if isinstance(prompt, str):
            prompt = self.tokenizer().encode(prompt)
        prompt = [int(t) for t in prompt]
        if len(prompt) > self.cfg.max_input_length:
            raise ValueError(f"a prompt of {len(prompt)} tokens exceeds max_input_length {self.cfg.max_input_length}")
        vocab = self.model.spec.vocab_size
        if any(t < 0 or t >= vocab for t in prompt):
            raise ValueError("a prompt token lies outside the vocabulary")
        max_new = params.max_new_tokens if params.max_new_tokens is not None else self.cfg.max_output_length
        req = Request(self._next_id, prompt, params, max_new, tuple(self.model.spec.eos_token_ids))
        self._next_id += 1
        if not self.scheduler.add(req):
            raise RuntimeError(f"the waiting queue is full (max_reqs = {self.cfg.max_reqs})")
        return req

    def step(self) -> List[Request]:
        """One scheduler step: plan, run, sample, commit.  Returns the requests that finished.

        While the step's kernels run, the step after it is launched as well whenever the scheduler
        can decide it without this step's tokens (``Scheduler.plan_ahead``: a pure decode step);
        its token ids are taken on the device from this step's sampled tokens.  So the GPU does not
        wait for the host between decode steps.  A request that ends with this step's token (an eos
        id) is simply ignored in the step that was launched ahead."""
        cur = self._ahead
        self._ahead = None
        if cur is not None and not any(p.request.status == RUNNING for p in cur.plan):
            cur = None                       # everyone in it has ended meanwhile: nothing to collect
        if cur is None:
            plan = self.scheduler.plan()
            if not plan:
                if self.scheduler.has_work():
                    raise RuntimeError("the scheduler has work but could plan nothing")
                return []
            cur = self._launch(plan, 0)
        if self.cfg.cuda_graphs and self._pipeline:
            nxt = self.scheduler.plan_ahead(cur.plan)
            if nxt is not None:
                self._ahead = self._launch(nxt, 1)
        return self._collect(cur)

    def _launch(self, plan: List[PlannedEntry], ahead: int) -> "_Launched":
        """Put a planned step on the stream: model, sampling, copy of the results to the host."""
        entries = []
        for p in plan:
            toks = [0] if p.feed >= 0 else p.request.token_slice(p.start, p.count)
            entries.append(StepEntry(p.request.slot, toks, (p.count - 1,) if p.samples else (), p.feed))
        logits = self.runner.step(entries)
        rows = [i for i, p in enumerate(plan) if p.samples]
        if rows:
            temps, unis = [], []
            for i in rows:
                r = plan[i].request
                greedy = r.params.greedy
                temps.append(0.0 if greedy else float(r.params.temperature))
                seed = r.params.seed if r.params.seed is not None else self.cfg.seed
                # (a step launched ahead samples the token after the one that is still on its way)
                unis.append(0.0 if greedy else uniform_for(seed, r.id, len(r.output) + ahead))
            self.sampler.sample(logits, temps, unis)
        # one copy brings the sampled tokens and the kernels' status word
        turn = self._result_turn
        self._result_turn = (turn + 1) % len(self._result_hosts)
        host = self._result_hosts[turn]
        host.copy_(self.runner.result_buf, non_blocking=True)
        self._result_events[turn].record()
        return _Launched(plan, rows, host, self._result_events[turn])

    def _collect(self, launched: "_Launched") -> List[Request]:
        if not launched.event.query():
            t0 = time.perf_counter()
            launched.event.synchronize()
            self.host_wait_s += time.perf_counter() - t0
        host = launched.host.numpy()
        if host[-1] != 0:
            self.runner.check_status()
        sampled: List[Optional[int]] = [None] * len(launched.plan)
        for k, i in enumerate(launched.rows):
            sampled[i] = int(host[k])
        return self.scheduler.commit(launched.plan, sampled)

    def generate(self, prompts: Sequence[Union[str, Sequence[int]]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[List[int]]:
        """New tokens for each prompt (token ids in, token ids out), in the order given."""
        if params is None or isinstance(params, SamplingParams):
            plist = [params or SamplingParams()] * len(prompts)
        else:
            plist = list(params)
            if len(plist) != len(prompts):
                raise ValueError("one SamplingParams per prompt is needed")
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        while self.scheduler.has_work():
            self.step()
        return [list(r.output) for r in reqs]

    def generate_text(self, prompts: Sequence[str], params=None) -> List[str]:
        outs = self.generate(prompts, params)
        tok = self.tokenizer()
        return [tok.decode(o) for o in outs]

    def stats(self) -> Dict[str, int]:
        d = dict(self.scheduler.counters)
        d.update(pages_handed_out=self.manager.pages_handed_out, pages_reused=self.manager.pages_reused,
                 graph_replays=self.runner.graph_replays, steps_run=self.runner.steps_run)
        return d


def generate(model_path: str, prompts, params=None, engine_config: Optional[EngineConfig] = None):
    """One-call form: build an engine for ``model_path`` and generate."""
    return Engine(model_path, engine_config).generate(prompts, params)
