#!/usr/bin/env python3
"""Measurement of the engine on one B200: decode tokens a second and a 2,048-token prefill.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The model has the layer sizes of Qwen2-1.5B (28 layers, hidden 1536, 12/2 heads of
128, intermediate 8960, vocabulary 151936, tied embeddings) with random bfloat16
weights; prompts are seeded uniform-random token ids.  A *step* is one decode step
of a batch of 8 requests that each hold a 2,048-token prompt and decode towards a
context of 4,096.  One JSON line is printed:

  value      decoded tokens a second, timed on the device with CUDA events around K
             steps (index arrays are uploaded every step, tokens are not read back);
  e2e        the same through the Python entry point (scheduler, sampling, token ids
             from the host and back to it every step);
  prefill    one request of 2,048 tokens in one step, logits of its last token: median and minimum over at
             least 20 repeats (about a second of them), with the SM clock sampled meanwhile;
  roofline   bytes a decode step has to read (every weight once, the cache of the live
             requests) over its time, against the measured copy bandwidth;
  points     decode at batch 1 and 64, on the device and through the entry point; host_ms: what the host
             spends a step (scheduler, batch, launches) while not waiting for the device;
  workloads  the two serving workloads named beside the headline configuration, through the scheduler.

A decode step reads about 3.1 GB of weights, far more than the 126 MB L2, so
iterations need no L2 flush.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN2_1P5B = dict(architectures=["Qwen2ForCausalLM"], hidden_size=1536, num_hidden_layers=28,
                  num_attention_heads=12, num_key_value_heads=2, intermediate_size=8960, vocab_size=151936,
                  rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                  max_position_embeddings=32768, use_sliding_window=False, torch_dtype="bfloat16")
PROMPT_LEN = 2048
CONTEXT = 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as fh:
                d = json.load(fh)
            out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in d:
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (read-only queries)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="lite_lang_b200_clocks_", suffix=".csv")
            self.fh = os.fdopen(fd, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=self.fh,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as fh:
            lines = fh.readlines()
        try:
            os.remove(self.path)
        except OSError:
            pass
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def build_engine(layers, max_batch, dtype="bfloat16", model=None):
    import torch
    from lite_lang_b200 import Engine, EngineConfig
    from lite_lang_b200.config import config_from_dict

    cfg = config_from_dict(dict(model or QWEN2_1P5B, num_hidden_layers=layers))
    pages_per_req = (CONTEXT + 15) // 16
    ecfg = EngineConfig(dtype=dtype, page_size=16, num_pages=max_batch * pages_per_req + 8,
                        max_batch_size=max_batch, max_input_length=PROMPT_LEN, max_output_length=CONTEXT - PROMPT_LEN,
                        max_model_len=CONTEXT, max_tokens_per_step=2048, cuda_graphs=True, seed=0)
    engine = Engine(config=cfg, engine_config=ecfg, random_seed=1234)
    engine.runner.capture_all()        # every batch-size bucket's decode step, before anything is timed
    return engine


def random_prompts(n, length, vocab, seed):
    import numpy as np
    rng = np.random.default_rng(seed)
    return [[int(t) for t in rng.integers(0, vocab, size=length)] for _ in range(n)]


def kv_bytes_per_token(engine):
    n = 0
    for g in engine.model.cache_groups:
        if g.kind == "paged":
            n += g.planes * 2 * g.num_kv_heads * g.head_dim * 2
    return n


def prefill_flops(cfg, tokens):
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    per_layer = cfg.hidden_size * qkv + cfg.num_attention_heads * cfg.head_dim * cfg.hidden_size \
        + 3 * cfg.hidden_size * cfg.intermediate_size
    linear = 2 * tokens * cfg.num_hidden_layers * per_layer
    attn = 2 * tokens * tokens * cfg.num_attention_heads * cfg.head_dim * cfg.num_hidden_layers   # causal: half of 4 T^2
    head = 2 * cfg.hidden_size * cfg.vocab_size
    return linear + attn + head


def device_decode(engine, batch, steps, warmup, sampler_on=True):
    """K decode steps of `batch` requests, timed on the device.  Returns (ms per step, mean context)."""
    import torch
    from lite_lang_b200.engine.batch import StepEntry

    m, runner = engine.manager, engine.runner
    vocab = engine.model.spec.vocab_size
    prompts = random_prompts(batch, PROMPT_LEN, vocab, 7)
    slots = []
    for p in prompts:                                   # prefill, untimed
        s = m.open()
        assert s is not None and runner.reserve(s, PROMPT_LEN)
        for c0 in range(0, PROMPT_LEN, 2048):           # in portions of the step's token limit
            runner.step([StepEntry(s, p[c0:c0 + 2048], ())])
        slots.append(s)
    torch.cuda.synchronize()
    toks = random_prompts(1, steps + warmup, vocab, 9)[0]

    def one(i):
        entries = []
        for s in slots:
            assert runner.reserve(s, 1)
            entries.append(StepEntry(s, [toks[i]], (0,)))
        logits = runner.step(entries)
        if sampler_on:
            engine.sampler.sample(logits, [0.0] * batch, [0.0] * batch)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    ctx0 = m.length(slots[0])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(warmup, warmup + steps):
        one(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    ctx1 = m.length(slots[0])
    runner.check_status()
    for s in slots:
        m.close(s)
    return ms, (ctx0 + ctx1) / 2.0


def e2e_decode(engine, batch, steps, warmup):
    """The same through Engine.step(): scheduler, sampling, tokens to the host every step.
    Returns tokens a second, bytes up and down a step, ms a step, and the host's own ms a step (wall clock
    less the time it waited for the device)."""
    import torch
    from lite_lang_b200 import SamplingParams

    vocab = engine.model.spec.vocab_size
    prompts = random_prompts(batch, PROMPT_LEN, vocab, 7)
    # (a prompt is admitted a step: the first request is `batch` tokens ahead of the last, and nobody may end
    # inside the timed steps)
    sp = SamplingParams(temperature=0.0, max_new_tokens=steps + warmup + batch + 8, ignore_eos=True)
    reqs = [engine.add_request(p, sp) for p in prompts]
    while any(len(r.output) < 1 + warmup for r in reqs):    # prefill and warm-up decode steps
        engine.step()
    torch.cuda.synchronize()
    n0 = sum(len(r.output) for r in reqs)
    wait0 = engine.host_wait_s
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    host_ms = (dt - (engine.host_wait_s - wait0)) / steps * 1e3
    n1 = sum(len(r.output) for r in reqs)
    while engine.scheduler.has_work():                      # drain: give the cache back
        for r in list(engine.scheduler.running):
            r.max_new_tokens = len(r.output) + 1
        engine.step()
    h2d = engine.runner.single_builder.total * 4
    d2h = engine._result_hosts[0].numel() * 4
    return (n1 - n0) / dt, h2d, d2h, dt / steps * 1e3, host_ms


def prefill_once(engine, repeats=20, seconds=1.0):
    """A 2,048-token prompt in one step, again and again: at least ``repeats`` times and for about ``seconds``,
    after three warm-ups, each timed with CUDA events; the SM clock is sampled meanwhile.  (The step reads
    3 GB of weights, far more than the L2 holds, so nothing is flushed between repeats.)"""
    import torch
    from lite_lang_b200.engine.batch import StepEntry

    m, runner = engine.manager, engine.runner
    prompt = random_prompts(1, PROMPT_LEN, engine.model.spec.vocab_size, 11)[0]

    def once():
        s = m.open()
        assert runner.reserve(s, PROMPT_LEN)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry(s, prompt, (PROMPT_LEN - 1,))])
        e1.record()
        torch.cuda.synchronize()
        m.close(s)
        return e0.elapsed_time(e1)

    for _ in range(3):
        once()
    clocks = ClockSampler()
    clocks.start()
    times = []
    t0 = time.perf_counter()
    while len(times) < repeats or (time.perf_counter() - t0 < seconds and len(times) < 400):
        times.append(once())
    clk = clocks.stop()
    return {"ms": statistics.median(times), "ms_min": min(times), "repeats": len(times), "clocks": clk}


def kernel_times(engine, batch, steps):
    """Mean duration of every kernel of a decode step, measured while the step's graph replays."""
    import collections
    import torch
    from torch.profiler import ProfilerActivity, profile
    from lite_lang_b200.engine.batch import StepEntry

    m, runner = engine.manager, engine.runner
    vocab = engine.model.spec.vocab_size
    slots = []
    for p in random_prompts(batch, PROMPT_LEN, vocab, 7):
        s = m.open()
        assert runner.reserve(s, PROMPT_LEN)
        runner.step([StepEntry(s, p, ())])
        slots.append(s)

    def one(i):
        for s in slots:
            assert runner.reserve(s, 1)
        logits = runner.step([StepEntry(s, [5 + i], (0,)) for s in slots])
        engine.sampler.sample(logits, [0.0] * batch, [0.0] * batch)

    for i in range(5):
        one(i)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for i in range(steps):
            one(5 + i)
        torch.cuda.synchronize()
    agg = collections.OrderedDict()
    for e in prof.events():
        if e.device_type == torch.autograd.DeviceType.CUDA:
            a = agg.setdefault(e.name[:72], [0, 0.0])
            a[0] += 1
            a[1] += e.device_time
    lines = [f"decode step of batch {batch}, mean over {steps} graph replays "
             f"(LITE_LANG_B200_PDL={os.environ.get('LITE_LANG_B200_PDL', '1')}; with 1 kernels overlap and their "
             "times include waiting for the kernel before)"]
    for k, (n, t) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        lines.append(f"{t / steps:9.1f} us/step {n / steps:6.1f} calls {t / n:8.2f} us each  {k}")
    lines.append(f"sum {sum(v[1] for v in agg.values()) / steps:.1f} us/step")
    for s in slots:
        m.close(s)
    return "\n".join(lines)


def layer_timeline(engine, batch, steps, warmup):
    """Decode steps of a timeline build (LITE_LANG_B200_TIMELINE=1: the kernels stamp %globaltimer), and a table of
    the last layer's products and attention: for each the earliest, median and latest CTA's start, release (its
    wait for the kernel before is over) and end, in microseconds from the q|k|v projection's release."""
    import numpy as np
    if engine.runner.timeline() is None:
        return "not a timeline build: set LITE_LANG_B200_TIMELINE=1 (the libraries are built a second time for it)"
    ms, ctx = device_decode(engine, batch, steps, warmup)
    tl = engine.runner.timeline()
    # only the CTAs of the last layer of the last step: a slot that this step's kernels did not write (another
    # kernel took the product, or it has fewer CTAs) still holds an older launch's stamps
    newest = max(float(ev[:, 2].max()) for ev in tl.values())
    tl = {name: ev[ev[:, 1] >= newest - 400.0] for name, ev in tl.items()}
    tl = {name: ev for name, ev in tl.items() if len(ev)}
    base = tl["qkv"][:, 1].min() if "qkv" in tl else min(float(ev[:, 1].min()) for ev in tl.values())
    lines = [f"batch {batch}, context {ctx:.0f}: {ms:.4f} ms a step with the stamps compiled in; us from q|k|v's release",
             f"{'kernel':10s} {'CTAs':>5s} | {'started: first median last':>27s} | {'released':>27s} | {'ended':>27s}"]

    def three(v):
        v = v[v > 0] - base
        return f"{v.min():8.2f} {np.median(v):8.2f} {v.max():8.2f}" if len(v) else " " * 26

    for name, ev in tl.items():
        lines.append(f"{name:10s} {len(ev):5d} | {three(ev[:, 0])}  | {three(ev[:, 1])}  | {three(ev[:, 2])}")
    if "attention" in tl and "qkv" in tl:
        ev = tl["attention"]
        late = ev[:, 0] - base > 0
        lines.append(f"attention: {int(late.sum())} of {len(ev)} CTAs started only after q|k|v's release; tile loop over "
                     f"at {np.median(ev[~late, 3] - base) if (~late).any() else float('nan'):.2f} (median of the others), "
                     f"{(ev[:, 3] - base).max():.2f} (last)")
    return "\n".join(lines)


def run_ours(args):
    import torch
    from lite_lang_b200.csrc import build as kbuild

    pk = peaks()
    shape = WORKLOADS[args.shape]["model"] if args.shape else QWEN2_1P5B   # (--only runs may use another shape)
    layers_full = shape["num_hidden_layers"]
    layers = args.layers or layers_full
    batch = args.batch
    engine = build_engine(layers, batch if args.only else max(64, batch), model=shape)
    cfg = engine.model_config
    weight_bytes = engine.model.weight_bytes_per_step()
    kvb = kv_bytes_per_token(engine)
    if args.only == "decode":
        ms, ctx = device_decode(engine, batch, args.steps, args.warmup)
        print(json.dumps({"only": "decode", "batch": batch, "layers": layers, "ms_per_step": round(ms, 4),
                          "mean_context": ctx}))
        return 0
    if args.only == "kernels":
        print(kernel_times(engine, batch, max(4, min(args.steps, 20))))
        return 0
    if args.only == "timeline":
        print(layer_timeline(engine, batch, args.steps, args.warmup))
        return 0
    if args.only == "prefill":
        r = prefill_once(engine, repeats=max(1, args.steps), seconds=0.0)
        print(json.dumps({"only": "prefill", "layers": layers, "tokens": PROMPT_LEN, "ms": round(r["ms"], 3),
                          "ms_min": round(r["ms_min"], 3), "repeats": r["repeats"]}))
        return 0

    points, host_ms = {}, {}
    for b in (1, 64):
        ms, _ = device_decode(engine, b, max(16, args.steps // 4), max(3, args.warmup))
        points[f"decode_b{b}"] = round(b / ms * 1e3, 1)
        v, _, _, _, hm = e2e_decode(engine, b, max(16, args.steps // 4), max(3, args.warmup))
        points[f"e2e_b{b}"] = round(v, 1)
        host_ms[f"b{b}"] = round(hm, 4)

    pre = prefill_once(engine)
    prefill_ms = pre["ms"]
    pf = prefill_flops(cfg, PROMPT_LEN)
    pclk = pre["clocks"]
    prefill = {"value": round(PROMPT_LEN / prefill_ms * 1e3, 1), "tokens": PROMPT_LEN, "ms": round(prefill_ms, 3),
               "frac": round(pf / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "ms_min": round(pre["ms_min"], 3), "repeats": pre["repeats"], "flops": pf,
               "sm_mhz": pclk.get("sm_mhz"), "sm_max_mhz": pclk.get("sm_max_mhz"), "reasons": pclk.get("reasons")}
    if pclk.get("sm_mhz") and pclk.get("sm_max_mhz"):
        # what the median would be at the highest clock, if the time went with the clock alone
        prefill["ms_at_max_clock"] = round(prefill_ms * pclk["sm_mhz"] / pclk["sm_max_mhz"], 3)
    if "bf16_tflops_sustained" in pk:
        prefill["frac_of_sustained"] = round(pf / (prefill_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)

    clocks = ClockSampler()
    clocks.start()
    ms, ctx = device_decode(engine, batch, args.steps, args.warmup)
    clk = clocks.stop()
    bucket = engine.runner._bucket(batch)
    per_step_kernels = engine.runner.graph_kernel_launches.get(bucket, 0) + 2        # + the two sampling kernels
    value = batch / ms * 1e3
    step_bytes = weight_bytes + batch * ctx * kvb
    achieved = step_bytes / (ms * 1e-3) / 1e9

    e2e_value, h2d, d2h, e2e_ms, hm = e2e_decode(engine, batch, args.steps, args.warmup)
    host_ms[f"b{batch}"] = round(hm, 4)

    out = {
        "metric": "decode tok/s (Qwen2-1.5B shape, 1xB200)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": "Qwen2-1.5B-shaped, random weights", "layers": layers, "layers_full": layers_full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied_embeddings": cfg.tie_word_embeddings, "global_batch": batch, "seq_len": CONTEXT,
                   "prompt_len": PROMPT_LEN, "mean_context_timed": round(ctx, 1), "page_size": 16,
                   "parallelism": "single GPU", "l2": "step inputs (3.1 GB of weights) exceed L2; no flush",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 4)},
        "gpu_launches": per_step_kernels * args.steps,
        "gpu_launches_per_step": per_step_kernels,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "step_bytes": int(step_bytes)},
        "points": points,
        "host_ms_per_step": host_ms,
        "clocks": clk,
    }
    if not args.no_workloads and not args.layers:
        # the two serving workloads, each with a model of its own (this one's memory is given back first)
        del engine
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        out["workloads"] = {}
        for name in sorted(WORKLOADS):
            r = workload_result(name, 0)
            out["workloads"][name] = {k: r[k] for k in ("seconds", "new_tokens_per_s", "all_tokens_per_s", "steps",
                                                        "preemptions")}
            gc.collect()
            torch.cuda.empty_cache()
    print(json.dumps(out))
    return 0


def run_reference(args):
    """The unmodified reference from baseline/_ref through its own runner API, if it is installed."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref, "litelang")):
        why = "the reference is not installed under baseline/_ref"
    if why is None:
        try:
            from baseline.reference_arm import run as run_ref   # noqa
            return run_ref(args)
        except Exception as exc:  # the reference could not run here: say why in one line
            why = f"{type(exc).__name__}: {str(exc).splitlines()[0] if str(exc) else ''}"[:300]
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


WORKLOADS = {
    # the two serving workloads named beside the headline configuration: layer sizes, requests, lengths
    "3b_batch40": dict(
        model=dict(architectures=["Qwen2ForCausalLM"], hidden_size=2048, num_hidden_layers=36, num_attention_heads=16,
                   num_key_value_heads=2, head_dim=128, intermediate_size=11008, vocab_size=151936, rope_theta=1e6,
                   rms_norm_eps=1e-6, max_position_embeddings=4096, tie_word_embeddings=True),
        requests=40, prompt=(600, 600), new_tokens=600, max_batch=40),
    "7b_mixed64": dict(
        model=dict(architectures=["Qwen2ForCausalLM"], hidden_size=3584, num_hidden_layers=28, num_attention_heads=28,
                   num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064, rope_theta=1e6,
                   rms_norm_eps=1e-6, max_position_embeddings=8192, tie_word_embeddings=False),
        requests=64, prompt=(128, 4096), new_tokens=256, max_batch=64),
}


def workload_result(name, layers_arg):
    """A whole serving workload through Engine.step(): admission, prompts cut into portions of at most 2,048
    tokens a step beside the decode tokens of the others, sampling, finishing.  Wall clock around all of it."""
    import numpy as np
    import torch
    from lite_lang_b200 import Engine, EngineConfig, SamplingParams
    from lite_lang_b200.config import config_from_dict

    w = WORKLOADS[name]
    layers_full = w["model"]["num_hidden_layers"]
    layers = layers_arg or layers_full
    cfg = config_from_dict(dict(w["model"], num_hidden_layers=layers))
    lo, hi = w["prompt"]
    rng = np.random.default_rng(11)
    lengths = [int(rng.integers(lo, hi + 1)) for _ in range(w["requests"])]
    longest = max(lengths) + w["new_tokens"] + 1
    pages = sum((n + w["new_tokens"] + 16) // 16 + 1 for n in lengths) + 8
    ecfg = EngineConfig(dtype="bfloat16", page_size=16, num_pages=pages, max_batch_size=w["max_batch"],
                        max_input_length=max(lengths), max_output_length=w["new_tokens"], max_model_len=longest,
                        max_tokens_per_step=2048, cuda_graphs=True, seed=0)
    engine = Engine(config=cfg, engine_config=ecfg, random_seed=1234)
    engine.runner.capture_all()
    sp = SamplingParams(temperature=0.0, max_new_tokens=w["new_tokens"], ignore_eos=True)
    prompts = [[int(t) for t in rng.integers(0, cfg.vocab_size, size=n)] for n in lengths]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    reqs = [engine.add_request(p, sp) for p in prompts]
    steps = 0
    while engine.scheduler.has_work():
        engine.step()
        steps += 1
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    new = sum(len(r.output) for r in reqs)
    st = engine.stats()
    return {"workload": name, "impl": "ours", "layers": layers, "layers_full": layers_full,
            "requests": len(reqs), "prompt_tokens": sum(lengths), "new_tokens": new,
            "seconds": round(dt, 3), "steps": steps, "new_tokens_per_s": round(new / dt, 1),
            "all_tokens_per_s": round((new + sum(lengths)) / dt, 1),
            "preemptions": st.get("preemptions", 0), "graph_replays": st.get("graph_replays", 0),
            "dtype": "bf16", "data": "synthetic"}


def run_workload(args):
    print(json.dumps(workload_result(args.workload, args.layers)))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (reported in config)")
    ap.add_argument("--only", default="", choices=["", "decode", "prefill", "kernels", "timeline"],
                    help="a small case for profilers: only the decode steps or only the prefill (prints a short "
                         "line), or 'kernels': the decode step's kernels timed inside its graph by torch.profiler, or "
                         "'timeline' (with LITE_LANG_B200_TIMELINE=1): when the CTAs of the last layer's kernels "
                         "started, were let go by the kernel before, and ended, inside the captured decode step")
    ap.add_argument("--workload", default="", choices=[""] + sorted(WORKLOADS),
                    help="instead of the headline measurement: a whole serving workload through the scheduler "
                         "(Qwen2.5-3B sizes, 40 requests of 600 + 600 tokens; Qwen2-7B sizes, 64 requests with prompts "
                         "of 128..4096 tokens cut into portions of 2,048 a step, 256 new tokens each)")
    ap.add_argument("--no-workloads", action="store_true", dest="no_workloads",
                    help="leave the two serving workloads out of the headline run")
    ap.add_argument("--prompt-len", type=int, default=0,
                    help="with --only decode: another context length than the headline's 2,048 prompt tokens")
    ap.add_argument("--shape", default="", choices=[""] + sorted(WORKLOADS),
                    help="with --only: the layer sizes of that workload's model instead of Qwen2-1.5B's")
    args = ap.parse_args()
    if args.shape and not args.only:
        ap.error("--shape goes with --only (the headline measurement is of the Qwen2-1.5B sizes)")
    if args.prompt_len:
        if args.only != "decode":
            ap.error("--prompt-len goes with --only decode")
        global PROMPT_LEN, CONTEXT
        PROMPT_LEN = args.prompt_len
        CONTEXT = args.prompt_len + args.steps + args.warmup + 64
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not built (this engine has no multi-GPU path)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    if args.workload:
        return run_workload(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
