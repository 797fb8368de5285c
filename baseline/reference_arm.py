"""The reference arm of bench.py: the unmodified reference, installed under baseline/_ref, driven
through its own runner API the way its benchmark script does (test/generate_token.py:24-67:
Qwen2Config -> Qwen2ModelRunner -> init_model -> RunnerBatch.create_batch -> forward /
update_forward_message).  Nothing of lite_lang_b200 is on that path; the random-weights writer
only produces the checkpoint folder that the reference then loads itself.

The reference computes in float16 (its only dtype, litelang/models/qwen2/layer_weights/
load_weights.py:84) with Triton kernels and cuBLAS; a forward is all-prefill or all-decode.
"""

import json
import os
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(args):
    import torch

    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    from bench import CONTEXT, PROMPT_LEN, QWEN2_1P5B, ClockSampler, random_prompts
    from lite_lang_b200.config import config_from_dict
    from lite_lang_b200.weights import write_random_model

    layers = args.layers or QWEN2_1P5B["num_hidden_layers"]
    cfg = config_from_dict(dict(QWEN2_1P5B, num_hidden_layers=layers))
    folder = os.path.join(tempfile.gettempdir(), f"ll_reference_arm_qwen2_1p5b_{layers}")
    if not os.path.isfile(os.path.join(folder, "model.safetensors")):
        write_random_model(folder, cfg, seed=1234, dtype="float16")

    from litelang.models.qwen2.model import Qwen2Config, Qwen2ModelRunner
    from litelang.models.runner_batch import RunnerBatch

    batch_size, steps, warmup = args.batch, args.steps, args.warmup
    rcfg = Qwen2Config(os.path.join(folder, "config.json"))
    runner = Qwen2ModelRunner(layer_nums=rcfg.layer_nums, max_batch_size=batch_size, config=rcfg, tp_rank=0,
                              world_size=1, model_path=folder, max_length=PROMPT_LEN + steps + warmup + 2,
                              mem_usage=0.5, use_radix_cache=False)
    runner.init_model()
    prompts = random_prompts(batch_size, PROMPT_LEN, cfg.vocab_size, 7)
    msgs = [{"id": i, "input_tokens": p, "temperature": 0.7, "top_p": 0.9, "top_k": 50, "do_sample": False,
             "ignore_eos": True} for i, p in enumerate(prompts)]
    batch = RunnerBatch.create_batch(msgs, "bench-batch", is_prefill=True, model_runner=runner)
    out = runner.forward(batch)                     # prefill, untimed
    batch.update_forward_message(out)
    for _ in range(warmup):
        out = runner.forward(batch)
        batch.update_forward_message(out)
    torch.cuda.synchronize()
    clocks = ClockSampler()
    clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        out = runner.forward(batch)
        batch.update_forward_message(out)
    e1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    clk = clocks.stop()
    ms = e0.elapsed_time(e1) / steps
    value = batch_size / ms * 1e3
    print(json.dumps({
        "impl": "reference", "metric": "decode tok/s (Qwen2-1.5B shape, 1xB200)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
        "config": {"model": "Qwen2-1.5B-shaped, random weights", "layers": layers,
                   "layers_full": QWEN2_1P5B["num_hidden_layers"], "global_batch": batch_size, "seq_len": CONTEXT,
                   "prompt_len": PROMPT_LEN, "page_size": 1, "parallelism": "single GPU",
                   "path": "Qwen2ModelRunner.forward as in the reference's test/generate_token.py"},
        "e2e": {"value": round(batch_size * steps / wall, 1), "unit": "tokens/s",
                "note": "the reference's forward reads every token back to the host itself"},
        "clocks": clk,
    }))
    return 0
