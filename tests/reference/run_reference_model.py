"""Runs the unmodified reference model on the GPU and saves the logits it computed.

Usage: run_reference_model.py REF_ROOT MODEL_DIR PROMPTS_JSON N_DECODE OUT_NPZ

``REF_ROOT`` is a folder that holds the reference's ``litelang`` package as installed
(unchanged).  The model is driven through the reference's own runner API exactly as its
benchmark script does (``test/generate_token.py:24-67``: ``Qwen2Config`` ->
``Qwen2ModelRunner`` -> ``init_model`` -> ``RunnerBatch.create_batch`` -> ``forward`` /
``update_forward_message``): one prefill of all prompts, then ``N_DECODE`` decode steps that
feed the tokens the reference itself chose.  The only thing added from outside is a wrapper
around ``Qwen2PostLayer._PostProcess`` (``qwen2/layer/post_layer.py:75-77``) that keeps a copy
of the logits it is handed; the reference's code and its results are untouched.

Saves ``logits`` [steps, requests, vocab] float32 and ``tokens`` [steps, requests] (the
reference's own argmax).  Runs in a process of its own because the reference's modules
grab ``cuda:0`` at import time.
"""
import json
import sys

import numpy as np


def main(argv):
    ref_root, model_dir, prompts_json, n_decode, out_path = argv[1], argv[2], argv[3], int(argv[4]), argv[5]
    sys.path.insert(0, ref_root)
    import torch
    from litelang.models.qwen2.model import Qwen2Config, Qwen2ModelRunner
    from litelang.models.runner_batch import RunnerBatch

    with open(prompts_json) as fh:
        prompts = json.load(fh)
    cfg = Qwen2Config(f"{model_dir}/config.json")
    longest = max(len(p) for p in prompts)
    runner = Qwen2ModelRunner(layer_nums=cfg.layer_nums, max_batch_size=len(prompts), config=cfg, tp_rank=0,
                              world_size=1, model_path=model_dir, max_length=longest + n_decode + 2,
                              mem_usage=0.01, use_radix_cache=False)
    runner.init_model()
    post = runner.model_ins_.post_layer
    kept = []
    inner = post._PostProcess

    def keep(logits, model_inputs):
        kept.append(logits.detach().float().cpu().numpy())
        return inner(logits, model_inputs)

    post._PostProcess = keep
    msgs = [{"id": i, "input_tokens": list(p), "temperature": 1.0, "top_p": 1.0, "top_k": 1, "do_sample": False,
             "ignore_eos": True} for i, p in enumerate(prompts)]
    batch = RunnerBatch.create_batch(msgs, "anchor", is_prefill=True, model_runner=runner)
    tokens = []
    for _ in range(1 + n_decode):
        out = runner.forward(batch)
        batch.update_forward_message(out)
        tokens.append(out.detach().cpu().numpy().reshape(-1))
    torch.cuda.synchronize()
    np.savez(out_path, logits=np.stack(kept), tokens=np.stack(tokens))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
