"""Command line: ``litelang --model_path DIR ...`` generates tokens for given prompts.

The option names and meanings are the reference's where it has them
(``litelang/apis/test_server.py:7-24``): ``--model_path``, ``--max_output_length``,
``--max_input_length``, ``--max_batch_size``, ``--tp``, ``--mem_usage``,
``--max_reqs``, ``--busy_scale``.  The reference's command starts an HTTP server
(``--port``); this one has no server: it reads prompts (token ids from a JSON
file, or text), generates, and prints one JSON line with the new tokens.
``--use_radix_cache`` is accepted only as false (there is no prefix cache) and
``--tp`` only as 1 (one GPU).
"""

from __future__ import annotations

import json
import sys

import click


@click.command()
@click.option("--model_path", required=True, help="folder with config.json and safetensors (and a tokenizer for text)")
@click.option("--max_output_length", default=200, type=int, help="most new tokens of a request")
@click.option("--max_input_length", default=4000, type=int, help="most prompt tokens of a request")
@click.option("--max_batch_size", default=32, type=int, help="most requests running at a time")
@click.option("--tp", default=1, type=int, help="tensor-parallel degree; only 1 is built")
@click.option("--port", default=None, type=int, help="ignored: there is no HTTP server")
@click.option("--mem_usage", default=0.5, type=float, help="fraction of free GPU memory for the cache")
@click.option("--max_reqs", default=1000, type=int, help="most waiting requests")
@click.option("--busy_scale", default=0.6, type=float,
              help="cache share above which requests are expected to use their whole output length")
@click.option("--use_radix_cache", default=False, type=bool, help="only false: there is no prefix cache")
@click.option("--dtype", default="bf16", type=click.Choice(["bf16", "bfloat16", "fp32", "float32"]))
@click.option("--page_size", default=16, type=int, help="tokens per cache page")
@click.option("--num_pages", default=None, type=int, help="pages of the cache (instead of --mem_usage)")
@click.option("--max_tokens_per_step", default=2048, type=int, help="token budget of a step")
@click.option("--random_weights", default=None, type=int, help="seed: ignore the folder's weights, draw random ones")
@click.option("--seed", default=0, type=int, help="seed of temperature sampling")
@click.option("--temperature", default=0.0, type=float, help="0 is greedy")
@click.option("--prompt_ids", default=None, help="JSON file: a list of prompts, each a list of token ids")
@click.option("--prompt", multiple=True, help="a text prompt (needs the folder's tokenizer); may be repeated")
@click.option("--ignore_eos", is_flag=True, default=False)
@click.option("--no_cuda_graphs", is_flag=True, default=False)
def run(model_path, max_output_length, max_input_length, max_batch_size, tp, port, mem_usage, max_reqs, busy_scale,
        use_radix_cache, dtype, page_size, num_pages, max_tokens_per_step, random_weights, seed, temperature,
        prompt_ids, prompt, ignore_eos, no_cuda_graphs):
    if tp != 1:
        raise click.UsageError("--tp: only 1 is built (one GPU)")
    if use_radix_cache:
        raise click.UsageError("--use_radix_cache: there is no prefix cache; only false is accepted")
    if port is not None:
        click.echo("note: --port is ignored, there is no HTTP server", err=True)
    if not prompt_ids and not prompt:
        raise click.UsageError("give --prompt_ids FILE or --prompt TEXT")
    from . import Engine, EngineConfig, SamplingParams

    cfg = EngineConfig(dtype=dtype, page_size=page_size, num_pages=num_pages, mem_usage=mem_usage,
                       max_batch_size=max_batch_size, max_input_length=max_input_length,
                       max_output_length=max_output_length, max_tokens_per_step=max_tokens_per_step,
                       max_reqs=max_reqs, busy_scale=busy_scale, cuda_graphs=not no_cuda_graphs, seed=seed)
    engine = Engine(model_path, cfg, random_seed=random_weights)
    prompts = []
    if prompt_ids:
        with open(prompt_ids, "r", encoding="utf-8") as fh:
            prompts.extend(json.load(fh))
    prompts.extend(prompt)
    params = SamplingParams(temperature=temperature, max_new_tokens=max_output_length, ignore_eos=ignore_eos,
                            seed=seed)
    outs = engine.generate(prompts, params)
    result = {"outputs": outs, "stats": engine.stats()}
    if prompt:
        tok = engine.tokenizer()
        result["texts"] = [tok.decode(o) for o in outs]
    click.echo(json.dumps(result))


def main():
    run()


if __name__ == "__main__":
    main()
