"""Makes scheduler_anchors.json: decisions of the reference's own host code on seeded random inputs.

    python tests/golden/make_scheduler_anchors.py <path to a checkout of ppppppppig/lite_lang>

The reference's scheduler queue code needs no GPU and runs as it is:

  Req.need_tokens                  litelang/scheduler/req_queue.py:59-66    (tokens held, tokens expected)
  ReadyQue._can_add_new_req        litelang/scheduler/req_queue.py:219-232  (the peak estimate against the pool)
  ReadyQue._is_system_busy         litelang/scheduler/req_queue.py:213-217
  Strategy.ordering (four of them) litelang/scheduler/pause_strategy.py:18-39
  select_swapped_reqs              litelang/scheduler/pause_strategy.py:42-55

For each admission case the file keeps the running requests and the candidate (prompt length, tokens
produced, limit of new tokens), whether the system counts as busy, the pool's size, the rows the
reference built and its answer; for each preemption case the requests (id, length), the tokens that are
missing, and for each strategy the reference's order and the requests it takes out.
tests/test_scheduler.py compares the engine's scheduler with the stored answers; the stored file is all
it needs.
"""
import json
import os
import queue
import random
import sys


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from litelang.scheduler.pause_strategy import STRATEGY_REGISTRY, select_swapped_reqs
    from litelang.scheduler.req_queue import ReadyQue, Req, ReqStatus

    def make_req(rid, n_in, n_out, max_out):
        r = Req(id=rid, status=ReqStatus.READY, prompt="", input_tokens=[0] * n_in, output_tokens=[0] * n_out,
                max_total_length=n_in + max_out, max_output_length=max_out, output_prompt_que=queue.Queue(),
                temperature=1.0, top_p=1.0, top_k=1, do_sample=False, input_length=n_in, eos_token=-1)
        r.output_length = n_out
        return r

    rng = random.Random(20251125)
    admission = []
    for case in range(160):
        n_run = rng.randint(0, 6)
        fresh = case % 2 == 0                       # half of the cases: nobody has produced anything yet
        reqs = []
        for i in range(n_run + 1):
            max_out = rng.randint(1, 60)
            n_out = 0 if fresh else rng.randint(0, max_out - 1)
            reqs.append((rng.randint(1, 80), n_out, max_out))
        busy = rng.random() < 0.5
        total = sum(a + b for a, b, _ in reqs)
        pool = max(1, int(total * rng.uniform(0.8, 2.5)))
        rq = ReadyQue(max_reqs=100, max_input_length=100, max_output_length=100, max_sum_kv_tokens=pool,
                      max_batch_size=16, busy_scale=0.6)
        running = [make_req(i, *r) for i, r in enumerate(reqs[:-1])]
        cand = make_req(n_run, *reqs[-1])
        rq._init_cache_len(running, busy)
        answer = rq._can_add_new_req(cand, busy)
        rows = [[int(a), int(b)] for a, b in rq.cache_len_list_]
        admission.append({"requests": [list(r) for r in reqs], "busy": busy, "pool": pool, "rows": rows,
                          "admitted": bool(answer)})

    preemption = []
    for case in range(120):
        n = rng.randint(1, 8)
        lengths = [rng.randint(1, 100) for _ in range(n)]
        reqs = [make_req(i, l, 0, 10) for i, l in enumerate(lengths)]
        need = rng.randint(1, max(1, sum(lengths)))
        per = {}
        for name, cls in STRATEGY_REGISTRY.items():
            s = cls()
            per[name] = {"order": [r.id for r in s.ordering(reqs)],
                         "out": [r.id for r in select_swapped_reqs(reqs, s, need)]}
        preemption.append({"lengths": lengths, "need": need, "strategies": per})

    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "scheduler_anchors.json")
    with open(out, "w") as fh:
        json.dump({"admission": admission, "preemption": preemption}, fh, separators=(",", ":"))
    print(f"wrote {out}: {len(admission)} admission cases, {len(preemption)} preemption cases")


if __name__ == "__main__":
    main(sys.argv[1])
