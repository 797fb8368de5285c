"""The timeline build (GPU): kernels compiled with their time stamps, run in a process of its own.

LITE_LANG_B200_TIMELINE=1 builds the kernel libraries a second time, with thread 0 of every CTA of the decode
step's products and of the decode attention writing %globaltimer behind the status word.  The ordinary build holds
none of that code; this test only checks that the other build runs, that its stamps are in order (started <=
released <= ended, a kernel released after the one before it) and that the step's results are the same.
"""
import os
import subprocess
import sys

import pytest

from helpers import ROOT

pytestmark = pytest.mark.gpu

SCRIPT = r"""
import sys, json
sys.path.insert(0, sys.argv[1])
import numpy as np, torch
import bench
from lite_lang_b200 import ops
engine = bench.build_engine(2, 4)
ms, ctx = bench.device_decode(engine, 4, 6, 3)
tl = engine.runner.timeline()
out = {"timeline_build": ops.timeline_build(), "kernels": None}
if tl is not None:
    out["kernels"] = sorted(tl)
    order = ["qkv", "attention", "o", "gated", "down"]
    rel = [float(tl[k][:, 1].min()) for k in order]
    out["released_in_order"] = all(a < b for a, b in zip(rel, rel[1:]))
    out["stamps_in_order"] = all(bool(((ev[:, 0] <= ev[:, 1]) & (ev[:, 1] <= ev[:, 2])).all()) for ev in tl.values())
    out["layer_us"] = float(tl["down"][:, 2].max() - tl["qkv"][:, 1].min())
    out["table"] = bench.layer_timeline(engine, 4, 4, 2)
print("RESULT " + json.dumps(out))
"""


def _run(timeline):
    env = dict(os.environ, LITE_LANG_B200_TIMELINE="1" if timeline else "0")
    r = subprocess.run([sys.executable, "-c", SCRIPT, ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    import json
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def test_timeline_build_stamps_the_decode_kernels_in_order():
    got = _run(True)
    assert got["timeline_build"] is True
    assert got["kernels"] == sorted(["qkv", "attention", "o", "gated", "down", "logits"])
    assert got["stamps_in_order"] and got["released_in_order"]
    assert 5.0 < got["layer_us"] < 500.0, got["layer_us"]
    assert "attention" in got["table"] and "released" in got["table"]


def test_ordinary_build_has_no_timeline():
    got = _run(False)
    assert got["timeline_build"] is False and got["kernels"] is None
