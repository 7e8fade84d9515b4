"""The engine on the GPU against the plain implementation, for every way of cutting the work."""

import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import traces
from conftest import ROOT, TINY
from gpu_util import expected_logits, gpu_runner, tolerances

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 70, 41, 64, 100], "B": [1, 9, 40, 64, 130, 77, 2], "C": [3, 66, 129, 50, 35, 200]}


@pytest.fixture(scope="module")
def expected(tiny_dirs):
    out = {}
    for name in TINY:
        reqs = traces.make_requests(LENGTHS[name], TINY[name]["vocab_size"], seed=11)
        out[name] = (reqs, expected_logits(tiny_dirs[name], reqs))
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_every_way_of_cutting_matches_plain(tiny_dirs, expected, name, mode, dtype):
    reqs, exp = expected[name]
    pool_tokens = traces.tokens_needed(reqs)
    runner = gpu_runner(tiny_dirs[name], name, pool_tokens // TINY[name]["page_tokens"], dtype)
    got = traces.replay(runner, getattr(traces, mode)(reqs))
    atol, rtol = tolerances(dtype)
    traces.compare(got, exp, atol=atol, rtol=rtol)
    assert runner.manager.usage() == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuts_agree_with_each_other_closely(tiny_dirs, expected, dtype):
    """Logits must not depend on the cut beyond rounding: whole vs mixed, engine against itself."""
    reqs, _ = expected["C"]
    pool = traces.tokens_needed(reqs) // TINY["C"]["page_tokens"]
    a = traces.replay(gpu_runner(tiny_dirs["C"], "C", pool, dtype), traces.whole(reqs))
    b = traces.replay(gpu_runner(tiny_dirs["C"], "C", pool, dtype), traces.mixed(reqs, seed=5))
    scale = max(v.abs().max().item() for v in a.values())
    worst = max((a[k] - b[k]).abs().max().item() for k in a)
    assert worst <= (1e-5 if dtype == "float32" else 0.02 * scale), worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(tiny_dirs, dtype):
    """300 tokens one by one from position 0: the first tokens of a sequence and a long decode."""
    reqs = traces.make_requests([300], TINY["B"]["vocab_size"], seed=21)
    exp = expected_logits(tiny_dirs["B"], reqs)
    runner = gpu_runner(tiny_dirs["B"], "B", 320 // 8, dtype)
    got = traces.replay(runner, traces.decode_tail(reqs, tail=300))
    atol, rtol = tolerances(dtype)
    traces.compare(got, exp, atol=atol, rtol=rtol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tiny_dirs, expected, tmp_path, dtype):
    """bin/trace_run as a user runs it: JSON steps on stdin, .f32 files out."""
    reqs, exp = expected["A"]
    steps = traces.mixed(reqs, seed=2)
    out = tmp_path / "out"
    p = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(tiny_dirs["A"]),
         "--dtype", dtype, "--out", str(out), "--max-tokens", str(traces.tokens_needed(reqs))],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
    )
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    V = TINY["A"]["vocab_size"]
    got, pos = {}, {}
    for s in steps:
        data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, V)
        row = 0
        for e in s["entries"]:
            p0 = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], p0 + w)] = torch.from_numpy(data[row].copy())
                row += 1
            pos[e["id"]] = p0 + len(e["tokens"])
        assert row == data.shape[0]
    atol, rtol = tolerances(dtype)
    traces.compare(got, exp, atol=atol, rtol=rtol)
