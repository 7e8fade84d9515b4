"""Throughput of the engine on one B200, random weights, synthetic token ids.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--parity]
    python bench.py --workload continuous | long
    python bench.py --impl reference [--steps K] [--warmup W]

The default workload is decoding at SmolLM2-1.7B sizes: a "step" is one decode step of the whole
model (one token per request from the paged cache, output projection, sampling). ``value`` is
decoded tokens per second from CUDA-event timing of exactly K steps replayed back to back; ``e2e``
is the same workload driven through ``LLMEngine.step()`` (scheduler, pinned host buffer -> device
copy of the step's inputs, the step, device -> host read of the sampled token ids) by wall clock.
After the timed region the logits of one captured step are compared with the same step run kernel
by kernel; ``--parity`` also compares a two-layer model of the same layer sizes with the plain
implementation in ``tests/``. One JSON line is printed.

``--workload continuous`` (SmolLM2-360M sizes: 64 requests, a 2048-token prompt arriving mid-run,
512-token budget) and ``--workload long`` (SmolLM2-135M sizes: 16 requests of 7936 + 256 tokens,
and a float32 replay of one 8192-token sequence against the plain implementation) follow the
reference's own harness (src/llmserve/bench/run.py:96,124-176): fixed output lengths, greedy, a
warm-up run that is thrown away, one JSON line with the environment.

``--impl reference`` runs the unmodified reference package from ``baseline/_ref`` through its own
``LLMEngine`` on the same device, sizes and workload, and prints the same line.
"""

from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import threading
import time
import traceback
from pathlib import Path

ROOT = Path(__file__).resolve().parent

PROMPT_LEN = 2048
CONTEXT = 4096
PREFILL_TOKENS = 2048
METRIC = "decode tok/s @ batch 8 (SmolLM2-1.7B sizes, 2048-token prompts)"


def peaks() -> dict:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.rows: list[list[str]] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm = [int(r[0]) for r in self.rows if r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


def random_prompts(n, length, vocab, seed):
    import torch

    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n, length), generator=g).tolist()


def environment() -> dict:
    import torch

    return {"gpu": torch.cuda.get_device_name(0), "torch": torch.__version__,
            "cuda": torch.version.cuda, "python": sys.version.split()[0]}


# --------------------------------------------------------------------------- this engine
def model_numbers(model, cfg) -> dict:
    """Bytes a decode step has to read and flops of the prefill, from the model's own parameter
    declarations (every weight once; the embedding table only where it is the output projection)."""
    import numpy as np

    decls = model.param_decls()
    count = lambda names: sum(int(np.prod(decls[n].shape)) for n in names)
    embed = [n for n in decls if decls[n].role == "embedding"]
    rest = [n for n in decls if decls[n].role != "embedding"]
    head = count(embed) if model.plan.tie_head else 0  # untied heads are "matrix" parameters
    weight_bytes = 2 * (count(rest) + head)
    layers = len(model.plan.run_order)
    kv_bytes_per_token = 2 * layers * cfg.kv_size * 2
    T = PREFILL_TOKENS
    matrices = count(n for n in rest if decls[n].role == "matrix" and n != "head.weight")
    prefill_flops = 2 * T * matrices + 2 * cfg.hidden_size * cfg.vocab_size  # one logits row
    prefill_flops += 4 * layers * cfg.num_attention_heads * cfg.head_dim * T * (T + 1) // 2
    return dict(weight_bytes=weight_bytes, kv_bytes_per_token=kv_bytes_per_token,
                prefill_flops=prefill_flops)


def make_engine(args, layers_full: int):
    from llmserve_b200 import EngineConfig, LLMEngine

    over = {"num_hidden_layers": args.layers} if args.layers != layers_full else None
    max_b = max(64, args.batch)
    page = args.page_tokens
    tokens_per_req = -(-(PROMPT_LEN + 2 * (args.steps + args.warmup) + 64) // page) * page
    return LLMEngine(EngineConfig(
        model=f"random:{args.model}", dtype="bfloat16", seed=4, block_size=page,
        num_kv_blocks=max_b * tokens_per_req // page, max_model_len=CONTEXT, max_num_seqs=max_b,
        max_num_batched_tokens=PREFILL_TOKENS, config_overrides=over))


def start_decoding(engine, batch, seed):
    """Admit ``batch`` requests with 2048-token prompts and run their prompts; all decode after."""
    from llmserve_b200 import SamplingParams

    sp = SamplingParams(temperature=0.0, max_tokens=CONTEXT - PROMPT_LEN - 1, ignore_eos=True)
    ids = [engine.add_request(p, sp) for p in
           random_prompts(batch, PROMPT_LEN, engine.model_cfg.vocab_size, seed)]
    while engine.scheduler.waiting or any(
            s.num_computed_tokens < s.num_prompt_tokens for s in engine.scheduler.running):
        engine.step()
    return ids


def graph_against_eager(engine) -> float:
    """Largest difference between the logits of the running requests' next step replayed as a
    captured graph and the same step launched kernel by kernel. Nothing is committed: both write
    the same keys and values to the same places."""
    from llmserve_b200.engine.batch import StepEntry

    if engine._pending is not None:  # a step launched ahead: let it finish, keep nothing of it
        engine.runner.collect_decode(engine._pending.pending)
        engine._pending = None
    seqs = list(engine.scheduler.running)
    entries = [StepEntry(s.seq_id, s.tokens_from(s.num_computed_tokens, 1), [0]) for s in seqs]
    for s in seqs:
        engine.manager.allocate(s.seq_id, 1)
    captured = engine.runner._graphs().captured_logits(entries)
    eager = engine.runner.step(entries)
    return float((captured - eager).abs().max())


def measure_decode(engine, batch, steps, warmup, seed, check=False):
    """Device and end-to-end ms per step, launches and bytes per step, contexts of the requests."""
    import torch

    ids = start_decoding(engine, batch, seed)
    for _ in range(max(3, warmup)):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        out = engine.step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    assert engine.last_step.num_decode_tokens == batch and len(out) == batch
    h2d, d2h = engine.runner.last_h2d_bytes, engine.runner.last_d2h_bytes
    # the same step, replayed back to back with no host in between
    graphs = engine.runner.decode_graphs.graphs
    g = max((x for x in graphs.values() if x.batch == batch and x.slots == 0 and x.graph is not None
             and x.sampled), key=lambda x: x.step.decode_splits)
    for _ in range(3):
        g.graph.replay()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        g.graph.replay()
    end.record()
    torch.cuda.synchronize()
    dev_ms = start.elapsed_time(end) / steps
    ctx_sum = sum(s.num_tokens for s in engine.scheduler.running)
    ctx_max = max(s.num_tokens for s in engine.scheduler.running)
    diff = graph_against_eager(engine) if check else None
    for i in ids:
        engine.abort_request(i)
    return dict(dev_ms=dev_ms, e2e_ms=e2e_ms, launches=g.launches, h2d=h2d, d2h=d2h, ctx=ctx_max,
                ctx_sum=ctx_sum, graph_vs_eager=diff)


def step_timeline(engine, batch, seed) -> dict:
    """Start and end of every kernel of one captured step of single tokens, from the framework's
    profiler (CUPTI), summed by kernel: launches, time resident, and what the kernel adds to the
    step (the time from the latest end of any kernel before it to its own end; a kernel that is
    resident while the one before it still runs adds less than it lasts)."""
    import collections

    import torch
    from torch.profiler import ProfilerActivity, profile

    ids = start_decoding(engine, batch, seed)
    for _ in range(4):
        engine.step()
    torch.cuda.synchronize()
    graphs = engine.runner.decode_graphs.graphs
    g = max((x for x in graphs.values() if x.batch == batch and x.slots == 0 and x.graph is not None
             and x.sampled), key=lambda x: x.step.decode_splits)
    for _ in range(3):
        g.graph.replay()
    torch.cuda.synchronize()
    reps = 4
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(reps):
            g.graph.replay()
        torch.cuda.synchronize()
    rows = sorted((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                  if e.device_type == torch.autograd.DeviceType.CUDA)
    n = len(rows) // reps
    step = rows[2 * n : 3 * n]  # the third replay
    fam = collections.OrderedDict()
    latest = step[0][0]
    for start, end, name in step:
        key = name.split("(")[0].replace("void ", "").replace("lse::", "")
        f = fam.setdefault(key, {"launches": 0, "resident_us": 0.0, "adds_us": 0.0})
        f["launches"] += 1
        f["resident_us"] += end - start
        f["adds_us"] += max(0.0, end - max(start, latest))
        latest = max(latest, end)
    for i in ids:
        engine.abort_request(i)
    out = {k: {a: (round(b, 1) if isinstance(b, float) else b) for a, b in v.items()}
           for k, v in sorted(fam.items(), key=lambda kv: -kv[1]["adds_us"])}
    return {"step_us": round(latest - step[0][0], 1), "kernels": len(step), "by_kernel": out}


def measure_prefill(engine, reps=5, warmup=3):
    import torch

    from llmserve_b200 import SamplingParams

    sp = SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True)
    times = []
    for k, p in enumerate(random_prompts(reps + warmup, PREFILL_TOKENS, engine.model_cfg.vocab_size, 99)):
        rid = engine.add_request(p, sp)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step()
        end.record()
        torch.cuda.synchronize()
        assert engine.last_step.num_prefill_tokens == PREFILL_TOKENS
        engine.abort_request(rid)
        if k >= warmup:
            times.append(start.elapsed_time(end))
    return statistics.median(times)


def plain_parity(model_alias: str, dtype: str, layers: int = 2, tokens: int = 2100) -> dict:
    """A ``layers``-layer model of the alias's layer sizes, written to a folder and read back by
    tensor name, against the plain implementation (float64, same device) on one request: whole,
    and with its last 32 tokens one by one. Largest difference over the compared logits rows."""
    import tempfile

    import torch

    sys.path.insert(0, str(ROOT / "tests"))
    import plain_llama

    from llmserve_b200.config.registry import architecture_for
    from llmserve_b200.engine.batch import StepEntry
    from llmserve_b200.engine.runner import ModelRunner, load_model
    from llmserve_b200.models.hub import preset_config_dict
    from llmserve_b200.ops import get_ops
    from llmserve_b200.weights import write_random_model

    d = {**preset_config_dict(model_alias), "num_hidden_layers": layers}
    cfg = architecture_for(d).config_cls.from_dict(d)
    ids = random_prompts(1, tokens, cfg.vocab_size, 5)[0]
    rows = sorted(set(range(0, tokens, 211)) | set(range(tokens - 32, tokens)))
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(folder, cfg, seed=4)
        w = {k: v.to("cuda") for k, v in plain_llama.read_weights(folder, torch.float64).items()}
        want = plain_llama.forward(plain_llama.read_config(folder), w, ids, dtype=torch.float64,
                                   device="cuda", rows=rows)
        del w
        _, _, model = load_model(folder, dtype, "cuda", get_ops("cuda"), CONTEXT)
    out = {}
    for name, cuts in (("whole", [tokens]), ("decode_tail", [tokens - 32] + [1] * 32)):
        runner = ModelRunner(model, page_tokens=16, num_pages=-(-tokens // 16) + 1,
                             max_model_len=CONTEXT, max_num_seqs=2, max_num_batched_tokens=CONTEXT)
        got, a = [], 0
        for n in cuts:
            here = [r - a for r in rows if a <= r < a + n]
            logits = runner.run([StepEntry("x", ids[a : a + n], here)])
            if here:
                got.append(logits.double().cpu())
            a += n
        out[name] = float((torch.cat(got) - want).abs().max())
    out["largest_logit"] = round(float(want.abs().max()), 3)
    return out


def decode_main(args) -> int:
    from llmserve_b200.config.registry import architecture_for
    from llmserve_b200.models.hub import preset_config_dict

    d = preset_config_dict(args.model)
    cfg = architecture_for(d).config_cls.from_dict(d)
    layers_full = cfg.num_hidden_layers
    args.layers = args.layers or layers_full
    pk = peaks()
    engine = make_engine(args, layers_full)
    nums = model_numbers(engine.model, cfg)
    with ClockSampler() as clocks:
        main_pt = measure_decode(engine, args.batch, args.steps, args.warmup, seed=1, check=True)
    value = args.batch * 1e3 / main_pt["dev_ms"]
    bytes_step = nums["weight_bytes"] + main_pt["ctx_sum"] * nums["kv_bytes_per_token"]
    achieved = bytes_step / (main_pt["dev_ms"] * 1e-3) / 1e9
    line = {
        "metric": METRIC,
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": round(main_pt["dev_ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform random token ids, random-init weights (seed 4)",
        "impl": "ours",
        "config": {
            "model": f"{args.model} sizes", "layers": args.layers, "layers_full": layers_full,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
            "decode_ctx": main_pt["ctx"], "page_tokens": args.page_tokens, "parallelism": "single-gpu",
            "cuda_graphs": True, "l2": "inputs larger than L2 (weights + cache streamed each step)",
            "peaks": pk["source"],
        },
        "e2e": {"value": round(args.batch * 1e3 / main_pt["e2e_ms"], 1), "unit": "tok/s",
                "ms_per_step": round(main_pt["e2e_ms"], 4),
                "h2d_bytes_per_step": main_pt["h2d"], "d2h_bytes_per_step": main_pt["d2h"]},
        "gpu_launches": main_pt["launches"] * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "clocks": clocks.summary(),
        "parity": {"graph_vs_eager_max_abs_diff": main_pt["graph_vs_eager"]},
    }
    if not args.no_points:
        ms = measure_prefill(engine)
        line["prefill"] = {
            "value": round(PREFILL_TOKENS * 1e3 / ms, 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
            "frac": round(nums["prefill_flops"] / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        pts = {}
        for b in (1, 64):
            r = measure_decode(engine, b, max(16, args.steps // 2), 3, seed=10 + b)
            pts[f"decode_b{b}"] = round(b * 1e3 / r["dev_ms"], 1)
            pts[f"decode_b{b}_e2e"] = round(b * 1e3 / r["e2e_ms"], 1)
            by = nums["weight_bytes"] + r["ctx_sum"] * nums["kv_bytes_per_token"]
            pts[f"decode_b{b}_hbm_frac"] = round(by / (r["dev_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        line["points"] = pts
    if args.timeline:
        line["timeline"] = step_timeline(engine, args.batch, seed=3)
    if args.parity:
        del engine
        import torch

        torch.cuda.empty_cache()
        for dtype in ("float32", "bfloat16"):
            r = plain_parity(args.model, dtype)
            line["parity"][f"{dtype}_2_layers_vs_plain_max_abs_diff"] = max(r["whole"], r["decode_tail"])
            line["parity"]["largest_logit"] = r["largest_logit"]
    print(json.dumps(line))
    return 0


def continuous_main(args) -> int:
    """Continuous batching at SmolLM2-360M sizes: 64 requests (prompts of 16 to 1024 tokens, 16 to
    256 new tokens each), a 2048-token prompt arriving after 60 steps, 512 tokens per step."""
    import torch

    from llmserve_b200 import EngineConfig, LLMEngine, SamplingParams

    engine = LLMEngine(EngineConfig(
        model="random:smollm2-360m", dtype="bfloat16", seed=5, block_size=16, kv_cache_memory_gb=8.0,
        max_model_len=4096, max_num_seqs=64, max_num_batched_tokens=512))
    V = engine.model_cfg.vocab_size
    rng = random.Random(0)
    reqs = [([rng.randrange(V) for _ in range(rng.randint(16, 1024))], rng.randint(16, 256))
            for _ in range(64)]
    late = ([rng.randrange(V) for _ in range(2048)], 64)
    sp = lambda n: SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)

    def run():
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for p, n in reqs:
            engine.add_request(p, sp(n))
        steps, kinds, added, preempted0 = 0, {"single_tokens_only": 0, "with_prompt_portions": 0}, False, \
            engine.scheduler.num_preemptions
        while engine.has_unfinished_requests():
            engine.step()
            steps += 1
            kinds["single_tokens_only" if engine.last_step.num_prefill_tokens == 0
                  else "with_prompt_portions"] += 1
            if not added and steps == 60:
                engine.add_request(late[0], sp(late[1]))
                added = True
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        engine.manager.check_invariants()
        assert engine.manager.usage() == 0.0 and added
        return dt, steps, kinds, engine.scheduler.num_preemptions - preempted0

    run()  # thrown away: graph captures, library handles
    with ClockSampler() as clocks:
        dt, steps, kinds, preempted = run()
    n_out = sum(n for _, n in reqs) + late[1]
    n_in = sum(len(p) for p, _ in reqs) + len(late[0])
    print(json.dumps({
        "metric": "generated tok/s, continuous batching of 64 requests (SmolLM2-360M sizes)",
        "value": round(n_out / dt, 1), "unit": "tok/s", "n_gpus": 1, "higher_is_better": True,
        "dtype": "bf16", "impl": "ours", "seconds": round(dt, 4),
        "total_tok_s": round((n_in + n_out) / dt, 1), "prompt_tokens": n_in, "generated_tokens": n_out,
        "steps": steps, "steps_by_kind": kinds, "preemptions": preempted,
        "data": "synthetic: uniform random token ids, random-init weights (seed 5); second of two runs",
        "config": {"model": "smollm2-360m sizes", "requests": 64, "prompt_len": "16..1024",
                   "new_tokens": "16..256", "late_prompt": 2048, "late_after_steps": 60,
                   "max_num_batched_tokens": 512, "max_num_seqs": 64, "page_tokens": 16},
        "clocks": clocks.summary(), "environment": environment()}))
    return 0


def long_main(args) -> int:
    """Long contexts at SmolLM2-135M sizes: 16 requests of 7936 prompt + 256 new tokens on pages of
    16 tokens, then one 8192-token sequence replayed in float32 (whole, and in portions followed by
    single tokens) against the plain implementation."""
    import torch

    from llmserve_b200 import EngineConfig, LLMEngine, SamplingParams

    engine = LLMEngine(EngineConfig(
        model="random:smollm2-135m", dtype="bfloat16", seed=6, block_size=16,
        num_kv_blocks=16 * 8192 // 16 + 64, max_model_len=8192, max_num_seqs=16,
        max_num_batched_tokens=2048))
    V = engine.model_cfg.vocab_size
    rng = random.Random(1)
    sp = SamplingParams(temperature=0.0, max_tokens=255, ignore_eos=True)  # 7936 + 255 + 1 = 8192

    def run():
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(16):
            engine.add_request([rng.randrange(V) for _ in range(7936)], sp)
        steps, t_prompts = 0, None
        while engine.has_unfinished_requests():
            engine.step()
            steps += 1
            if t_prompts is None and not engine.scheduler.waiting and all(
                    s.num_computed_tokens >= s.num_prompt_tokens for s in engine.scheduler.running):
                torch.cuda.synchronize()
                t_prompts = time.perf_counter() - t0
        torch.cuda.synchronize()
        engine.manager.check_invariants()
        assert engine.manager.usage() == 0.0
        return t_prompts, time.perf_counter() - t0 - t_prompts, steps

    run()  # thrown away
    with ClockSampler() as clocks:
        t_prompts, t_decode, steps = run()
    del engine
    torch.cuda.empty_cache()
    parity = long_parity(args.parity_layers)
    print(json.dumps({
        "metric": "prompt tok/s, 16 requests of 7936 tokens (SmolLM2-135M sizes)",
        "value": round(16 * 7936 / t_prompts, 1), "unit": "tok/s", "n_gpus": 1,
        "higher_is_better": True, "dtype": "bf16", "impl": "ours",
        "decode_ms_per_step_b16_ctx8k": round(t_decode / 255 * 1e3, 4),
        "decode_tok_s": round(16 * 255 / t_decode, 1), "steps": steps,
        "data": "synthetic: uniform random token ids, random-init weights (seed 6); second of two runs",
        "config": {"model": "smollm2-135m sizes", "requests": 16, "prompt_len": 7936, "new_tokens": 255,
                   "max_model_len": 8192, "page_tokens": 16, "max_num_batched_tokens": 2048},
        "parity": parity, "clocks": clocks.summary(), "environment": environment()}))
    return 0


def long_parity(layers: int) -> dict:
    """float32 logits of one 8192-token sequence, whole and cut into portions and single tokens,
    against the plain implementation in float64 (``layers`` = 0: all of the model's layers)."""
    import tempfile

    import torch

    sys.path.insert(0, str(ROOT / "tests"))
    import plain_llama

    from llmserve_b200.config.registry import architecture_for
    from llmserve_b200.engine.batch import StepEntry
    from llmserve_b200.engine.runner import ModelRunner, load_model
    from llmserve_b200.models.hub import preset_config_dict
    from llmserve_b200.ops import get_ops
    from llmserve_b200.weights import write_random_model

    d = preset_config_dict("smollm2-135m")
    if layers:
        d["num_hidden_layers"] = layers
    cfg = architecture_for(d).config_cls.from_dict(d)
    N = 8192
    ids = random_prompts(1, N, cfg.vocab_size, 8)[0]
    rows = sorted(set(range(0, N, 509)) | set(range(N - 48, N)))
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(folder, cfg, seed=6)
        w = {k: v.to("cuda") for k, v in plain_llama.read_weights(folder, torch.float64).items()}
        want = plain_llama.forward(plain_llama.read_config(folder), w, ids, dtype=torch.float64,
                                   device="cuda", rows=rows)
        del w
        torch.cuda.empty_cache()
        _, _, model = load_model(folder, "float32", "cuda", get_ops("cuda"), N)
    out = {"layers": cfg.num_hidden_layers, "tokens": N, "rows_compared": len(rows),
           "largest_logit": round(float(want.abs().max()), 3)}
    for name, cuts in (("whole", [N]), ("portions_then_single", [2048, 2048, 2048, 1000, 1032] + [1] * 16)):
        runner = ModelRunner(model, page_tokens=16, num_pages=N // 16, max_model_len=N, max_num_seqs=2,
                             max_num_batched_tokens=N)
        got, a = [], 0
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for n in cuts:
            here = [r - a for r in rows if a <= r < a + n]
            logits = runner.run([StepEntry("x", ids[a : a + n], here)])
            if here:
                got.append(logits.double().cpu())
            a += n
        end.record()
        torch.cuda.synchronize()
        out[f"float32_{name}_vs_plain_max_abs_diff"] = float((torch.cat(got) - want).abs().max())
        # the true float32 path is the parity path (FFMA products, no tensor cores): its speed, for the record
        out[f"float32_{name}_ms"] = round(start.elapsed_time(end), 1)
    return out


# --------------------------------------------------------------------------- the reference
def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def reference_main(args) -> int:
    """The unmodified reference package, driven through its own ``LLMEngine.add_request`` / ``step``
    (src/llmserve/engine.py:83-156,219-264,308-408) on the decode workload. Nothing of this
    repository's package, extensions or tests is imported."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "llmserve" / "engine.py").exists():
        return unavailable("baseline/_ref holds no copy of the reference package (llmserve/)")
    if args.workload != "decode":
        return unavailable("the reference arm runs the decode workload only")
    sys.path[:] = [str(ref)] + [p for p in sys.path if p and Path(p).resolve() != ROOT]
    try:
        import torch
        from llmserve.config import ModelConfig
        from llmserve.engine import EngineConfig, LLMEngine
        from llmserve.models.transformer import CausalLM
        from llmserve.sampling import SamplingParams

        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        d = json.loads((ROOT / "llm-serving-engine_b200" / "config" / "presets" /
                        f"{args.model}.json").read_text())
        layers_full = d["num_hidden_layers"]
        args.layers = args.layers or layers_full
        d["num_hidden_layers"] = args.layers
        mcfg = ModelConfig.from_dict(d)
        torch.manual_seed(4)
        with torch.device("cuda"):
            model = CausalLM(mcfg, max_positions=CONTEXT).to(torch.bfloat16)
        with torch.no_grad():
            for name, p in model.named_parameters():
                if p.dim() >= 2:
                    p.normal_(0.0, 0.02)
                else:
                    p.normal_(0.0, 0.02).add_(1.0)
        model.rope.cos = model.rope.cos.float()
        model.rope.sin = model.rope.sin.float()
        model.eval()
        batch = args.batch
        warm = max(3, args.warmup)
        tokens_per_req = -(-(PROMPT_LEN + 2 * (args.steps + warm) + 64) // 16) * 16
        engine = LLMEngine(EngineConfig(
            dtype="bfloat16", device="cuda", block_size=16, max_model_len=CONTEXT, max_num_seqs=64,
            max_num_batched_tokens=PREFILL_TOKENS, num_kv_blocks=batch * tokens_per_req // 16),
            model=model, tokenizer=None)
        sp = SamplingParams(temperature=0.0, max_tokens=CONTEXT - PROMPT_LEN - 1, ignore_eos=True)
        for p in random_prompts(batch, PROMPT_LEN, mcfg.vocab_size, 1):
            engine.add_request(p, sp)
        while engine.scheduler.waiting or any(
                s.num_computed_tokens < s.num_prompt_tokens for s in engine.scheduler.running):
            engine.step()
        for _ in range(warm):
            engine.step()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler() as clocks:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            start.record()
            for _ in range(args.steps):
                out = engine.step()
            end.record()
            torch.cuda.synchronize()
            wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        dev_ms = start.elapsed_time(end) / args.steps
        assert engine.last_step.num_decode_tokens == batch and len(out) == batch
        ctx = max(s.num_tokens for s in engine.scheduler.running)
        # per step its runner uploads token ids, positions, write slots and the padded table of
        # cache rows with its mask, and downloads the float32 logits of every row
        h2d = batch * 8 * 4 + batch * ctx * (8 + 1)
        d2h = batch * mcfg.vocab_size * 4
    except Exception:  # noqa: BLE001
        return unavailable("the reference failed on this box: " +
                           traceback.format_exc().strip().splitlines()[-1][:300])
    print(json.dumps({
        "metric": METRIC, "value": round(batch * 1e3 / dev_ms, 1), "unit": "tok/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warm, "ms_per_step": round(dev_ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform random token ids, random-init weights (seed 4)",
        "impl": "reference",
        "config": {
            "model": f"{args.model} sizes", "layers": args.layers, "layers_full": layers_full,
            "hidden": mcfg.hidden_size, "heads": mcfg.num_attention_heads,
            "kv_heads": mcfg.num_key_value_heads, "head_dim": mcfg.head_dim,
            "intermediate": mcfg.intermediate_size, "vocab": mcfg.vocab_size,
            "global_batch": batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "decode_ctx": ctx,
            "page_tokens": 16, "parallelism": "single-gpu", "cuda_graphs": False,
            "l2": "inputs larger than L2 (weights + cache streamed each step)",
            "peaks": peaks()["source"]},
        "e2e": {"value": round(batch * 1e3 / wall_ms, 1), "unit": "tok/s",
                "ms_per_step": round(wall_ms, 4), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": 0,
        "note": "the reference's own engine, scheduler, runner and torch attention path on cuda; "
                "it has no GPU kernels of its own, so gpu_launches counts none",
        "clocks": clocks.summary()}))
    return 0


def main() -> int:
    global PROMPT_LEN, CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "continuous", "long"])
    ap.add_argument("--model", default="smollm2-1.7b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0 = all)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 and prefill points")
    ap.add_argument("--timeline", action="store_true",
                    help="add what each kernel adds to a captured step (from the profiler; not a timing run)")
    ap.add_argument("--parity", action="store_true",
                    help="also compare a two-layer model of the same layer sizes with the plain implementation")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN,
                    help="prompt length of the decode workload (the context grows from there)")
    ap.add_argument("--page-tokens", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--parity-layers", type=int, default=0,
                    help="layers of the float32 replay of --workload long (0 = all)")
    args = ap.parse_args()
    if args.prompt_len != PROMPT_LEN:  # another point of the same workload: longer or shorter contexts
        PROMPT_LEN = args.prompt_len
        CONTEXT = max(CONTEXT, -(-(PROMPT_LEN + 2 * (args.steps + args.warmup) + 128) // 1024) * 1024)
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print("bench.py: this engine runs on one GPU; --gpus > 1 is not built")
        return 2
    if args.impl == "reference":
        return reference_main(args)
    sys.path.insert(0, str(ROOT))
    return {"decode": decode_main, "continuous": continuous_main, "long": long_main}[args.workload](args)


if __name__ == "__main__":
    sys.exit(main())
