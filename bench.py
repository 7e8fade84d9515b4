"""Decode and prefill throughput of the engine at SmolLM2-1.7B sizes, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

A "step" is one decode step of the whole model (forward of one token per request from the paged
cache, output projection and sampling). ``value`` is decoded tokens per second from CUDA-event
timing of exactly K steps replayed back to back; ``e2e`` is the same workload driven through
``LLMEngine.step()`` (scheduler, pinned host buffer -> device copy of the step's inputs, the step,
device -> host read of the sampled token ids) by wall clock. One JSON line is printed.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_LEN = 2048
CONTEXT = 4096
PREFILL_TOKENS = 2048


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


def model_numbers(cfg, layers: int) -> dict:
    h, i, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv = cfg.q_size, cfg.kv_size
    layer_params = h * (q + 2 * kv) + q * h + 3 * h * i
    weight_bytes = 2 * (layers * (layer_params + 2 * h) + h + v * h)  # every weight read once a step
    kv_bytes_per_token = 2 * layers * kv * 2
    T = PREFILL_TOKENS
    prefill_flops = 2 * T * layers * layer_params + 2 * h * v  # one logits row
    prefill_flops += 4 * layers * cfg.num_attention_heads * cfg.head_dim * T * (T + 1) // 2
    return dict(weight_bytes=weight_bytes, kv_bytes_per_token=kv_bytes_per_token,
                prefill_flops=prefill_flops)


def make_engine(args, layers_full: int):
    from llmserve_b200 import EngineConfig, LLMEngine

    over = {"num_hidden_layers": args.layers} if args.layers != layers_full else None
    max_b = max(64, args.batch)
    tokens_per_req = -(-(PROMPT_LEN + 2 * (args.steps + args.warmup) + 64) // 16) * 16
    return LLMEngine(EngineConfig(
        model=f"random:{args.model}", dtype="bfloat16", seed=4, block_size=16,
        num_kv_blocks=max_b * tokens_per_req // 16, max_model_len=CONTEXT, max_num_seqs=max_b,
        max_num_batched_tokens=PREFILL_TOKENS, config_overrides=over))


def random_prompts(n, length, vocab, seed):
    import torch

    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n, length), generator=g).tolist()


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


def measure_decode(engine, batch, steps, warmup, seed):
    """Returns (device ms per step, e2e ms per step, launches per step, h2d, d2h bytes per step)."""
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
    g = max((x for x in graphs.values() if x.batch == batch and x.slots == 0 and x.graph is not None),
            key=lambda x: x.step.decode_splits)
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
    ctx = max(s.num_tokens for s in engine.scheduler.running)
    for i in ids:
        engine.abort_request(i)
    return dict(dev_ms=dev_ms, e2e_ms=e2e_ms, launches=g.launches, h2d=h2d, d2h=d2h, ctx=ctx)


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


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="smollm2-1.7b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0 = all)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 and prefill points")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference cannot be installed offline: its build backend (hatchling) is "
                          "not in /opt/wheelhouse; it also has no GPU code path of its own"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print("bench.py: this engine runs on one GPU; --gpus > 1 is not built")
        return 2

    import torch

    from llmserve_b200.config.registry import architecture_for
    from llmserve_b200.models.hub import preset_config_dict

    d = preset_config_dict(args.model)
    cfg = architecture_for(d).config_cls.from_dict(d)
    layers_full = cfg.num_hidden_layers
    args.layers = args.layers or layers_full
    pk = peaks()
    nums = model_numbers(cfg, args.layers)
    engine = make_engine(args, layers_full)
    with ClockSampler() as clocks:
        main_pt = measure_decode(engine, args.batch, args.steps, args.warmup, seed=1)
    value = args.batch * 1e3 / main_pt["dev_ms"]
    bytes_step = nums["weight_bytes"] + args.batch * main_pt["ctx"] * nums["kv_bytes_per_token"]
    achieved = bytes_step / (main_pt["dev_ms"] * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s @ batch 8 (SmolLM2-1.7B sizes, 2048-token prompts)",
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
            "decode_ctx": main_pt["ctx"], "page_tokens": 16, "parallelism": "single-gpu",
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
            by = nums["weight_bytes"] + b * r["ctx"] * nums["kv_bytes_per_token"]
            pts[f"decode_b{b}_hbm_frac"] = round(by / (r["dev_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        line["points"] = pts
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
