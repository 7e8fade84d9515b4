"""``llmserve_b200 generate``: generate from the command line and report the speed.

The options that the reference's command has (src/llmserve/generate_cli.py:13-20) keep their names,
defaults and meanings: prompts as positional arguments, ``--model``, ``--chat``, ``--max-tokens``
(64), ``--temperature`` (0 = greedy), ``--top-p``, ``--seed``. Added: prompts as token ids for
folders without a tokenizer, and the engine's dtype, cache and batching options.
"""

from __future__ import annotations

import argparse
import time

ENGINE_OPTIONS = ("dtype", "block_size", "num_kv_blocks", "kv_cache_memory_gb", "max_model_len",
                  "max_num_seqs", "max_num_batched_tokens", "profile")


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="llmserve_b200 generate")
    ap.add_argument("prompt", nargs="*", help="text prompts (need a tokenizer in the model folder)")
    ap.add_argument("--prompt-ids", action="append", default=[], metavar="ID,ID,...",
                    help="a prompt as comma-separated token ids (may be given several times)")
    ap.add_argument("--model", default="smollm2-135m",
                    help="model folder, alias under $LLMSERVE_MODELS, or random:<alias>")
    ap.add_argument("--chat", action="store_true", help="apply the model's chat template")
    sampling = ap.add_argument_group("sampling")
    sampling.add_argument("--max-tokens", type=int, default=64)
    sampling.add_argument("--temperature", type=float, default=0.0)
    sampling.add_argument("--top-p", type=float, default=1.0)
    sampling.add_argument("--seed", type=int, default=None)
    sampling.add_argument("--ignore-eos", action="store_true")
    eng = ap.add_argument_group("engine")
    eng.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    eng.add_argument("--block-size", type=int, default=16)
    eng.add_argument("--num-kv-blocks", type=int, default=None)
    eng.add_argument("--kv-cache-memory-gb", type=float, default=2.0)
    eng.add_argument("--max-model-len", type=int, default=4096)
    eng.add_argument("--max-num-seqs", type=int, default=64)
    eng.add_argument("--max-num-batched-tokens", type=int, default=1024)
    eng.add_argument("--profile", action="store_true",
                     help="time every step on the device (CUDA events) and mark it with an NVTX range")
    return ap


def main(argv: list[str] | None = None) -> None:
    ap = parser()
    args = ap.parse_args(argv)
    prompts: list = [*args.prompt, *([int(t) for t in ids.split(",")] for ids in args.prompt_ids)]
    if not prompts:
        ap.error("give a prompt or --prompt-ids")

    from .engine import LLM
    from .sampling import SamplingParams

    llm = LLM(args.model, **{name: getattr(args, name) for name in ENGINE_OPTIONS})
    how = SamplingParams(temperature=args.temperature, top_p=args.top_p, max_tokens=args.max_tokens,
                         seed=args.seed, ignore_eos=args.ignore_eos)
    started = time.monotonic()
    if args.chat:
        results = llm.chat([[{"role": "user", "content": p}] for p in prompts], how)
    else:
        results = llm.generate(prompts, how)
    seconds = time.monotonic() - started
    total = 0
    for prompt, result in zip(prompts, results, strict=True):
        out = result.outputs[0]
        total += len(out.token_ids)
        print(f"### {prompt}")
        print(out.text if llm.tokenizer is not None else " ".join(str(t) for t in out.token_ids))
        print()
    print(f"[{total} tokens in {seconds:.2f}s, {total / seconds:.1f} tok/s]")
    if args.profile:
        st = llm.engine.last_step
        device = "n/a" if st.gpu_ms is None else f"{st.gpu_ms:.3f} ms"
        print(f"[last step: schedule {st.t_schedule * 1e3:.3f} ms, launch {st.t_forward * 1e3:.3f} ms, "
              f"wait and read {st.t_sample * 1e3:.3f} ms, host {st.t_postprocess * 1e3:.3f} ms, device {device}]")


if __name__ == "__main__":
    main()
