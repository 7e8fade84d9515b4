"""``llmserve_b200 generate``: quick generation from the command line.

Options of the reference's command (src/llmserve/generate_cli.py:13-20) keep their names and
meanings: positional prompts, ``--model``, ``--chat``, ``--max-tokens``, ``--temperature``
(0 = greedy), ``--top-p``, ``--seed``. Added here: token-id prompts for folders without a
tokenizer, and the engine's dtype and cache options.
"""

from __future__ import annotations

import argparse
import time


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(prog="llmserve_b200 generate")
    ap.add_argument("prompt", nargs="*")
    ap.add_argument("--model", default="smollm2-135m",
                    help="model folder, alias under $LLMSERVE_MODELS, or random:<alias>")
    ap.add_argument("--chat", action="store_true", help="apply the model's chat template")
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--prompt-ids", action="append", default=[],
                    help="a prompt as comma-separated token ids (may be given several times)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--num-kv-blocks", type=int, default=None)
    ap.add_argument("--kv-cache-memory-gb", type=float, default=2.0)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--max-num-batched-tokens", type=int, default=1024)
    ap.add_argument("--ignore-eos", action="store_true")
    args = ap.parse_args(argv)

    from .engine import LLM
    from .sampling import SamplingParams

    prompts: list = list(args.prompt) + [[int(t) for t in s.split(",")] for s in args.prompt_ids]
    if not prompts:
        ap.error("give a prompt or --prompt-ids")
    llm = LLM(args.model, dtype=args.dtype, block_size=args.block_size,
              num_kv_blocks=args.num_kv_blocks, kv_cache_memory_gb=args.kv_cache_memory_gb,
              max_model_len=args.max_model_len, max_num_seqs=args.max_num_seqs,
              max_num_batched_tokens=args.max_num_batched_tokens)
    sp = SamplingParams(temperature=args.temperature, top_p=args.top_p, max_tokens=args.max_tokens,
                        seed=args.seed, ignore_eos=args.ignore_eos)
    t = time.monotonic()
    if args.chat:
        outs = llm.chat([[{"role": "user", "content": p}] for p in prompts], sp)
    else:
        outs = llm.generate(prompts, sp)
    dt = time.monotonic() - t
    n = 0
    for p, o in zip(prompts, outs, strict=True):
        c = o.outputs[0]
        n += len(c.token_ids)
        shown = c.text if llm.tokenizer is not None else " ".join(map(str, c.token_ids))
        print(f"### {p}\n{shown}\n")
    print(f"[{n} tokens in {dt:.2f}s, {n / dt:.1f} tok/s]")


if __name__ == "__main__":
    main()
