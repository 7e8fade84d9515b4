"""Helpers shared by the GPU tests."""

from __future__ import annotations

from conftest import TINY

# Tolerances.
#   float32: the engine and the plain model differ only in the order of float32 additions.
#   bfloat16: activations are rounded to 8 bits of mantissa between kernels (about 6 roundings per
#   layer); the bound is 2 % of the largest logit of the compared requests. (It was 3 % before the
#   first GPU run; measured since: at most 0.8 % on the tiny configurations, 0.9 % at SmolLM2-1.7B
#   layer widths, 1.5 % with the sharpened attention of tests/test_gpu_widths.py, so it was tightened.)
F32_ATOL = 2e-5
BF16_RTOL = 0.02


def tolerances(dtype):
    return (F32_ATOL, 0.0) if dtype == "float32" else (0.0, BF16_RTOL)


def gpu_runner(folder, name, num_pages, dtype, max_num_seqs=4, page_tokens=None, **kw):
    from llmserve_b200.engine.runner import ModelRunner, load_model
    from llmserve_b200.ops import get_ops

    cfg = TINY[name]
    ops = get_ops("cuda")
    _, _, model = load_model(folder, dtype, "cuda", ops, cfg["max_position_embeddings"])
    return ModelRunner(model, page_tokens=page_tokens or cfg["page_tokens"], num_pages=num_pages,
                       max_model_len=cfg["max_position_embeddings"], max_num_seqs=max_num_seqs, **kw)


def expected_logits(folder, reqs):
    import plain_llama

    return {r: plain_llama.model_logits(folder, t) for r, t in reqs.items()}
