"""The plain implementation against the reference's stored logits, and its own parts."""

from pathlib import Path

import pytest
import torch
from safetensors.torch import load_file

import plain_llama

GOLDEN = Path(__file__).parent / "golden" / "tiny_llama_reference_logits.safetensors"


@pytest.mark.parametrize("case", ["gqa_tied", "mqa_untied", "bias_d64", "rope_linear", "rope_llama3"])
def test_plain_matches_reference_logits(case, tmp_path):
    """The plain implementation against logits that the reference's own model code produced
    (tests/golden/make_golden.py). The golden file carries the weights and the config of each case,
    so nothing here depends on which random numbers this torch draws."""
    import json

    from safetensors import safe_open
    from safetensors.torch import save_file

    with safe_open(str(GOLDEN), framework="pt") as f:
        config = json.loads(f.metadata()["configs"])[case]
    gold = load_file(str(GOLDEN))
    prefix = f"{case}.weights."
    weights = {k[len(prefix):]: v for k, v in gold.items() if k.startswith(prefix)}
    assert weights, "the golden file holds no weights for this case"
    (tmp_path / "config.json").write_text(json.dumps(config))
    save_file(weights, str(tmp_path / "model.safetensors"))
    logits = plain_llama.model_logits(tmp_path, gold[f"{case}.ids"].tolist())
    assert logits.shape == gold[f"{case}.logits"].shape
    assert (logits - gold[f"{case}.logits"]).abs().max() < 1e-5


def test_rms_norm_formula():
    x = torch.randn(5, 48, dtype=torch.float64)
    w = torch.randn(48, dtype=torch.float64)
    y = plain_llama.rms_norm(x, w, 1e-5)
    for t in range(5):
        ref = x[t] / (x[t].pow(2).sum() / 48 + 1e-5).sqrt() * w
        assert torch.allclose(y[t], ref, atol=1e-12)


def test_rope_is_a_rotation_and_relative():
    D = 32
    q = torch.randn(6, 2, D, dtype=torch.float64)
    k = torch.randn(6, 2, D, dtype=torch.float64)

    def scores(offset):
        pos = torch.arange(6) + offset
        c, s = plain_llama.rope_tables(pos, D, 10000.0, None, torch.float64)
        qr, kr = plain_llama.apply_rope(q, c, s), plain_llama.apply_rope(k, c, s)
        assert torch.allclose(qr.norm(dim=-1), q.norm(dim=-1), atol=1e-10)
        return torch.einsum("thd,shd->hts", qr, kr)

    assert torch.allclose(scores(0), scores(37), atol=1e-9)  # depends on distance only


def test_attention_causal_window_and_groups():
    T, D = 9, 16
    q = torch.randn(T, 4, D, dtype=torch.float64)
    k = torch.randn(T, 2, D, dtype=torch.float64)
    v = torch.randn(T, 2, D, dtype=torch.float64)
    o = plain_llama.attention(q, k, v, 0.25)
    for t in (0, 4, 8):
        for h in range(4):
            s = (k[: t + 1, h // 2] @ q[t, h]) * 0.25
            ref = s.softmax(0) @ v[: t + 1, h // 2]
            assert torch.allclose(o[t, h], ref, atol=1e-12)
    ow = plain_llama.attention(q, k, v, 0.25, window=3)
    t, h = 7, 3
    s = (k[5:8, 1] @ q[t, h]) * 0.25
    assert torch.allclose(ow[t, h], s.softmax(0) @ v[5:8, 1], atol=1e-12)


def test_forward_is_causal(tiny_dirs):
    ids = torch.randint(0, 256, (20,), generator=torch.Generator().manual_seed(5)).tolist()
    full = plain_llama.model_logits(tiny_dirs["A"], ids)
    part = plain_llama.model_logits(tiny_dirs["A"], ids[:11])
    assert (full[:11] - part).abs().max() < 1e-5


def test_the_two_plain_samplers_agree():
    """The all-pairs rule and its sorted form keep the same elements and draw the same tokens."""
    import torch

    from plain_ops import PlainOps

    R, V = 8, 611
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(R, V, generator=g) * 2
    logits[2] = (logits[2] * 2).round() / 2
    logits[3, ::5] = float("-inf")
    f = lambda v, dt: torch.full((R,), v, dtype=dt)
    for k, tp, mp, t in [(0, 1.0, 0.0, 1.0), (7, 1.0, 0.0, 0.8), (0, 0.6, 0.0, 1.3), (40, 0.9, 0.05, 0.7),
                         (1, 1.0, 0.0, 1.0), (0, 0.0, 0.0, 1.0)]:
        args = (f(t, torch.float32), f(k, torch.int32), f(tp, torch.float32), f(mp, torch.float32),
                torch.arange(R) * 31 + 1, torch.arange(R, dtype=torch.int32))
        assert PlainOps().sample(logits, *args).tolist() == PlainOps().sample_sorted(logits, *args).tolist()
