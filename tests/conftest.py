"""Shared fixtures: tiny random-weight Llama folders, written fresh into a temporary folder."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

# Tiny configurations that differ in every size and option.
TINY = {
    "A": dict(vocab_size=256, hidden_size=64, intermediate_size=160, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, rope_theta=10000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=256, seed=0,
              page_tokens=16),
    "B": dict(vocab_size=384, hidden_size=128, intermediate_size=352, num_hidden_layers=3,
              num_attention_heads=4, num_key_value_heads=1, head_dim=32, rope_theta=100000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=512, seed=2,
              page_tokens=8),
    # head size 64 (the tensor-core attention path), three query heads per key head, widths that
    # are no power of two, untied head, attention biases
    "C": dict(vocab_size=515, hidden_size=192, intermediate_size=272, num_hidden_layers=2,
              num_attention_heads=6, num_key_value_heads=2, head_dim=64, rope_theta=50000.0,
              rms_norm_eps=3e-6, tie_word_embeddings=False, attention_bias=True,
              max_position_embeddings=1024, seed=7, page_tokens=32),
}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def tiny_config(name: str):
    from llmserve_b200.config import LlamaConfig

    d = {k: v for k, v in TINY[name].items() if k not in ("seed", "page_tokens")}
    return LlamaConfig.from_dict({"model_type": "llama", **d})


@pytest.fixture(scope="session")
def tiny_dirs(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (bfloat16 storage)."""
    from llmserve_b200.weights import write_random_model

    out = {}
    for name, spec in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny-{name}")
        write_random_model(d, tiny_config(name), spec["seed"])
        out[name] = d
    return out


@pytest.fixture(scope="session")
def sharp_dirs(tmp_path_factory):
    """Same shapes, weights scaled up so that logits are far from flat (argmax ties unlikely)."""
    from safetensors.torch import load_file, save_file

    from llmserve_b200.weights import write_random_model

    out = {}
    for name, spec in TINY.items():
        d = tmp_path_factory.mktemp(f"sharp-{name}")
        write_random_model(d, tiny_config(name), spec["seed"] + 100)
        f = d / "model.safetensors"
        t = load_file(str(f))
        t = {k: (v.float() * 6).to(v.dtype) if v.dim() > 1 else v for k, v in t.items()}
        save_file(t, str(f))
        out[name] = d
    return out
