"""Random-weights mode: make a model folder (config.json, model.safetensors) from a configuration
and a seed, or draw the same parameters straight onto a device.

Draws: projection and embedding tensors N(0, 0.02^2); norm scales 1 + N(0, 0.02^2); biases
N(0, 0.02^2). Every checkpoint tensor is drawn on the CPU in float32 from one generator, in the
order of the architecture's checkpoint layout, and then rounded to the storage dtype, so a folder
written twice from the same configuration and seed is identical, and the float32 path and any
independent implementation that read the folder see the same values as the bfloat16 path.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any

import torch
from safetensors.torch import save_file

from ..parts.base import role_dtype

STD = 0.02


def _draw(shape, role: str, gen: torch.Generator, device="cpu") -> torch.Tensor:
    t = torch.randn(tuple(shape), generator=gen, dtype=torch.float32, device=device) * STD
    return t + 1.0 if role == "scale" else t


def random_checkpoint_tensors(arch, cfg, seed: int, store_dtype=torch.bfloat16):
    """Checkpoint tensor name -> CPU tensor, as it would be stored."""
    gen = torch.Generator().manual_seed(seed)
    layout = arch.checkpoint_layout(cfg)
    return {
        s.name: _draw(s.shape, e.role, gen).to(store_dtype).contiguous()
        for e in layout.entries
        for s in e.sources
    }


def write_random_model(
    folder: str | Path, config: Any, seed: int, store_dtype: torch.dtype = torch.bfloat16
) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed config object)."""
    from ..config.registry import ARCHITECTURES

    arch = ARCHITECTURES[config.architecture]
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=1))
    tensors = random_checkpoint_tensors(arch, config, seed, store_dtype)
    save_file(tensors, str(folder / "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    return folder


def random_parameters(arch, cfg, seed: int, compute_dtype, device) -> dict[str, torch.Tensor]:
    """Model parameters drawn directly on ``device`` (no folder; for benchmarks at full size).

    Same distributions as :func:`write_random_model`; the values differ from a folder written
    with the same seed because the generator is the device's.
    """
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(seed)
    layout = arch.checkpoint_layout(cfg)
    out = {}
    for e in layout.entries:
        parts = [_draw(s.shape, e.role, gen, device).to(torch.bfloat16) for s in e.sources]
        t = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
        out[e.param] = t.to(role_dtype(e.role, compute_dtype)).contiguous()
    return out
