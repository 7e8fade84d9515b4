"""Read a model folder's safetensors files by tensor name into model parameters.

Behaviour follows src/llmserve/models/loader.py:27-85 (every ``*.safetensors`` in the folder,
q|k|v and gate|up concatenated along dim 0, a tied output projection not read from the file), with
one difference: the file set is checked against the architecture's layout *before* anything is
copied, and every problem is reported in a single :class:`CheckpointError` that lists the missing
tensors, the unexpected tensors and the tensors with a wrong shape.

Dtypes: a parameter that feeds a matrix product takes the compute dtype (bfloat16 files stay
bfloat16 in the bfloat16 path and are widened exactly for the float32 path); per-channel scales are
held in float32; integer tensors become int32.
"""

from __future__ import annotations

from pathlib import Path

import torch
from safetensors import safe_open

from ..models.plan import CheckpointLayout
from ..parts.base import role_dtype

_ST_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}


class CheckpointError(ValueError):
    """The checkpoint does not hold what the model needs."""

    def __init__(self, path, missing, unexpected, wrong_shape):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        lines = [f"checkpoint {path} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(
                f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected)
            )
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}):")
            lines += [f"    {n}: file has {got}, model needs {want}" for n, got, want in self.wrong_shape]
        super().__init__("\n".join(lines))


def checkpoint_index(path: str | Path) -> dict[str, tuple[Path, tuple[int, ...], str]]:
    """tensor name -> (file, shape, safetensors dtype string) over every safetensors file."""
    path = Path(path)
    files = sorted(path.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {path}")
    index: dict[str, tuple[Path, tuple[int, ...], str]] = {}
    for f in files:
        with safe_open(str(f), framework="pt") as fh:
            for name in fh.keys():  # noqa: SIM118
                sl = fh.get_slice(name)
                index[name] = (f, tuple(sl.get_shape()), str(sl.get_dtype()))
    return index


def check_layout(path, index, layout: CheckpointLayout) -> None:
    expected = {s.name: s.shape for e in layout.entries for s in e.sources}
    missing = [n for n in expected if n not in index]
    unexpected = [
        n
        for n in index
        if n not in expected
        and n not in layout.ignored_names
        and not any(sub in n for sub in layout.ignored_substrings)
    ]
    wrong = [
        (n, index[n][1], tuple(shape))
        for n, shape in expected.items()
        if n in index and tuple(index[n][1]) != tuple(shape)
    ]
    if missing or unexpected or wrong:
        raise CheckpointError(path, missing, unexpected, wrong)


def load_parameters(
    path: str | Path,
    layout: CheckpointLayout,
    compute_dtype: torch.dtype,
    device: torch.device | str,
) -> dict[str, torch.Tensor]:
    """Model parameter name -> tensor on ``device``."""
    path = Path(path)
    index = checkpoint_index(path)
    check_layout(path, index, layout)
    handles: dict[Path, object] = {}
    out: dict[str, torch.Tensor] = {}
    try:
        for entry in layout.entries:
            parts = []
            for s in entry.sources:
                f = index[s.name][0]
                if f not in handles:
                    handles[f] = safe_open(str(f), framework="pt").__enter__()
                parts.append(handles[f].get_tensor(s.name))
            stored = parts[0].dtype
            want = role_dtype(entry.role, compute_dtype, stored)
            t = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
            out[entry.param] = t.to(device=device, dtype=want).contiguous()
    finally:
        for h in handles.values():
            h.__exit__(None, None, None)
    return out
