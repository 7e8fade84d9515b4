"""Where model folders are found.

A model is named by a folder path, by an alias, or by ``random:<alias>`` (random weights of that
alias's sizes, drawn on the device). Aliases are the reference's short names
(src/llmserve/models/hub.py:14-20); their folders are looked up under ``$LLMSERVE_MODELS`` (default
``./models``). Nothing is downloaded: a missing folder is an error that says where it was sought.
"""

from __future__ import annotations

import json
import os
from pathlib import Path

PRESETS = Path(__file__).resolve().parent.parent / "config" / "presets"


def aliases() -> list[str]:
    return sorted(p.stem for p in PRESETS.glob("*.json"))


def preset_config_dict(alias: str) -> dict:
    f = PRESETS / f"{alias}.json"
    if not f.exists():
        raise KeyError(f"no size preset {alias!r}; known: {aliases()}")
    return json.loads(f.read_text())


def models_dir() -> Path:
    return Path(os.environ.get("LLMSERVE_MODELS", Path.cwd() / "models"))


def resolve_model_path(name_or_path: str) -> Path:
    p = Path(name_or_path)
    if p.is_dir():
        return p
    local = models_dir() / name_or_path.replace("/", "--")
    if (local / "config.json").exists() and any(local.glob("*.safetensors")):
        return local
    raise FileNotFoundError(
        f"model {name_or_path!r}: neither a folder nor found at {local} "
        f"(set LLMSERVE_MODELS, or use 'random:<alias>' with one of {aliases()})"
    )
