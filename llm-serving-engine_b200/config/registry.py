"""One registry from an architecture's name to everything needed to build its model.

The name is ``config.json["architectures"][0]``; files without that key are matched on
``model_type``. An :class:`Architecture` gives the typed config class, a function from that config
to a :class:`~llmserve_b200.models.plan.ModelPlan` (the layers as data) and a function to the
:class:`~llmserve_b200.models.plan.CheckpointLayout` (which checkpoint tensors make up which model
parameter). Registering another architecture is one ``register_architecture`` call.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable


@dataclass(frozen=True)
class Architecture:
    name: str
    model_type: str
    config_cls: Any  # has from_dict / from_pretrained / to_dict
    plan: Callable[[Any], Any]
    checkpoint_layout: Callable[[Any], Any]


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    ARCHITECTURES[arch.name] = arch


def architecture_for(config_dict: dict[str, Any]) -> Architecture:
    names = config_dict.get("architectures") or []
    for n in names:
        if n in ARCHITECTURES:
            return ARCHITECTURES[n]
    mt = config_dict.get("model_type")
    if not names:
        for arch in ARCHITECTURES.values():
            if arch.model_type == mt:
                return arch
    raise KeyError(
        f"no architecture registered for architectures={names} model_type={mt!r}; "
        f"known: {sorted(ARCHITECTURES)}"
    )


def load_model_config(path: str | Path) -> tuple[Architecture, Any]:
    """Read ``path/config.json`` and return (architecture, typed config)."""
    path = Path(path)
    f = path / "config.json"
    if not f.exists():
        raise FileNotFoundError(f"{f} not found")
    arch = architecture_for(json.loads(f.read_text()))
    return arch, arch.config_cls.from_pretrained(path)


def _register_builtin() -> None:
    from ..models.llama import llama_checkpoint_layout, llama_plan
    from .llama import LlamaConfig

    register_architecture(
        Architecture(
            name="LlamaForCausalLM",
            model_type="llama",
            config_cls=LlamaConfig,
            plan=llama_plan,
            checkpoint_layout=llama_checkpoint_layout,
        )
    )


_register_builtin()
