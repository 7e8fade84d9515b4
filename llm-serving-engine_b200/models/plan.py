"""What a model is, as data: a list of layer specs and the order in which they run."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True)
class RunEntry:
    """One run of a layer.

    layer: index into ``ModelPlan.layers`` (a layer may be named by several entries: its weights
    are then shared). cache: id of the cache layer this run uses. The first entry in the run order
    that names a cache id fills it; later entries with the same id only read it (they compute
    their own queries and write nothing).
    """

    layer: int
    cache: int


@dataclass(frozen=True)
class ModelPlan:
    vocab_size: int
    hidden_size: int
    layers: tuple[Any, ...]  # block specs
    run_order: tuple[RunEntry, ...]
    final_norm: Any  # norm spec
    tie_head: bool
    embed_position: Any = None  # position-encoding spec applied to the embedded tokens, or None
    # constants that some architectures put around the stack of layers (all off by default):
    embed_scale: float = 1.0  # the embedded tokens are multiplied by this
    logit_scale: float = 1.0  # the logits are multiplied by this ...
    logit_softcap: float = 0.0  # ... and then, if > 0, squashed to cap * tanh(logits / cap)

    def validate(self) -> None:
        if not self.run_order:
            raise ValueError("run_order is empty")
        for e in self.run_order:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"run_order names layer {e.layer}; the plan has {len(self.layers)}")
        ids = sorted({e.cache for e in self.run_order})
        if ids != list(range(len(ids))):
            raise ValueError(f"cache ids must be 0..n-1 without gaps, got {ids}")


@dataclass(frozen=True)
class Source:
    name: str  # tensor name in the checkpoint
    shape: tuple[int, ...]


@dataclass(frozen=True)
class ParamSource:
    """A model parameter and the checkpoint tensors it is made of (concatenated along dim 0)."""

    param: str
    sources: tuple[Source, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class CheckpointLayout:
    entries: tuple[ParamSource, ...]
    ignored_substrings: tuple[str, ...] = ()  # tensors that may be present and are not read
    ignored_names: tuple[str, ...] = ()
