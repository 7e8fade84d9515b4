"""Interfaces that every part of a layer implements, and the registries that build them.

A model is put together from five kinds of part: norm, position encoding, mixer, feed-forward and
block (the arrangement of the other four around the residual stream). Each kind has a registry
from a ``kind`` string to a class. A part is described by a frozen *spec* dataclass that carries
its ``kind`` and every size and constant it needs; it never sees a model configuration and does
not know which model it is in.

Contract of a part class ``P`` registered under a kind:

* ``P(spec, env)``: ``env`` is a :class:`BuildEnv` (kernel set, compute dtype, device, longest
  position the engine will run).
* ``P.param_decls() -> dict[name, ParamDecl]``: the tensors it owns, with shape and role.
* ``P.bind(params)``: receives those tensors, already on the device, in the dtype that the role
  implies (see :func:`role_dtype`).
* a forward method whose signature depends on the kind (see each base class).

Parts that keep something per request also implement ``cache_need()`` (mixers only).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


# --------------------------------------------------------------------------- parameters
@dataclass(frozen=True)
class ParamDecl:
    """One tensor a part owns.

    role: ``matrix`` (a projection weight ``[out, in]``), ``embedding`` (``[vocab, width]``),
    ``bias`` or ``scale`` (a norm's per-channel weight). The role decides the random draw and the
    dtype on the device.
    """

    shape: tuple[int, ...]
    role: str = "matrix"


def role_dtype(role: str, compute_dtype: torch.dtype, stored: torch.dtype | None = None) -> torch.dtype:
    """Dtype a parameter has on the device.

    Projection, embedding and bias tensors feed matrix products and take the compute dtype.
    Per-channel scales are small and are read by 32-bit arithmetic, so they are held in float32
    (an exact widening of a bfloat16 file; a 32-bit file stays 32-bit). Integer tensors become
    int32.
    """
    if stored is not None and not stored.is_floating_point:
        return torch.int32
    if role == "scale":
        return torch.float32
    return compute_dtype


@dataclass
class BuildEnv:
    """What a part needs from the engine when it is built."""

    ops: Any  # the kernel set (llmserve_b200.ops.CudaOps on the product path)
    dtype: torch.dtype  # compute dtype: torch.bfloat16 or torch.float32
    device: torch.device
    max_positions: int  # longest sequence the engine will run (sizes position tables)
    branch_dtype: torch.dtype | None = None  # dtype of a branch's output before the residual add

    @property
    def residual_dtype(self) -> torch.dtype:
        """Dtype in which a mixer or feed-forward hands its result to the residual add."""
        return self.branch_dtype or self.dtype


# --------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class PagedKVNeed:
    """A mixer that keeps a key row and a value row per token, in pages.

    window: 0 keeps every token; ``w > 0`` means a query at position p reads keys p-w+1 .. p only,
    so pages that lie wholly before that range can be given back while the request is still live.
    """

    num_kv_heads: int
    head_dim: int
    window: int = 0
    kind: str = "paged_kv"
    dtype: object = None  # of the pages; None: the model's compute dtype (what the attention kernels here read)


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps one fixed-size tensor per request (a recurrent or convolution state)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32
    kind: str = "state"


# --------------------------------------------------------------------------- part base classes
class Part:
    kind: str = ""
    # True for a part whose forward reads ``step.host`` (the batch as host arrays) or otherwise
    # works from the host while the step runs: a model with such a part is never replayed as a
    # captured CUDA graph, where there is no host step and nothing may synchronise.
    needs_host_step: bool = False

    def __init__(self, spec: Any, env: BuildEnv) -> None:
        self.spec = spec
        self.env = env
        self.ops = env.ops

    def param_decls(self) -> dict[str, ParamDecl]:
        return {}

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        for name in self.param_decls():
            setattr(self, name.replace(".", "_"), params[name])


class Norm(Part):
    """``forward(x, residual, rows=None) -> h``.

    ``x`` is the float32 residual stream ``[T, H]``. If ``residual`` is given it is first added to
    ``x`` in place (in float32). Returns the normalised rows in the compute dtype. With ``rows``
    (int32 indices) only those rows are read and returned and ``x`` is left untouched.
    """

    def forward(self, x, residual=None, rows=None):  # pragma: no cover - interface
        raise NotImplementedError


class PositionEncoding(Part):
    """How positions enter the model. Two hooks, both optional:

    * ``rotary_tables() -> (cos, sin) | None``: float32 tables ``[max_positions, head_dim/2]``
      that the attention mixer applies to queries and keys when it writes them;
    * ``embed(x, positions)``: change the embedded tokens in place (absolute encodings).
    """

    def rotary_tables(self):
        return None

    def embed(self, x, positions) -> None:
        return None


class Mixer(Part):
    """Mixes information between the tokens of a request.

    ``forward(h, step, cache) -> [T, H]`` in the compute dtype (or float32). ``h`` holds the normed
    rows of this step's tokens only. ``step`` is the :class:`~llmserve_b200.engine.batch.DeviceStep`
    that describes the ragged batch. ``cache`` is the :class:`~llmserve_b200.cache.pools.CacheView`
    of the cache layer this run of the layer is bound to; ``cache.writes`` is False when the layer
    only reads a cache that an earlier layer filled.

    A mixer (or feed-forward) class with ``accepts_residual = True`` is also handed the float32
    residual stream as ``residual=x``; it may add its result into it and return None instead of
    returning the result. A block that can pass on a *pending* add also says ``may_defer=True``:
    the part may then return an object with a ``resolve()`` method (the kernel set's pending sums)
    which the block hands to the norm that reads ``x`` next, see :func:`settle`.

    ``cache_need()`` says what the mixer keeps per request (None for nothing).
    ``plan_step(host_step, group) -> dict[str, np.ndarray]`` may return int32 work lists that are
    the same for every layer with the same ``plan_key()``; the runner uploads them once per step
    and hands them back in ``step.plans[plan_key()]``. A mixer with work lists whose steps should
    also be captured as CUDA graphs when they hold portions of prompts gives the lists' largest
    sizes with ``plan_rows(single, portions, tokens) -> dict[str, int]`` (see
    ``PagedAttention.plan_rows``); without it such steps run uncaptured.
    """

    def cache_need(self):
        return None

    def plan_key(self):
        return None

    def reserve(self, max_seqs: int) -> None:
        """Allocate whatever scratch the mixer's kernels need for ``max_seqs`` sequences a step."""

    def plan_step(self, host_step, group):
        return {}

    def forward(self, h, step, cache):  # pragma: no cover - interface
        raise NotImplementedError


class FeedForward(Part):
    """``forward(h, step) -> [T, H]``: works on each token alone."""

    def forward(self, h, step):  # pragma: no cover - interface
        raise NotImplementedError


class Block(Part):
    """Arranges norm, mixer and feed-forward around the residual stream.

    ``forward(x, pending, step, cache) -> (x, pending)``: ``x`` is the float32 residual stream,
    updated in place; ``pending`` is a branch output that has not been added to ``x`` yet (or
    None), so that the add can be fused into whichever norm reads ``x`` next.
    """

    def __init__(self, spec: Any, env: BuildEnv) -> None:
        super().__init__(spec, env)
        self.children: dict[str, Part] = {}

    def param_decls(self) -> dict[str, ParamDecl]:
        out = {}
        for cname, child in self.children.items():
            for pname, decl in child.param_decls().items():
                out[f"{cname}.{pname}"] = decl
        return out

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        for cname, child in self.children.items():
            prefix = cname + "."
            child.bind({k[len(prefix):]: v for k, v in params.items() if k.startswith(prefix)})

    def mixer_part(self) -> Mixer | None:
        m = self.children.get("mixer")
        return m if isinstance(m, Mixer) else None

    def forward(self, x, pending, step, cache):  # pragma: no cover - interface
        raise NotImplementedError


def project_into(ops, a, w, bias, out_dtype, residual, may_defer: bool = False):
    """A branch's output projection ``a @ w.T (+ bias)``: added into ``residual`` (the float32
    stream) where one is given. Returns None (added), the product, or pending sums (only if
    ``may_defer``)."""
    if residual is None:
        return ops.linear(a, w, bias, out_dtype=out_dtype)
    if may_defer and getattr(ops, "defers_adds", False):
        return ops.linear(a, w, bias, out_dtype=out_dtype, accumulate_into=residual, may_defer=True)
    return ops.linear(a, w, bias, out_dtype=out_dtype, accumulate_into=residual)


def settle(pending, norm):
    """What ``norm`` can take as its ``residual``: pending sums are handed on only to a norm that
    declares ``takes_pending_sums``; for any other they are added now."""
    if hasattr(pending, "resolve") and not getattr(norm, "takes_pending_sums", False):
        return pending.resolve()
    return pending


# --------------------------------------------------------------------------- registries
@dataclass
class Registry:
    what: str
    classes: dict[str, type] = field(default_factory=dict)

    def register(self, kind: str) -> Callable[[type], type]:
        def deco(cls: type) -> type:
            if kind in self.classes and self.classes[kind] is not cls:
                raise KeyError(f"{self.what} kind {kind!r} is already registered")
            cls.kind = kind
            self.classes[kind] = cls
            return cls

        return deco

    def unregister(self, kind: str) -> None:
        self.classes.pop(kind, None)

    def build(self, spec: Any, env: BuildEnv) -> Any:
        kind = getattr(spec, "kind", None)
        if kind not in self.classes:
            raise KeyError(f"no {self.what} registered under {kind!r}; known: {sorted(self.classes)}")
        return self.classes[kind](spec, env)


NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")
