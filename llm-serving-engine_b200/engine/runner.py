"""The step function: run one ragged batch through the model from the cache.

``ModelRunner.step(entries)`` takes ``(request, its next tokens, wanted places)`` entries
(portions of prompts beside single decoded tokens, cut anywhere), runs exactly those tokens as one
batch against what earlier steps left in the cache, writes their keys and values, and returns
float32 logits for the wanted places only. It is what the reference calls
``ModelRunner.execute`` (src/llmserve/model_runner.py:39-87). Pages must have been allocated for the
new tokens before the call (``manager.allocate``) and are committed after it (``manager.commit``);
:meth:`ModelRunner.run` does both around a step for callers without a scheduler.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Sequence

import numpy as np
import torch

from ..cache import CacheManager, CachePools, group_cache_layers, pages_for_memory
from ..config.registry import load_model_config
from ..models.decoder import DecoderModel
from ..parts.base import BuildEnv
from ..weights.loader import load_parameters
from .batch import DeviceStep, HostStep, StepEntry, build_host_step

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def resolve_dtype(dtype: str | torch.dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    if dtype not in DTYPES:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {dtype!r}")
    return DTYPES[dtype]


def build_model(arch, cfg, params_fn, dtype, device, ops, max_positions) -> DecoderModel:
    """Assemble the architecture's plan into a model and bind parameters from ``params_fn``."""
    dtype = resolve_dtype(dtype)
    env = BuildEnv(ops=ops, dtype=dtype, device=torch.device(device), max_positions=max_positions,
                   branch_dtype=ops.branch_dtype(dtype))
    model = DecoderModel(arch.plan(cfg), env)
    model.bind(params_fn(arch.checkpoint_layout(cfg), dtype, device))
    return model


def load_model(path: str | Path, dtype, device, ops, max_positions: int):
    """Read ``path`` (config.json + safetensors); the model class follows config.json."""
    arch, cfg = load_model_config(path)
    model = build_model(
        arch, cfg, lambda layout, dt, dev: load_parameters(path, layout, dt, dev),
        dtype, device, ops, max_positions,
    )
    return arch, cfg, model


class ModelRunner:
    def __init__(
        self,
        model: DecoderModel,
        *,
        page_tokens: int = 16,
        num_pages: int | Sequence[int] | None = None,
        cache_memory_bytes: int | None = None,
        max_model_len: int = 4096,
        max_num_seqs: int = 64,
        max_num_batched_tokens: int = 1024,
    ) -> None:
        self.model = model
        self.ops = model.ops
        self.device = model.env.device
        self.dtype = model.env.dtype
        self.max_model_len = max_model_len
        if max_model_len > model.env.max_positions:
            raise ValueError("max_model_len exceeds the positions the model was built for")
        kv_groups, state_groups = group_cache_layers(model.cache_needs(), page_tokens)
        dtype_bytes = torch.empty(0, dtype=self.dtype).element_size()
        if num_pages is None:
            if cache_memory_bytes is None:
                raise ValueError("give num_pages or cache_memory_bytes")
            pages = pages_for_memory(kv_groups, cache_memory_bytes, dtype_bytes, max_model_len,
                                     max_num_batched_tokens)
        elif isinstance(num_pages, int):
            pages = [num_pages] * len(kv_groups)
        else:
            pages = list(num_pages)
        self.manager = CacheManager(kv_groups, pages, max_num_seqs)
        self.pools = CachePools(kv_groups, state_groups, pages, max_num_seqs, self.dtype, self.device)
        self.planners = model.step_planners()
        for mixer, _ in self.planners.values():
            mixer.reserve(max_num_seqs)
        self.decode_graphs = None
        self.last_h2d_bytes = 0
        self.last_d2h_bytes = 0
        self._staging: list[tuple[torch.Tensor, Any]] = []
        self._staging_turn = 0
        self.steps_run = 0

    # ------------------------------------------------------------------ upload
    def _stage(self, n: int) -> tuple[torch.Tensor, int]:
        """A pinned int32 buffer of at least ``n`` elements that no copy in flight still reads."""
        if len(self._staging) < 2:
            self._staging.append((torch.empty(max(n, 4096), dtype=torch.int32).pin_memory(), None))
        self._staging_turn = (self._staging_turn + 1) % len(self._staging)
        i = self._staging_turn
        buf, ev = self._staging[i]
        if ev is not None:
            ev.synchronize()
        if buf.numel() < n:
            buf = torch.empty(2 * n, dtype=torch.int32).pin_memory()
            self._staging[i] = (buf, None)
        return buf, i

    def upload(self, host: HostStep, decode_splits: int = 0) -> DeviceStep:
        plans_host = {
            key: mixer.plan_step(host, self.pools.view(cid, False).group)
            for key, (mixer, cid) in self.planners.items()
        }
        arrays: list[tuple[Any, np.ndarray]] = [
            ("token_ids", host.token_ids), ("positions", host.positions),
            ("token_seq", host.token_seq), ("cu_q", host.cu_q), ("ctx_lens", host.ctx_lens),
            ("state_slots", host.state_slots), ("first_portion", host.first_portion),
            ("logit_rows", host.logit_rows),
        ]
        arrays += [(("table", g), t) for g, t in enumerate(host.block_tables)]
        for key, plan in plans_host.items():
            arrays += [(("plan", key, name), a) for name, a in plan.items()]
        offsets, total = [], 0
        for _, a in arrays:
            offsets.append(total)
            total += (a.size + 3) // 4 * 4
        total = max(total, 4)
        if self.device.type == "cuda":
            stage, idx = self._stage(total)
            flat = stage.numpy()
        else:
            flat = np.zeros(total, dtype=np.int32)
        for (_, a), off in zip(arrays, offsets):
            flat[off : off + a.size] = a.reshape(-1)
        if self.device.type == "cuda":
            dev = torch.empty(total, dtype=torch.int32, device=self.device)
            dev.copy_(stage[:total], non_blocking=True)
            self.last_h2d_bytes = 4 * total
            ev = torch.cuda.Event()
            ev.record()
            self._staging[idx] = (stage, ev)
        else:
            dev = torch.from_numpy(flat)
        # one split instead of a slice per array; only arrays of rank 2 need a view on top
        sizes = [offsets[i + 1] - offsets[i] for i in range(len(offsets) - 1)] + [total - offsets[-1]]
        got: dict[Any, torch.Tensor] = {}
        for (name, a), piece in zip(arrays, dev.split(sizes)):
            t = piece if piece.shape[0] == a.size else piece[: a.size]
            got[name] = t if a.ndim == 1 else t.view(a.shape)
        plans = {
            key: {name: got[("plan", key, name)] for name in plan} for key, plan in plans_host.items()
        }
        dec = host.q_lens == 1
        return DeviceStep(
            token_ids=got["token_ids"], positions=got["positions"], token_seq=got["token_seq"],
            cu_q=got["cu_q"], ctx_lens=got["ctx_lens"], state_slots=got["state_slots"],
            first_portion=got["first_portion"],
            block_tables=[got[("table", g)] for g in range(len(host.block_tables))],
            logit_rows=got["logit_rows"], num_tokens=host.num_tokens, num_seqs=host.num_seqs,
            num_logit_rows=int(host.logit_rows.shape[0]),
            max_decode_ctx=int(host.ctx_lens[dec].max()) if dec.any() else 0,
            decode_splits=decode_splits, plans=plans, host=host,
            every_row_wanted=bool(host.logit_rows.shape[0] == host.num_tokens
                                  and np.array_equal(host.logit_rows, np.arange(host.num_tokens))),
        )

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens as one batch; float32 logits ``[wanted places, vocab]``."""
        host = build_host_step(entries, self.manager, self.model.plan.vocab_size, self.max_model_len)
        dev = self.upload(host)
        logits = self.model.forward(dev, self.pools)
        self.steps_run += 1
        return logits

    def run(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Admit new requests, allocate pages, step, commit: a step for callers with no scheduler."""
        for e in entries:
            if not self.manager.is_live(e.rid):
                self.manager.admit(e.rid)
        for e in entries:
            self.manager.allocate(e.rid, len(e.tokens))
        logits = self.step(entries)
        for e in entries:
            self.manager.commit(e.rid, len(e.tokens))
        return logits

    def finish(self, rid) -> None:
        """Give back everything ``rid`` holds."""
        self.manager.release(rid)

    def _graphs(self):
        from .decode_graph import DecodeGraphs

        if self.decode_graphs is None:
            self.decode_graphs = DecodeGraphs(self)
        return self.decode_graphs

    def can_launch_decode(self, entries: Sequence[StepEntry], rows) -> bool:
        """Does this step run as a captured CUDA graph (see :meth:`DecodeGraphs.accepts`)?"""
        return self.device.type == "cuda" and self._graphs().accepts(entries, rows)

    def launch_decode(self, entries: Sequence[StepEntry], rows, ahead_of=None, sampler=None):
        """Enqueue a step as a CUDA graph (see :meth:`DecodeGraphs.launch`);
        :meth:`collect_decode` waits and returns the sampler's output. Rows with penalties, banned
        tokens or log-probabilities need ``sampler`` and are sampled before this returns."""
        pending = self._graphs().launch(entries, rows, ahead_of, sampler)
        self.last_h2d_bytes = 4 * pending.graph.words
        self.last_d2h_bytes = 4 * len(rows)
        return pending

    def collect_decode(self, pending):
        return self.decode_graphs.collect_checked(pending)

    def step_and_sample(self, entries: Sequence[StepEntry], sampler, rows, graphs: bool = False):
        """A step followed by sampling on the device; only token ids come back to the host.

        ``rows`` has one :class:`~llmserve_b200.sampling.SampleRow` per wanted place, in order.
        """
        if graphs and self.can_launch_decode(entries, rows):
            return self.collect_decode(self.launch_decode(entries, rows, sampler=sampler))
        logits = self.step(entries)
        out = sampler.sample(logits, rows)  # reads the tokens: the step has finished
        self.last_d2h_bytes = 4 * len(rows)
        self.check_kernels()
        return out

    def check_kernels(self) -> None:
        """Raise if a kernel recorded that it gave up a bounded wait. Call after a synchronisation."""
        check = getattr(self.ops, "check_kernel_errors", None)
        if check is not None:
            check()
