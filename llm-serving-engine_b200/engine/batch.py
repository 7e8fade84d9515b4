"""One step's ragged batch, on the host and on the device.

A step is a list of entries ``(request, its next tokens, the places among them whose logits are
wanted)``. Portions of prompts and single decoded tokens sit side by side in one flat token batch,
as in the reference's runner (src/llmserve/model_runner.py:50-69): ``token_ids[T]``,
``positions[T]``, and per sequence its row range, context length and block tables.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    rid: Any  # request id known to the cache manager
    tokens: Sequence[int]  # the request's next tokens (at least one)
    want: Sequence[int] = ()  # places among ``tokens`` whose logits are returned


@dataclass
class HostStep:
    """The batch as numpy int32 arrays (what is uploaded) plus a few host-side scalars."""

    token_ids: np.ndarray  # [T]
    positions: np.ndarray  # [T] absolute position of each token in its request
    token_seq: np.ndarray  # [T] index of the token's sequence in this batch
    cu_q: np.ndarray  # [N+1] row offsets of the sequences
    q_lens: np.ndarray  # [N]
    ctx_lens: np.ndarray  # [N] tokens of the sequence in the cache once this step has written
    state_slots: np.ndarray  # [N]
    first_portion: np.ndarray  # [N] 1 where the sequence starts at position 0 in this step
    block_tables: list[np.ndarray]  # per key/value group: [N, max_blocks]
    logit_rows: np.ndarray  # [R] flat row indices whose logits are wanted
    rids: list[Any] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return int(self.token_ids.shape[0])

    @property
    def num_seqs(self) -> int:
        return int(self.q_lens.shape[0])


@dataclass
class DeviceStep:
    """What the model's parts read during a forward pass (all int32 tensors on the device)."""

    token_ids: torch.Tensor
    positions: torch.Tensor
    token_seq: torch.Tensor
    cu_q: torch.Tensor
    ctx_lens: torch.Tensor
    state_slots: torch.Tensor
    first_portion: torch.Tensor
    block_tables: list[torch.Tensor]
    logit_rows: torch.Tensor
    num_tokens: int
    num_seqs: int
    num_logit_rows: int
    max_decode_ctx: int  # longest context among the single-token sequences (0 if none)
    decode_splits: int  # fixed number of context partitions, or 0 to let the kernels choose
    plans: dict[Any, dict[str, Any]]
    host: HostStep | None = None


def build_host_step(entries: Sequence[StepEntry], manager, vocab_size: int, max_positions: int) -> HostStep:
    """Flatten ``entries`` and check everything a kernel would otherwise trust blindly."""
    if not entries:
        raise ValueError("a step needs at least one entry")
    n = len(entries)
    q_lens = np.empty(n, dtype=np.int32)
    starts = np.empty(n, dtype=np.int32)
    slots = np.empty(n, dtype=np.int32)
    seen = set()
    for i, e in enumerate(entries):
        if e.rid in seen:
            raise ValueError(f"request {e.rid!r} appears twice in one step")
        seen.add(e.rid)
        if len(e.tokens) < 1:
            raise ValueError(f"request {e.rid!r}: an entry needs at least one token")
        q_lens[i] = len(e.tokens)
        starts[i] = manager.num_computed(e.rid)
        slots[i] = manager.state_slot(e.rid)
    cu_q = np.zeros(n + 1, dtype=np.int32)
    np.cumsum(q_lens, out=cu_q[1:])
    total = int(cu_q[-1])
    ctx_lens = starts + q_lens
    if int(ctx_lens.max()) > max_positions:
        raise ValueError(
            f"a sequence would reach {int(ctx_lens.max())} tokens; the engine was built for {max_positions}"
        )
    token_ids = np.empty(total, dtype=np.int32)
    positions = np.empty(total, dtype=np.int32)
    token_seq = np.empty(total, dtype=np.int32)
    rows: list[int] = []
    for i, e in enumerate(entries):
        a, b = int(cu_q[i]), int(cu_q[i + 1])
        token_ids[a:b] = e.tokens if isinstance(e.tokens, np.ndarray) else np.asarray(e.tokens, dtype=np.int64)
        positions[a:b] = np.arange(starts[i], starts[i] + q_lens[i], dtype=np.int32)
        token_seq[a:b] = i
        for w in e.want:
            if not 0 <= w < q_lens[i]:
                raise ValueError(f"request {e.rid!r}: wanted place {w} is outside its {q_lens[i]} tokens")
            rows.append(a + int(w))
    if token_ids.min() < 0 or token_ids.max() >= vocab_size:
        raise ValueError(f"token ids must lie in [0, {vocab_size})")
    tables = []
    for g, spec in enumerate(manager.groups):
        need = -(-ctx_lens.astype(np.int64) // spec.page_tokens)
        width = max(1, int(need.max()))
        t = np.zeros((n, width), dtype=np.int32)
        first_key = np.maximum(0, starts - spec.window + 1) if spec.window > 0 else np.zeros(n, np.int32)
        for i, e in enumerate(entries):
            tab = manager.block_table(e.rid, g)
            if len(tab) < need[i]:
                raise ValueError(
                    f"request {e.rid!r}: block table of group {g} has {len(tab)} pages, needs {int(need[i])}"
                )
            row = np.asarray(tab[: int(need[i])], dtype=np.int32)
            lo = int(first_key[i]) // spec.page_tokens
            if (row[lo:] < 0).any() or (row[lo:] >= manager.num_pages(g)).any():
                raise ValueError(f"request {e.rid!r}: block table of group {g} names a page it does not hold")
            t[i, : row.shape[0]] = np.maximum(row, 0)
        tables.append(t)
    return HostStep(
        token_ids=token_ids,
        positions=positions,
        token_seq=token_seq,
        cu_q=cu_q,
        q_lens=q_lens,
        ctx_lens=ctx_lens.astype(np.int32),
        state_slots=slots,
        first_portion=(starts == 0).astype(np.int32),
        block_tables=tables,
        logit_rows=np.asarray(rows, dtype=np.int32),
        rids=[e.rid for e in entries],
    )
