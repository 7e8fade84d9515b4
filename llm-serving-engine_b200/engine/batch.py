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
    every_row_wanted: bool = False  # logit_rows is 0, 1, ..., num_tokens - 1: the final norm need not gather


def build_host_step(entries: Sequence[StepEntry], manager, vocab_size: int, max_positions: int) -> HostStep:
    """Flatten ``entries`` and check everything a kernel would otherwise trust blindly."""
    if not entries:
        raise ValueError("a step needs at least one entry")
    n = len(entries)
    held = []
    for e in entries:
        h = manager.held.get(e.rid)
        if h is None:
            raise KeyError(f"request {e.rid!r} is not live")
        held.append(h)
    if len({e.rid for e in entries}) != n:
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
    lens = [len(e.tokens) for e in entries]
    if min(lens) < 1:
        rid = entries[lens.index(min(lens))].rid
        raise ValueError(f"request {rid!r}: an entry needs at least one token")
    q_lens = np.asarray(lens, dtype=np.int32)
    starts = np.asarray([h.computed for h in held], dtype=np.int32)
    slots = np.asarray([h.slot for h in held], dtype=np.int32)
    cu_q = np.zeros(n + 1, dtype=np.int32)
    np.cumsum(q_lens, out=cu_q[1:])
    total = int(cu_q[-1])
    ctx_lens = starts + q_lens
    if int(ctx_lens.max()) > max_positions:
        raise ValueError(
            f"a sequence would reach {int(ctx_lens.max())} tokens; the engine was built for {max_positions}"
        )
    if total == n:  # single tokens only
        tokens64 = np.asarray([e.tokens[0] for e in entries], dtype=np.int64)
    else:
        tokens64 = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
    if tokens64.min() < 0 or tokens64.max() >= vocab_size:
        raise ValueError(f"token ids must lie in [0, {vocab_size})")
    token_seq = np.repeat(np.arange(n, dtype=np.int32), q_lens)
    # a token's position: its row, minus its sequence's first row, plus the sequence's start
    positions = np.arange(total, dtype=np.int32) + np.repeat(starts - cu_q[:-1], q_lens)
    rows: list[int] = []
    for i, e in enumerate(entries):
        for w in e.want:
            if not 0 <= w < lens[i]:
                raise ValueError(f"request {e.rid!r}: wanted place {w} is outside its {lens[i]} tokens")
            rows.append(int(cu_q[i]) + int(w))
    tables = []
    for g, spec in enumerate(manager.groups):
        need = (-(-ctx_lens.astype(np.int64) // spec.page_tokens)).tolist()
        t = np.zeros((n, max(1, max(need))), dtype=np.int32)
        for i, h in enumerate(held):
            k = need[i]
            if len(h.tables[g]) < k:
                raise ValueError(
                    f"request {entries[i].rid!r}: block table of group {g} has {len(h.tables[g])} pages, "
                    f"needs {k}"
                )
            t[i, :k] = h.arrays[g][:k]
        if spec.window > 0:
            # pages that the window has passed are given back (-1) and never read: the kernels start
            # at the page of key ``start - window + 1``; all later entries must be pages held
            first_page = np.maximum(0, starts - spec.window + 1) // spec.page_tokens
            live = np.arange(t.shape[1])[None, :] >= first_page[:, None]
            bad = ((t < 0) & live).any(axis=1)
            np.maximum(t, 0, out=t)
        else:
            bad = (t < 0).any(axis=1)
        bad |= (t >= manager.num_pages(g)).any(axis=1)
        if bad.any():
            rid = entries[int(np.argmax(bad))].rid
            raise ValueError(f"request {rid!r}: block table of group {g} names a page it does not hold")
        tables.append(t)
    return HostStep(
        token_ids=tokens64.astype(np.int32),
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
