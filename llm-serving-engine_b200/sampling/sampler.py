"""Batched sampling on the device: one token per row of logits.

Order of operations as in src/llmserve/sampling.py:151-204: raw log-probabilities (if asked for)
-> penalties -> banned tokens -> greedy argmax, or temperature, top-k / top-p / min-p and an
exponential-race draw. Only token ids (and the few log-probabilities asked for) cross to the host.

Randomness: the reference gives each seeded request its own CPU generator
(src/llmserve/sequence.py:57-59); here each request has a 64-bit seed and the kernel's counter
generator is keyed by (seed, index of the token being generated), which also makes a request's
samples independent of what else is in the batch and of preemption.
"""

from __future__ import annotations

from collections import Counter
from dataclasses import dataclass, field

import torch

from .params import SamplingParams


@dataclass
class SampleRow:
    """What the sampler needs to know about one row of the logits batch."""

    params: SamplingParams
    output_token_ids: list[int]
    prompt_token_ids: list[int]
    seed: int  # the request's 64-bit seed
    banned_token_ids: list[int] = field(default_factory=list)  # e.g. EOS before min_tokens
    draw: int | None = None  # index of the token being generated, if not len(output_token_ids)

    @property
    def draw_index(self) -> int:
        return len(self.output_token_ids) if self.draw is None else self.draw


@dataclass
class SamplerOutput:
    token_ids: list[int]
    logprobs: list[float] | None
    top_logprobs: list[list[tuple[int, float]]] | None


class Sampler:
    def __init__(self, ops, device) -> None:
        self.ops = ops
        self.device = torch.device(device)
        self._greedy_params: dict[int, tuple] = {}

    def _greedy(self, n: int):
        """Constant parameter tensors for a batch of ``n`` greedy rows (made once per size)."""
        if n not in self._greedy_params:
            z = lambda dt, v=0: torch.full((n,), v, dtype=dt, device=self.device)
            self._greedy_params[n] = (z(torch.float32), z(torch.int32, -1), z(torch.float32, 1.0),
                                      z(torch.float32), z(torch.int64), z(torch.int32))
        return self._greedy_params[n]

    def _dev(self, values, dtype):
        t = torch.tensor(values, dtype=dtype)
        if self.device.type == "cuda":
            return t.pin_memory().to(self.device, non_blocking=True)
        return t

    def sample(self, logits: torch.Tensor, rows: list[SampleRow]) -> SamplerOutput:
        """logits: float32 ``[len(rows), vocab]`` on the device (modified in place)."""
        if logits.shape[0] != len(rows):
            raise ValueError("one SampleRow per row of logits is needed")
        if not rows:
            return SamplerOutput([], None, None)
        want_lp = any(r.params.logprobs is not None for r in rows)
        if not want_lp and all(
            r.params.greedy and not r.params.has_penalties and not r.banned_token_ids for r in rows
        ):
            return SamplerOutput(self.ops.sample(logits, *self._greedy(len(rows))).tolist(), None, None)
        raw = logits.clone() if want_lp else None

        pen = [(i, r) for i, r in enumerate(rows) if r.params.has_penalties]
        if pen:
            row, tok, cnt, pres, freq, rep = [], [], [], [], [], []
            for i, r in pen:
                counts = Counter(r.output_token_ids)
                seen = set(r.prompt_token_ids) | set(counts)
                for t in seen:
                    row.append(i)
                    tok.append(t)
                    cnt.append(counts.get(t, 0))
                    pres.append(r.params.presence_penalty)
                    freq.append(r.params.frequency_penalty)
                    rep.append(r.params.repetition_penalty)
            if row:
                self.ops.apply_penalties(
                    logits, self._dev(row, torch.int32), self._dev(tok, torch.int32),
                    self._dev(cnt, torch.int32), self._dev(pres, torch.float32),
                    self._dev(freq, torch.float32), self._dev(rep, torch.float32))
        ban = [(i, t) for i, r in enumerate(rows) for t in r.banned_token_ids]
        if ban:
            self.ops.ban_tokens(logits, self._dev([b[0] for b in ban], torch.int32),
                                self._dev([b[1] for b in ban], torch.int32))
        p = [r.params for r in rows]
        tokens = self.ops.sample(
            logits,
            self._dev([q.temperature for q in p], torch.float32),
            self._dev([q.top_k for q in p], torch.int32),
            self._dev([q.top_p for q in p], torch.float32),
            self._dev([q.min_p for q in p], torch.float32),
            self._dev([_as_int64(r.seed) for r in rows], torch.int64),
            self._dev([r.draw_index for r in rows], torch.int32),
        )
        if not want_lp:
            return SamplerOutput(tokens.tolist(), None, None)
        lse = self.ops.logsumexp(raw)
        idx = tokens.long()
        chosen = (raw.gather(1, idx[:, None])[:, 0] - lse).tolist()
        token_list = idx.tolist()
        tops: list[list[tuple[int, float]]] = []
        for i, r in enumerate(rows):
            k = r.params.logprobs or 0
            if k > 0:
                v, ix = (raw[i] - lse[i]).topk(k)
                tops.append(list(zip(ix.tolist(), v.tolist(), strict=True)))
            else:
                tops.append([])
        return SamplerOutput(token_list, chosen, tops)


def _as_int64(seed: int) -> int:
    seed &= 0xFFFFFFFFFFFFFFFF
    return seed - (1 << 64) if seed >= (1 << 63) else seed
