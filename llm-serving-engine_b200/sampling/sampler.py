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
    # where the request's token state for the penalties lives on the device: its state slot and
    # the slot's epoch (it changes when the slot is given to another request); -1: no slot, the
    # penalised tokens are listed on the host each time
    slot: int = -1
    epoch: int = 0

    @property
    def draw_index(self) -> int:
        return len(self.output_token_ids) if self.draw is None else self.draw


@dataclass
class SamplerOutput:
    token_ids: list[int]
    logprobs: list[float] | None
    top_logprobs: list[list[tuple[int, float]]] | None


class Sampler:
    """``max_slots`` > 0: requests carry a state slot, and the tokens that the penalties look at
    (prompt tokens, and how often each token was generated) are kept per slot on the device,
    ``[max_slots, vocab]`` int32, allocated when penalties are first used. Each step only the
    tokens generated since the last one are entered; the penalties then read that state."""

    def __init__(self, ops, device, max_slots: int = 0) -> None:
        self.ops = ops
        self.device = torch.device(device)
        self.max_slots = max_slots
        self._greedy_params: dict[int, tuple] = {}
        self._token_state: torch.Tensor | None = None
        self._entered: dict[int, tuple[int, int]] = {}  # slot -> (epoch, output tokens entered)

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
            return SamplerOutput(
                self.ops.sample(logits, *self._greedy(len(rows)), kinds=1).tolist(), None, None)
        pen = [(i, r) for i, r in enumerate(rows) if r.params.has_penalties]
        ban = [(i, t) for i, r in enumerate(rows) for t in r.banned_token_ids]
        # log-probabilities are those of the model, before penalties and bans change the logits
        raw = (logits.clone() if (pen or ban) else logits) if want_lp else None
        if pen and self.max_slots > 0 and all(0 <= r.slot < self.max_slots for _, r in pen):
            self._penalties_from_state(logits, pen)
        elif pen:
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
            kinds=sample_kinds(p),
        )
        if not want_lp:
            return SamplerOutput(tokens.tolist(), None, None)
        # everything asked for goes to the host in one transfer
        lse = self.ops.logsumexp(raw)
        idx = tokens.long()
        chosen = raw.gather(1, idx[:, None])[:, 0] - lse
        kmax = max((r.params.logprobs or 0) for r in rows)
        parts = [idx.to(torch.float64), chosen.to(torch.float64)]
        if kmax > 0:
            v, ix = raw.topk(kmax, dim=1)
            parts += [(v - lse[:, None]).to(torch.float64).flatten(), ix.to(torch.float64).flatten()]
        flat = torch.cat(parts).tolist()  # float64 holds token ids and float32 values exactly
        n = len(rows)
        token_list = [int(t) for t in flat[:n]]
        chosen_list = flat[n : 2 * n]
        tops: list[list[tuple[int, float]]] = []
        for i, r in enumerate(rows):
            k = r.params.logprobs or 0
            if k > 0:
                vals = flat[2 * n + i * kmax : 2 * n + i * kmax + k]
                ids = flat[2 * n + n * kmax + i * kmax : 2 * n + n * kmax + i * kmax + k]
                tops.append([(int(t), x) for t, x in zip(ids, vals, strict=True)])
            else:
                tops.append([])
        return SamplerOutput(token_list, chosen_list, tops)

    def _penalties_from_state(self, logits: torch.Tensor, pen) -> None:
        """Enter what each penalised request generated since its last step into the token state
        on the device, then apply the penalties from that state."""
        V = logits.shape[1]
        if self._token_state is None or self._token_state.shape[1] != V:
            self._token_state = torch.zeros(self.max_slots, V, dtype=torch.int32, device=self.device)
            self._entered.clear()
        slot, tok, flag = [], [], []
        for _, r in pen:
            epoch, done = self._entered.get(r.slot, (None, 0))
            if epoch != r.epoch or done > len(r.output_token_ids):
                # the slot belongs to this request now: start from its prompt
                self._token_state[r.slot].zero_()
                unique = set(r.prompt_token_ids)
                slot += [r.slot] * len(unique)
                tok += unique
                flag += [1] * len(unique)
                done = 0
            new = r.output_token_ids[done:]
            slot += [r.slot] * len(new)
            tok += new
            flag += [0] * len(new)
            self._entered[r.slot] = (r.epoch, len(r.output_token_ids))
        if slot:
            self.ops.token_state_add(self._token_state, self._dev(slot, torch.int32),
                                     self._dev(tok, torch.int32), self._dev(flag, torch.int32))
        self.ops.apply_penalties_dense(
            logits,
            self._dev([i for i, _ in pen], torch.int32),
            self._dev([r.slot for _, r in pen], torch.int32),
            self._dev([r.params.presence_penalty for _, r in pen], torch.float32),
            self._dev([r.params.frequency_penalty for _, r in pen], torch.float32),
            self._dev([r.params.repetition_penalty for _, r in pen], torch.float32),
            self._token_state)


def sample_kinds(params) -> int:
    """Which of the two sampling kernels a batch needs (see ``CudaOps.sample``)."""
    kinds = 0
    for q in params:
        kinds |= 1 if (q.greedy or q.has_cut) else 2
    return kinds


def _as_int64(seed: int) -> int:
    seed &= 0xFFFFFFFFFFFFFFFF
    return seed - (1 << 64) if seed >= (1 << 63) else seed
