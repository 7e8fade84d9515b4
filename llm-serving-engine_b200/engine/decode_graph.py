"""CUDA graphs for the steps that are bound by launching kernels, not by running them.

A decode step at small batch is a few hundred short kernels; launching them one by one costs more
than running them. Such a step (every entry one token, every entry sampled) is therefore captured
once per (batch size, number of context partitions) as a CUDA graph over fixed device buffers and
replayed: per step the host fills one pinned buffer (token ids, positions, context lengths, block
tables, sampling parameters), copies it to the device in one transfer, replays the graph (model
forward and sampling kernel) and reads the sampled token ids back.

A graph has a fixed batch size. So that a batch that shrinks or grows by one does not need a new
capture each time, batches are padded to the next of a few sizes (1, 2, 3, 4, 6, 8, 12, 16, ...):
a padding row is a one-token sequence at position 0 whose block table names the cache's spare
page and whose state slot is the spare slot, so it reads and writes nothing that a request owns,
costs next to nothing in the attention, and its sample is dropped.

Rows that need more than the sampling kernel (penalties, banned tokens, log-probabilities) use a
second capture of the same step that ends with the logits; the sampler then runs on them
uncaptured. The model forward is replayed either way.

Steps that hold portions of prompts beside single tokens (what a loaded server runs all the time)
are captured too while they are small enough to be bound by the host (:class:`_MixedGraph`): the
single-token rows come first, padded as above, then a fixed number of portion slots with a fixed
number of tokens together. Real portions fill the first slots; the other slots and the remaining
tokens are padding sequences on the spare page and slot. A shape is captured the second time it
is asked for; until then, and for shapes that do not fit, the step runs uncaptured.

The graph runs the same model code, kernels and cache as an uncaptured step; only the launch
mechanism differs.
"""

from __future__ import annotations

import gc
from typing import Sequence

import numpy as np
import torch

from ..sampling.sampler import sample_kinds
from .batch import DeviceStep, HostStep, StepEntry, build_host_step


class _Graph:
    def __init__(self, owner: "DecodeGraphs", batch: int, splits: int, sampled: bool = True,
                 kinds: int = 3) -> None:
        runner = owner.runner
        self.batch = B = batch
        self.slots = 0  # no portions of prompts
        self.sampled = sampled  # the capture ends with the sampling kernel (else with the logits)
        self.kinds = kinds  # which sampling kernels the capture holds (see CudaOps.sample)
        dev = runner.device
        widths = [-(-runner.max_model_len // g.page_tokens) for g in runner.manager.groups]
        # layout of the per-step buffer, in int32 words
        names = ["token_ids", "positions", "ctx_lens", "state_slots", "first_portion",
                 "temperature", "top_k", "top_p", "min_p", "draw"]
        self.off, n = {}, 0
        for name in names:
            self.off[name] = n
            n += (B + 3) // 4 * 4
        self.off["seed"] = n  # int64: two words each, at an even offset
        n += 2 * ((B + 1) // 2 * 2)
        self.table_off = []
        for w in widths:
            self.table_off.append((n, w))
            n += B * w
        self.words = n
        self.host = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.h = self.host.numpy()
        self.dev = torch.zeros(n, dtype=torch.int32, device=dev)
        ar = torch.arange(B + 1, dtype=torch.int32, device=dev)
        view = lambda name: self.dev[self.off[name] : self.off[name] + B]
        plans = {
            key: {"tiles": torch.zeros(0, 2, dtype=torch.int32, device=dev), "decode_seqs": ar[:B]}
            for key in runner.planners
        }
        self.step = DeviceStep(
            token_ids=view("token_ids"), positions=view("positions"), token_seq=ar[:B], cu_q=ar,
            ctx_lens=view("ctx_lens"), state_slots=view("state_slots"),
            first_portion=view("first_portion"),
            block_tables=[self.dev[o : o + B * w].view(B, w) for o, w in self.table_off],
            logit_rows=ar[:B], num_tokens=B, num_seqs=B, num_logit_rows=B, max_decode_ctx=0,
            decode_splits=splits, plans=plans, host=None, every_row_wanted=True,
        )
        f32 = lambda name: view(name).view(torch.float32)
        so = self.off["seed"]
        self.sample_args = (f32("temperature"), view("top_k"), f32("top_p"), f32("min_p"),
                            self.dev[so : so + 2 * B].view(torch.int64), view("draw"))
        self.tokens_host = [torch.zeros(B, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.turn = 0
        self.h2d_done: torch.cuda.Event | None = None  # the pinned input buffer may be rewritten after it
        self.graph: torch.cuda.CUDAGraph | None = None
        self.tokens: torch.Tensor | None = None
        self.logits: torch.Tensor | None = None
        self.launches = 0

    def hview(self, name, dtype=np.int32):
        B = self.batch
        return self.h[self.off[name] : self.off[name] + B].view(dtype)


def token_bucket(n: int) -> int:
    """Token counts of captured portions: multiples of 64, coarser above 1024 tokens (a sixteenth
    of the next power of two), so that padding stays a few percent of the step."""
    step = 64
    while step * 16 < n:
        step *= 2
    return -(-n // step) * step


def slot_bucket(n: int) -> int:
    """Portion slots of a captured step: 8, 16, 32, ... (an unused slot costs two padding tokens)."""
    return max(8, pow2_at_least(n))


def row_bucket(n: int, limit: int) -> int:
    """One-token rows of a captured step with portions: 0, 4, 16, 64, ... up to ``limit``. Coarser
    than the decode graphs' sizes: a padding row costs little beside the portions, a shape that is
    met only once or twice costs a capture that is never paid back."""
    if n == 0:
        return 0
    b = 4
    while b < n:
        b *= 4
    return min(b, limit)


def pow2_at_least(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


class _MixedGraph:
    """Fixed buffers of a step of ``batch`` one-token rows, then ``slots`` portions of prompts with
    ``tokens`` tokens together. ``plans`` are the work lists of one such step, at their full size:
    they give the lists' names and shapes."""

    def __init__(self, owner: "DecodeGraphs", batch: int, slots: int, tokens: int, splits: int,
                 sampled: bool, kinds: int, plans: dict) -> None:
        runner = owner.runner
        dev = runner.device
        self.batch, self.slots, self.pre_tokens = batch, slots, tokens
        self.N = N = batch + slots
        self.T = T = batch + tokens
        self.sampled, self.kinds = sampled, kinds
        sizes = {"token_ids": T, "positions": T, "token_seq": T, "cu_q": N + 1, "ctx_lens": N,
                 "state_slots": N, "first_portion": N, "logit_rows": N, "temperature": N,
                 "top_k": N, "top_p": N, "min_p": N, "draw": N, "seed": 2 * N}
        for gi, g in enumerate(runner.manager.groups):
            sizes[("table", gi)] = N * -(-runner.max_model_len // g.page_tokens)
        for key, plan in plans.items():
            for name, a in plan.items():
                sizes[("plan", key, name)] = a.size
        self.off, self.size, n = {}, sizes, 0
        for name, k in sizes.items():  # every array starts on a 16-byte boundary
            self.off[name] = n
            n += (k + 3) // 4 * 4
        self.words = max(n, 4)
        self.host = torch.zeros(self.words, dtype=torch.int32).pin_memory()
        self.h = self.host.numpy()
        self.dev = torch.zeros(self.words, dtype=torch.int32, device=dev)
        view = lambda name: self.dev[self.off[name] : self.off[name] + sizes[name]]
        self.step = DeviceStep(
            token_ids=view("token_ids"), positions=view("positions"), token_seq=view("token_seq"),
            cu_q=view("cu_q"), ctx_lens=view("ctx_lens"), state_slots=view("state_slots"),
            first_portion=view("first_portion"),
            block_tables=[view(("table", gi)).view(N, -1) for gi in range(len(runner.manager.groups))],
            logit_rows=view("logit_rows"), num_tokens=T, num_seqs=N, num_logit_rows=N,
            max_decode_ctx=0, decode_splits=splits,
            plans={key: {name: view(("plan", key, name)).view(a.shape) for name, a in plan.items()}
                   for key, plan in plans.items()},
            host=None,
        )
        f32 = lambda name: view(name).view(torch.float32)
        self.sample_args = (f32("temperature"), view("top_k"), f32("top_p"), f32("min_p"),
                            view("seed").view(torch.int64), view("draw"))
        self.tokens_host = [torch.zeros(N, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.turn = 0
        self.h2d_done: torch.cuda.Event | None = None
        self.graph: torch.cuda.CUDAGraph | None = None
        self.tokens: torch.Tensor | None = None
        self.logits: torch.Tensor | None = None
        self.launches = 0

    def hview(self, name, dtype=np.int32):
        return self.h[self.off[name] : self.off[name] + self.size[name]].view(dtype)


def batch_sizes(limit: int) -> list[int]:
    """1, 2, 3, 4, 6, 8, 12, 16, ... up to ``limit`` (which is always one of them)."""
    out, b = [], 1
    while b < limit:
        out.append(b)
        if b >= 2 and b + b // 2 < limit:
            out.append(b + b // 2)
        b *= 2
    return out + [limit]


class DecodeGraphs:
    def __init__(self, runner) -> None:
        self.runner = runner
        self.graphs: dict[tuple, _Graph | _MixedGraph] = {}
        self.pool = None
        self.side: torch.cuda.Stream | None = None  # the stream that captures are recorded on
        groups = runner.manager.groups
        self.min_kv_heads = min((g.num_kv_heads for g in groups), default=1)
        slots = runner.manager.max_requests
        self.sizes = batch_sizes(slots)
        # host mirror of every live request's block tables, by state slot, grown page by page;
        # the row after the last slot is the padding rows' table: the spare page
        self.mirror = [
            np.zeros((slots + 1, -(-runner.max_model_len // g.page_tokens)), np.int32)
            for g in groups
        ]
        for gi in range(len(groups)):
            self.mirror[gi][slots, :] = runner.pools.spare_page(gi)
        self.mirror_len = np.zeros((len(groups), slots), dtype=np.int64)
        self.mirror_epoch = np.zeros(slots, dtype=np.int64)
        # Steps with portions of prompts are captured while launching them kernel by kernel takes
        # longer than running them. Measured on SmolLM2 sizes: launching costs about 130 us per
        # layer that runs; the device needs about 45 us per layer for its eleven kernels, however
        # few the tokens, plus 2 x weights x tokens / 0.8e15 s. The two meet at
        # tokens = 4.5e10 / (weights per layer); beyond that the step is bound by the device and
        # padding would only make it longer. Attention over long contexts is not in this estimate,
        # so the count is capped where padding (a sixteenth at most) could cost more than the
        # launches that are saved.
        model = runner.model
        matrix = sum(int(np.prod(d.shape)) for d in model.param_decls().values()
                     if d.role == "matrix" and len(d.shape) == 2 and d.shape[0] != model.plan.vocab_size)
        estimate = int(len(model.plan.run_order) * 4.5e10 / max(matrix, 1))
        self.max_mixed_tokens = max(128, min(estimate, 1024))
        self.capture_after = 2  # a shape is captured the second time it is asked for
        self.asked: dict[tuple, int] = {}
        self.mixed_plannable = all(hasattr(m, "plan_rows") for m, _ in runner.planners.values())
        # a part that works from the host while a step runs rules out captures altogether
        self.capturable = not any(getattr(p, "needs_host_step", False) for p in model.parts())

    def padded(self, n: int) -> int:
        """The captured batch size that serves ``n`` rows."""
        for b in self.sizes:
            if b >= n:
                return b
        return n

    @staticmethod
    def forward_usable(entries: Sequence[StepEntry], rows) -> bool:
        """Every entry is one token whose logits are sampled."""
        if len(rows) != len(entries):
            return False
        for e in entries:
            if len(e.tokens) != 1 or list(e.want) != [0]:
                return False
        return True

    def mixed_shape(self, entries: Sequence[StepEntry]):
        """(one-token rows, portion slots, portion tokens) of the capture that serves ``entries``, or
        None if they should run uncaptured. One slot more than the portions and two tokens for
        every unused slot are kept for the padding sequences."""
        single = portions = tokens = 0
        for e in entries:
            n = len(e.tokens)
            if n == 1:
                single += 1
            else:
                portions += 1
                tokens += n
            if len(e.want) > 1 or (len(e.want) == 1 and e.want[0] != n - 1):
                return None
        if not self.mixed_plannable or portions == 0 or single > self.sizes[-1]:
            return None
        B = row_bucket(single, self.sizes[-1])
        P = slot_bucket(portions + 1)
        TP = token_bucket(tokens + 2 * (P - portions))
        if B + TP > self.max_mixed_tokens or TP > self.runner.max_model_len:
            return None
        return B, P, TP

    def accepts(self, entries: Sequence[StepEntry], rows) -> bool:
        """Should this step run as a captured graph? Steps of single tokens always; steps with
        portions once their shape has been asked for ``capture_after`` times."""
        if not self.capturable:
            return False
        if self.forward_usable(entries, rows):
            return True
        shape = self.mixed_shape(entries)
        if shape is None or len(rows) != sum(len(e.want) for e in entries):
            return False
        seen = self.asked[shape] = self.asked.get(shape, 0) + 1
        return seen >= self.capture_after

    @staticmethod
    def simple(rows) -> bool:
        """The sampling kernel alone serves these rows, so it is captured with the step."""
        for r in rows:
            if r.params.has_penalties or r.banned_token_ids or r.params.logprobs is not None:
                return False
        return True

    @staticmethod
    def usable(entries: Sequence[StepEntry], rows) -> bool:
        return DecodeGraphs.forward_usable(entries, rows) and DecodeGraphs.simple(rows)

    def _fill(self, g: _Graph, entries, rows, ahead: int = 0) -> int:
        """Write the step's inputs into the pinned buffer. ``ahead`` = 1 describes the step *after*
        one that is still running: every position is one further and the token ids are not known
        on the host (they are copied on the device from that step's samples)."""
        m = self.runner.manager
        B = g.batch
        tok, pos, ctx = g.hview("token_ids"), g.hview("positions"), g.hview("ctx_lens")
        slots, first = g.hview("state_slots"), g.hview("first_portion")
        for i, e in enumerate(entries):
            held = m.held[e.rid]
            c = held.computed + ahead
            tok[i] = e.tokens[0]
            pos[i] = c
            ctx[i] = c + 1
            slots[i] = s = held.slot
            first[i] = c == 0
            if self.mirror_epoch[s] != held.epoch:
                self.mirror_epoch[s] = held.epoch
                self.mirror_len[:, s] = 0
            for gi, table in enumerate(held.tables):
                known = self.mirror_len[gi, s]
                if len(table) > known:
                    self.mirror[gi][s, known : len(table)] = np.maximum(table[known:], 0)
                    self.mirror_len[gi, s] = len(table)
                need = -(-(c + 1) // m.groups[gi].page_tokens)
                if len(table) < need:
                    raise ValueError(f"request {e.rid!r}: block table has {len(table)} pages, needs {need}")
        n = len(entries)
        # padding rows: one token at position 0 of a sequence that lives on the spare page and slot
        tok[n:] = 0
        pos[n:] = 0
        ctx[n:] = 1
        slots[n:] = m.max_requests
        first[n:] = 1
        if int(ctx.max()) > self.runner.max_model_len:
            raise ValueError("a sequence would outgrow max_model_len")
        v = self.runner.model.plan.vocab_size
        if int(tok.min()) < 0 or int(tok.max()) >= v:
            raise ValueError(f"token ids must lie in [0, {v})")
        for gi, (o, w) in enumerate(g.table_off):
            g.h[o : o + B * w].reshape(B, w)[:] = self.mirror[gi][slots]
        if g.sampled:
            p = [r.params for r in rows]
            pad = [0] * (B - n)
            g.hview("temperature", np.float32)[:] = [q.temperature for q in p] + pad  # 0: greedy
            g.hview("top_k")[:] = [q.top_k for q in p] + pad
            g.hview("top_p", np.float32)[:] = [q.top_p for q in p] + [1.0] * (B - n)
            g.hview("min_p", np.float32)[:] = [q.min_p for q in p] + pad
            g.hview("draw")[:] = [r.draw_index for r in rows] + pad
            so = g.off["seed"]
            g.h[so : so + 2 * B].view(np.uint64)[:] = [r.seed & 0xFFFFFFFFFFFFFFFF for r in rows] + pad
        return int(ctx.max())

    def _fill_mixed(self, shape, entries):
        """The padded batch of a step with portions, as arrays; the graph's buffers are filled
        from them. Returns (arrays by buffer name, padded HostStep, row of each sampled entry)."""
        runner = self.runner
        m = runner.manager
        B, P, TP = shape
        N, T = B + P, B + TP
        order = sorted(range(len(entries)), key=lambda i: len(entries[i].tokens) != 1)
        host = build_host_step([entries[i] for i in order], m, runner.model.plan.vocab_size,
                               runner.max_model_len)
        nd = int((host.q_lens == 1).sum())
        npre = host.num_seqs - nd
        real = host.num_tokens - nd  # tokens of the real portions
        n_pad = P - npre
        pad_lens = np.full(n_pad, 2, dtype=np.int32)
        pad_lens[-1] = TP - real - 2 * (n_pad - 1)
        q_lens = np.ones(N, dtype=np.int32)
        q_lens[B : B + npre] = host.q_lens[nd:]
        q_lens[B + npre :] = pad_lens
        cu_q = np.zeros(N + 1, dtype=np.int32)
        np.cumsum(q_lens, out=cu_q[1:])
        tok = np.zeros(T, dtype=np.int32)
        tok[:nd] = host.token_ids[:nd]
        tok[B : B + real] = host.token_ids[nd:]
        pos = np.zeros(T, dtype=np.int32)
        pos[:nd] = host.positions[:nd]
        pos[B : B + real] = host.positions[nd:]
        pad_first = cu_q[B + npre : N]  # a padding sequence starts at position 0
        pos[B + real :] = np.arange(B + real, T, dtype=np.int32) - np.repeat(pad_first, pad_lens)
        ctx = np.ones(N, dtype=np.int32)
        ctx[:nd] = host.ctx_lens[:nd]
        ctx[B : B + npre] = host.ctx_lens[nd:]
        ctx[B + npre :] = pad_lens
        slots = np.full(N, m.max_requests, dtype=np.int32)  # the spare slot
        slots[:nd] = host.state_slots[:nd]
        slots[B : B + npre] = host.state_slots[nd:]
        first = np.ones(N, dtype=np.int32)
        first[:nd] = host.first_portion[:nd]
        first[B : B + npre] = host.first_portion[nd:]
        arrays = {"token_ids": tok, "positions": pos, "cu_q": cu_q, "ctx_lens": ctx,
                  "state_slots": slots, "first_portion": first, "logit_rows": cu_q[1:] - 1,
                  "token_seq": np.repeat(np.arange(N, dtype=np.int32), q_lens)}
        tables = []
        for gi, spec in enumerate(m.groups):
            w = -(-runner.max_model_len // spec.page_tokens)
            t = np.full((N, w), runner.pools.spare_page(gi), dtype=np.int32)
            ht = host.block_tables[gi]
            t[:nd, : ht.shape[1]] = ht[:nd]
            t[B : B + npre, : ht.shape[1]] = ht[nd:]
            arrays[("table", gi)] = t
            tables.append(t)
        padded = HostStep(token_ids=tok, positions=pos, token_seq=arrays["token_seq"], cu_q=cu_q,
                          q_lens=q_lens, ctx_lens=ctx, state_slots=slots, first_portion=first,
                          block_tables=tables, logit_rows=arrays["logit_rows"], rids=[])
        # where each sampled entry's row is: the last token of its sequence
        place = {}
        for k, i in enumerate(order):
            place[i] = k if k < nd else B + (k - nd)
        index = [place[i] for i, e in enumerate(entries) if len(e.want)]
        return arrays, padded, index

    def _plans_mixed(self, shape, padded: HostStep) -> dict:
        """The padded step's work lists, each filled up to its full size with its last row."""
        runner = self.runner
        B, P, TP = shape
        plans = {}
        for key, (mixer, cid) in runner.planners.items():
            plan = mixer.plan_step(padded, runner.pools.view(cid, False).group)
            rows = mixer.plan_rows(B, P, TP)
            out = {}
            for name, a in plan.items():
                want = rows[name]
                if a.shape[0] > want or (a.shape[0] == 0 and want > 0):
                    raise ValueError(f"work list {name!r} has {a.shape[0]} rows; the capture holds {want}")
                if a.shape[0] < want:
                    a = np.concatenate([a, np.repeat(a[-1:], want - a.shape[0], axis=0)])
                out[name] = np.ascontiguousarray(a, dtype=np.int32)
            plans[key] = out
        return plans

    def _launch_mixed(self, entries, rows, sampler) -> "Pending":
        runner = self.runner
        shape = self.mixed_shape(entries)
        if shape is None:
            raise ValueError("this step cannot run as a captured graph")
        B, P, TP = shape
        simple = self.simple(rows)
        if not simple and sampler is None:
            raise ValueError("these rows need a sampler")
        arrays, padded, index = self._fill_mixed(shape, entries)
        plans = self._plans_mixed(shape, padded)
        # context partitions as for the next power of two of the longest context: fewer shapes
        max_ctx = pow2_at_least(int(arrays["ctx_lens"][:B].max())) if B else 1
        splits = runner.ops.decode_splits(B, self.min_kv_heads, max_ctx) if B else 1
        # unsampled and padding rows are greedy, so the one-block kernel is always there
        kinds = (sample_kinds(r.params for r in rows) | 1) if simple else 0
        key = (B, P, TP, splits, simple, kinds)
        g = self.graphs.get(key)
        if g is None:
            g = self.graphs[key] = _MixedGraph(self, B, P, TP, splits, simple, kinds, plans)
        if g.h2d_done is not None:
            g.h2d_done.synchronize()
        for name, a in arrays.items():
            g.hview(name)[:] = a.reshape(-1)
        for pkey, plan in plans.items():
            for name, a in plan.items():
                g.hview(("plan", pkey, name))[:] = a.reshape(-1)
        if simple:
            N = g.N
            temp, top_k = np.zeros(N, np.float32), np.zeros(N, np.int32)
            top_p, min_p = np.ones(N, np.float32), np.zeros(N, np.float32)
            draw, seed = np.zeros(N, np.int32), np.zeros(N, np.uint64)
            for j, r in zip(index, rows):
                q = r.params
                temp[j], top_k[j], top_p[j], min_p[j] = q.temperature, q.top_k, q.top_p, q.min_p
                draw[j], seed[j] = r.draw_index, r.seed & 0xFFFFFFFFFFFFFFFF
            g.hview("temperature", np.float32)[:] = temp
            g.hview("top_k")[:] = top_k
            g.hview("top_p", np.float32)[:] = top_p
            g.hview("min_p", np.float32)[:] = min_p
            g.hview("draw")[:] = draw
            g.hview("seed", np.uint64)[:] = seed
        return self._replay(g, index, rows, simple, sampler)

    def _replay(self, g, index, rows, simple: bool, sampler, ahead_of=None) -> "Pending":
        """Copy the filled buffer, replay (capturing first if need be), start the read-back.
        ``index``: the batch rows that belong to ``rows``, in order."""
        runner = self.runner
        g.dev.copy_(g.host, non_blocking=True)
        g.h2d_done = torch.cuda.Event()
        g.h2d_done.record()
        if ahead_of is not None:
            g.step.token_ids.copy_(ahead_of.graph.tokens, non_blocking=True)
        if g.graph is None:
            self._capture(g)
        g.graph.replay()
        runner.ops.launches += g.launches
        runner.steps_run += 1
        if not simple:
            if index == list(range(len(index))):
                picked = g.logits[: len(index)]
            else:
                picked = g.logits[torch.tensor(index, dtype=torch.long, device=g.logits.device)]
            return Pending(g, None, None, index, sampler.sample(picked, rows))
        buf = g.tokens_host[g.turn]
        g.turn ^= 1
        buf.copy_(g.tokens, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return Pending(g, done, buf, index)

    def _forward(self, g):
        runner = self.runner
        logits = runner.model.forward(g.step, runner.pools)
        return runner.ops.sample(logits, *g.sample_args, kinds=g.kinds) if g.sampled else logits

    def _capture(self, g) -> None:
        """Run the step once uncaptured (lazy allocations happen here; its writes are idempotent),
        then record it. The record is made with ``capture_begin`` / ``capture_end`` rather than the
        ``torch.cuda.graph`` context, which collects garbage and empties the allocator's cache
        first: with captures made while requests are served that costs more than the capture."""
        ops = self.runner.ops
        cur = torch.cuda.current_stream()
        if self.side is None:
            self.side = torch.cuda.Stream()
        side = self.side
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            self._forward(g)
        cur.wait_stream(side)
        torch.cuda.synchronize()
        before = ops.launches
        g.graph = torch.cuda.CUDAGraph()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        # No cyclic garbage collection while the stream captures: an engine of earlier use that
        # is collected just then destroys its graphs, which is not permitted during a capture and
        # would invalidate this one.
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.stream(side):
                g.graph.capture_begin(pool=self.pool)
                try:
                    out = self._forward(g)
                finally:
                    g.graph.capture_end()
        finally:
            if collecting:
                gc.enable()
        cur.wait_stream(side)
        if g.sampled:
            g.tokens = out
        else:
            g.logits = out
        g.launches = ops.launches - before

    def launch(self, entries: Sequence[StepEntry], rows, ahead_of: "Pending | None" = None,
               sampler=None) -> "Pending":
        """Enqueue a step (inputs copy, graph replay, token read-back) without waiting for it.

        With ``ahead_of`` the step continues the same sequences one position after that still
        running step and takes its input token ids on the device from that step's samples.
        Rows that the sampling kernel alone cannot serve need ``sampler``: the replay then ends
        with the logits and the sampler runs on them before this method returns.
        """
        runner = self.runner
        if not self.capturable:
            raise ValueError("this model has a part that works from the host: its steps are not captured")
        if not self.forward_usable(entries, rows):
            if ahead_of is not None:
                raise ValueError("only a step of single tokens can run ahead")
            return self._launch_mixed(entries, rows, sampler)
        n = len(entries)
        B = self.padded(n)
        simple = self.simple(rows)
        if not simple and (sampler is None or ahead_of is not None):
            raise ValueError("these rows need a sampler and cannot run ahead")
        ahead = 0 if ahead_of is None else 1
        max_ctx = 1 + ahead + max(runner.manager.held[e.rid].computed for e in entries)
        splits = runner.ops.decode_splits(B, self.min_kv_heads, max_ctx)
        # padding rows are greedy, so a padded batch always holds the one-block kernel
        kinds = (sample_kinds(r.params for r in rows) | (1 if B > n else 0)) if simple else 0
        key = (B, splits, simple, kinds)
        g = self.graphs.get(key)
        if g is None:
            g = self.graphs[key] = _Graph(self, B, splits, simple, kinds)
        if g.h2d_done is not None:
            g.h2d_done.synchronize()
        self._fill(g, entries, rows, ahead)
        return self._replay(g, list(range(n)), rows, simple, sampler, ahead_of)

    def captured_logits(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Float32 logits of a step of single tokens, run as a captured graph: what a check of
        the captured path against the kernel-by-kernel path compares. Pages for the tokens must
        have been allocated; nothing is committed."""
        if not all(len(e.tokens) == 1 for e in entries):
            raise ValueError("only a step of single tokens")
        runner = self.runner
        n = len(entries)
        B = self.padded(n)
        max_ctx = 1 + max(runner.manager.held[e.rid].computed for e in entries)
        splits = runner.ops.decode_splits(B, self.min_kv_heads, max_ctx)
        key = (B, splits, False, 0)
        g = self.graphs.get(key)
        if g is None:
            g = self.graphs[key] = _Graph(self, B, splits, False, 0)
        if g.h2d_done is not None:
            g.h2d_done.synchronize()
        self._fill(g, entries, [], 0)
        g.dev.copy_(g.host, non_blocking=True)
        g.h2d_done = torch.cuda.Event()
        g.h2d_done.record()
        if g.graph is None:
            self._capture(g)
        g.graph.replay()
        runner.ops.launches += g.launches
        return g.logits[:n].clone()

    @staticmethod
    def collect(pending: "Pending"):
        """The step's :class:`~llmserve_b200.sampling.sampler.SamplerOutput` (waits for it)."""
        from ..sampling.sampler import SamplerOutput

        if pending.result is not None:
            return pending.result
        pending.done.synchronize()
        tokens = pending.tokens_host.tolist()
        return SamplerOutput([tokens[i] for i in pending.index], None, None)

    def collect_checked(self, pending: "Pending"):
        """:meth:`collect`, then raise if a kernel of the step gave up a bounded wait (its results
        would be wrong; the flag lives in host memory and is read once the step has finished)."""
        out = self.collect(pending)
        self.runner.ops.check_kernel_errors()
        return out

    def run(self, entries: Sequence[StepEntry], rows, sampler=None):
        return self.collect(self.launch(entries, rows, sampler=sampler))


class Pending:
    """A launched step whose sampled tokens have not been read yet (``result``: already sampled)."""

    def __init__(self, graph, done, tokens_host, index: list[int], result=None) -> None:
        self.graph, self.done, self.tokens_host, self.result = graph, done, tokens_host, result
        self.index = index  # the batch rows that are sampled requests, in the order of the step's rows
        # the graph's samples are, row by row, the next step's input tokens
        self.feeds_next = graph.slots == 0 and result is None
