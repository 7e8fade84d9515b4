"""CUDA graphs for steps that hold single tokens only.

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

The graph runs the same model code, kernels and cache as an uncaptured step; only the launch
mechanism differs.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ..sampling.sampler import sample_kinds
from .batch import DeviceStep, StepEntry


class _Graph:
    def __init__(self, owner: "DecodeGraphs", batch: int, splits: int, sampled: bool = True,
                 kinds: int = 3) -> None:
        runner = owner.runner
        self.batch = B = batch
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
            decode_splits=splits, plans=plans, host=None,
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
        self.graphs: dict[tuple[int, int, bool, int], _Graph] = {}
        self.pool = None
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

    def _forward(self, g: _Graph):
        runner = self.runner
        logits = runner.model.forward(g.step, runner.pools)
        return runner.ops.sample(logits, *g.sample_args, kinds=g.kinds) if g.sampled else logits

    def _capture(self, g: _Graph) -> None:
        ops = self.runner.ops
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(2):  # warm-up on the step's own data: the writes are idempotent
                self._forward(g)
        cur.wait_stream(side)
        torch.cuda.synchronize()
        before = ops.launches
        g.graph = torch.cuda.CUDAGraph()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(g.graph, pool=self.pool):
            out = self._forward(g)
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
            return Pending(g, None, None, n, sampler.sample(g.logits[:n], rows))
        buf = g.tokens_host[g.turn]
        g.turn ^= 1
        buf.copy_(g.tokens, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return Pending(g, done, buf, n)

    @staticmethod
    def collect(pending: "Pending"):
        """The step's :class:`~llmserve_b200.sampling.sampler.SamplerOutput` (waits for it)."""
        from ..sampling.sampler import SamplerOutput

        if pending.result is not None:
            return pending.result
        pending.done.synchronize()
        return SamplerOutput(pending.tokens_host.tolist()[: pending.rows], None, None)

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

    def __init__(self, graph: _Graph, done, tokens_host, rows: int, result=None) -> None:
        self.graph, self.done, self.tokens_host, self.result = graph, done, tokens_host, result
        self.rows = rows  # rows of the batch that are requests (the rest pads the captured size)
