"""The engine: request intake, the step loop, and the offline ``LLM`` API.

Names and meanings follow src/llmserve/engine.py (``EngineConfig`` :30-66, ``LLMEngine`` :83-533,
``LLM`` :536-577) where they apply to one GPU and unquantized weights.
"""

from __future__ import annotations

import contextlib
import itertools
import random
import time
from dataclasses import dataclass

from ..config.registry import architecture_for
from ..models.hub import preset_config_dict, resolve_model_path
from ..sampling import Sampler, SampleRow, SamplingParams
from ..weights.random_init import random_parameters
from .batch import StepEntry
from .detokenizer import TextStream, find_stop
from .runner import ModelRunner, build_model, load_model, resolve_dtype
from .scheduler import Scheduler, SchedulerConfig
from .sequence import Request, RequestOutput, Sequence


@dataclass
class EngineConfig:
    model: str = "smollm2-135m"  # folder, alias under $LLMSERVE_MODELS, or "random:<alias>"
    dtype: str = "bfloat16"  # "bfloat16" | "float32" (true 32-bit everywhere)
    device: str = "cuda"
    block_size: int = 16  # tokens per cache page
    kv_cache_memory_gb: float = 2.0  # used when num_kv_blocks is None
    num_kv_blocks: int | None = None
    max_model_len: int = 4096
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 1024
    enable_chunked_prefill: bool = True
    enable_prefix_caching: bool = False  # not built: pages are reused, their contents are not
    seed: int = 0  # weights seed of "random:<alias>" models
    cuda_graphs: bool = True  # replay captured graphs for steps of single tokens only
    run_ahead: bool = True  # launch the next decode step before this one's tokens are read
    warm_up: bool = True  # run a throw-away step at start-up (library handles, kernel modules)
    profile: bool = False  # time every step on the device with CUDA events and mark it with an NVTX range
    config_overrides: dict | None = None  # config.json keys to replace in a "random:<alias>" model

    def scheduler_config(self) -> SchedulerConfig:
        return SchedulerConfig(
            max_num_seqs=self.max_num_seqs,
            max_num_batched_tokens=self.max_num_batched_tokens,
            enable_chunked_prefill=self.enable_chunked_prefill,
            max_model_len=self.max_model_len,
        )


class _InFlight:
    """A step that has been launched: who was scheduled, and the handle or result of the GPU work."""

    def __init__(self, scheduled, sample_seqs, stats, t0) -> None:
        self.scheduled = scheduled  # [(sequence, new tokens)]
        self.sample_seqs = sample_seqs
        self.stats = stats
        self.t0 = t0
        self.t_launched = t0  # when the step's kernels had been enqueued
        self.gpu_events = None  # (before, after) the step on the stream, with EngineConfig.profile
        self.pending = None  # handle of a launched CUDA-graph step
        self.result = None  # SamplerOutput of a step that ran synchronously


@dataclass
class StepStats:
    """What the last finished step did and where its time went. The ``t_*`` are host wall-clock
    seconds (names of src/llmserve/engine.py:70-80); ``gpu_ms`` is the device time between the
    step's launch and the end of its sampling, from CUDA events, when ``EngineConfig.profile`` is
    set (it costs a synchronisation per step)."""

    num_seqs: int = 0
    num_tokens: int = 0
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0
    num_preempted: int = 0
    step_time: float = 0.0
    t_schedule: float = 0.0
    t_forward: float = 0.0  # building the batch, uploading it, launching the model's kernels
    t_sample: float = 0.0  # waiting for the device and reading the sampled tokens back
    t_postprocess: float = 0.0  # appending tokens, text, stop checks, output objects
    gpu_ms: float | None = None


class LLMEngine:
    def __init__(self, cfg: EngineConfig, ops=None, tokenizer=None) -> None:
        self.cfg = cfg
        if cfg.enable_prefix_caching:
            raise ValueError("enable_prefix_caching=True: prefix caching is not built")
        dtype = resolve_dtype(cfg.dtype)
        if ops is None:
            from ..ops import get_ops

            ops = get_ops(cfg.device)
        self.ops = ops
        if cfg.model.startswith("random:"):
            d = {**preset_config_dict(cfg.model.split(":", 1)[1]), **(cfg.config_overrides or {})}
            arch = architecture_for(d)
            mcfg = arch.config_cls.from_dict(d)
            self.model = build_model(
                arch, mcfg,
                lambda layout, dt, dev: random_parameters(arch, mcfg, cfg.seed, dt, dev),
                dtype, cfg.device, ops, cfg.max_model_len,
            )
            path = None
        else:
            path = resolve_model_path(cfg.model)
            arch, mcfg, self.model = load_model(path, dtype, cfg.device, ops, cfg.max_model_len)
        self.model_cfg = mcfg
        if tokenizer is None and path is not None and any(
            (path / f).exists() for f in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json")
        ):
            from transformers import AutoTokenizer  # a tokenizer, not model code

            tokenizer = AutoTokenizer.from_pretrained(str(path))
        self.tokenizer = tokenizer
        self.runner = ModelRunner(
            self.model,
            page_tokens=cfg.block_size,
            num_pages=cfg.num_kv_blocks,
            cache_memory_bytes=int(cfg.kv_cache_memory_gb * 2**30),
            max_model_len=cfg.max_model_len,
            max_num_seqs=cfg.max_num_seqs,
            max_num_batched_tokens=cfg.max_num_batched_tokens,
        )
        self.manager = self.runner.manager
        self.scheduler = Scheduler(cfg.scheduler_config(), self.manager)
        self.sampler = Sampler(ops, cfg.device, max_slots=self.manager.max_requests)
        self.requests: dict[str, Request] = {}
        self._seq_ids = itertools.count()
        self._req_ids = itertools.count()
        self._seed_source = random.Random()
        self.eos_ids = set(getattr(mcfg, "eos_token_ids", ()))
        if tokenizer is not None and getattr(tokenizer, "eos_token_id", None) is not None:
            self.eos_ids.add(tokenizer.eos_token_id)
        self.last_step = StepStats()
        self.total_steps = 0
        self._pending: _InFlight | None = None  # a step launched ahead, not yet collected
        if cfg.warm_up and self.runner.device.type == "cuda":
            self._warm_up()

    def _warm_up(self) -> None:
        """One throw-away portion of a prompt (as long as the token budget, the size that a loaded
        engine runs most) and one single token, sampled, on a request that is released again: the
        first use of a process creates library handles and workspaces and loads kernel modules
        (0.2 s and more), which would otherwise be the first request's wait."""
        n = min(2048, self.cfg.max_num_batched_tokens, self.cfg.max_model_len - 2)
        if n < 2 or not self.manager.fits_at_all(n + 1, n):
            return
        rid = ("warm-up",)
        row = SampleRow(SamplingParams(temperature=0.0), [], [0], 0)
        self.manager.admit(rid)
        try:
            for tokens in ([0] * n, [0]):
                self.manager.allocate(rid, len(tokens))
                self.runner.step_and_sample([StepEntry(rid, tokens, [len(tokens) - 1])], self.sampler, [row])
                self.manager.commit(rid, len(tokens))
        finally:
            self.manager.release(rid)

    # ------------------------------------------------------------------ intake
    def add_request(self, prompt: str | list[int], params: SamplingParams | None = None,
                    request_id: str | None = None, arrival_time: float | None = None) -> str:
        """Queue a prompt (text, if the engine has a tokenizer, or token ids). Returns the request's
        id. A request that could never run is refused here (src/llmserve/engine.py:237-245)."""
        params = params or SamplingParams()
        text, ids = self._token_ids(prompt)
        self._refuse_what_can_never_run(ids, params)
        rid = request_id if request_id else f"req-{next(self._req_ids)}"
        if rid in self.requests:
            raise ValueError(f"duplicate request id {rid}")
        request = Request(rid, text, ids, params, arrival_time)
        # a request without a seed draws one, so that its samples too come from the device
        # generator keyed by (seed, token index, vocabulary index)
        seed = self._seed_source.getrandbits(63) if params.seed is None else params.seed
        seq = Sequence(next(self._seq_ids), request, ids, seed)
        if self.tokenizer is not None:
            seq.text_stream = TextStream(self.tokenizer, ids)
        request.seqs.append(seq)
        self.requests[rid] = request
        self.scheduler.add(seq)
        return rid

    def _token_ids(self, prompt) -> tuple[str | None, list[int]]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("text prompts need a tokenizer")
            return prompt, list(self.tokenizer(prompt, add_special_tokens=False).input_ids)
        return None, [int(t) for t in prompt]

    def _refuse_what_can_never_run(self, ids: list[int], params: SamplingParams) -> None:
        limit, vocab = self.cfg.max_model_len, self.model_cfg.vocab_size
        if not ids:
            raise ValueError("empty prompt")
        if len(ids) >= limit:
            raise ValueError(f"prompt has {len(ids)} tokens; max_model_len is {limit}")
        if min(ids) < 0 or max(ids) >= vocab:
            raise ValueError(f"prompt token ids must lie in [0, {vocab})")
        longest = min(len(ids) + params.max_tokens, limit)
        if not self.manager.fits_at_all(longest, self.cfg.max_num_batched_tokens):
            raise ValueError("request can never fit in the KV cache; raise kv_cache_memory_gb")

    def abort_request(self, request_id: str) -> None:
        """Stop a request wherever it is; what it holds is given back at once. Unknown ids are ignored."""
        request = self.requests.pop(request_id, None)
        for seq in (request.seqs if request is not None else ()):
            if not seq.is_finished:
                seq.finish_reason = "abort"
                self.scheduler.finish(seq)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished()

    @property
    def num_unfinished_requests(self) -> int:
        return len(self.requests)

    # ------------------------------------------------------------------ step
    def step(self) -> list[RequestOutput]:
        """One engine iteration: returns the outputs of the step it completes.

        Steps of single tokens are launched as CUDA graphs without waiting. Before the tokens of
        such a step are read, the step after it is launched *ahead* when nothing can change the
        batch in between (nobody can finish by length, nobody waits, pages are there): its input
        token ids are copied on the device from the running step's samples. So the host's work
        (reading tokens, stop checks, outputs, preparing inputs) overlaps the GPU's. If a sequence
        does end (EOS, stop token, abort), the step launched ahead is dropped; what it wrote lies
        beyond every live sequence's committed tokens and is never read.
        """
        cur = self._pending
        self._pending = None
        if cur is not None and all(seq.is_finished for seq, _ in cur.scheduled):
            self.runner.collect_decode(cur.pending)  # every sequence of it was aborted: nothing to keep
            cur = None
        if cur is None:
            cur = self._start_step()
            if cur is None:
                return []
        ahead = self._launch_ahead(cur)
        outputs, unchanged = self._finish_step(cur)
        if ahead is not None and unchanged:
            self._pending = ahead
        return outputs

    def _start_step(self):
        t0 = time.monotonic()
        sched = self.scheduler.schedule()
        t1 = time.monotonic()
        stats = StepStats(num_preempted=len(sched.preempted), t_schedule=t1 - t0)
        if sched.is_empty:
            self.last_step = stats
            return None
        # Sequences that reach the end of their known tokens this step get a new token
        # (src/llmserve/engine.py:323-332); the others are in the middle of a prompt.
        entries, sample_seqs = [], []
        for s in sched.scheduled:
            seq, n = s.seq, s.num_new_tokens
            last = seq.num_computed_tokens + n == seq.num_tokens
            entries.append(StepEntry(seq.seq_id, seq.tokens_from(seq.num_computed_tokens, n),
                                     [n - 1] if last else []))
            if last:
                sample_seqs.append(seq)
        rows = [self._sample_row(seq) for seq in sample_seqs]
        scheduled = [(s.seq, s.num_new_tokens) for s in sched.scheduled]
        flight = _InFlight(scheduled, sample_seqs, stats, t0)
        with self._profiled(flight, sum(n for _, n in scheduled)):
            if self.cfg.cuda_graphs and self.runner.can_launch_decode(entries, rows):
                flight.pending = self.runner.launch_decode(entries, rows, sampler=self.sampler)
            else:
                flight.result = self.runner.step_and_sample(entries, self.sampler, rows, graphs=False)
        flight.t_launched = time.monotonic()
        return flight

    @contextlib.contextmanager
    def _profiled(self, flight: "_InFlight", tokens: int):
        """With ``EngineConfig.profile``: CUDA events around the step's work on the stream and an
        NVTX range around its launch, so a timeline shows which kernels belong to which step."""
        if not (self.cfg.profile and self.runner.device.type == "cuda"):
            yield
            return
        import torch

        before, after = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.nvtx.range_push(f"step {self.total_steps}: {len(flight.scheduled)} sequences, {tokens} tokens")
        before.record()
        try:
            yield
        finally:
            after.record()
            torch.cuda.nvtx.range_pop()
            flight.gpu_events = (before, after)

    def _launch_ahead(self, cur: "_InFlight"):
        """Launch the step after ``cur`` before ``cur``'s tokens are known, if the batch cannot change."""
        if cur.pending is None or not self.cfg.run_ahead or self.scheduler.waiting:
            return None
        if not cur.pending.feeds_next:  # sampled outside the graph, or rows in another order
            return None
        seqs = cur.sample_seqs
        if len(seqs) != len(cur.scheduled) or len(seqs) != len(self.scheduler.running):
            return None
        if len(seqs) > self.cfg.max_num_batched_tokens:
            return None
        for seq in seqs:
            p = seq.params
            if (seq.is_finished or len(seq.output_token_ids) + 1 >= p.max_tokens
                    or seq.num_tokens + 1 >= self.cfg.max_model_len):
                return None
        if not self._pages_for_all(seqs, 2):
            return None
        rows = [self._sample_row(seq, ahead=1) for seq in seqs]
        entries = [StepEntry(seq.seq_id, [0], [0]) for seq in seqs]
        from .decode_graph import DecodeGraphs

        if not (self.runner.can_launch_decode(entries, rows) and DecodeGraphs.simple(rows)):
            return None
        for seq in seqs:
            self.manager.allocate(seq.seq_id, 2)
        t0 = time.monotonic()
        flight = _InFlight([(seq, 1) for seq in seqs], list(seqs), StepStats(), t0)
        with self._profiled(flight, len(seqs)):
            flight.pending = self.runner.launch_decode(entries, rows, ahead_of=cur.pending)
        flight.t_launched = time.monotonic()
        return flight

    def _pages_for_all(self, seqs, n: int) -> bool:
        """Are there pages for ``n`` more tokens of *every* one of ``seqs`` at once? The needs are
        added up group by group: each sequence alone may fit while all of them together do not
        (equal prompts cross a page's edge in the same step), and then the step is not launched
        ahead, so that the scheduler can preempt in the next one."""
        need = [0] * len(self.manager.groups)
        for seq in seqs:
            for g, k in enumerate(self.manager.pages_needed(seq.seq_id, n)):
                need[g] += k
        return all(k <= self.manager.num_free_pages(g) for g, k in enumerate(need))

    def _finish_step(self, cur: "_InFlight"):
        """Read the step's tokens and do the host's part. Returns (outputs, batch unchanged)."""
        stats = cur.stats
        t_wait = time.monotonic()
        result = self.runner.collect_decode(cur.pending) if cur.pending is not None else cur.result
        tokens, logprobs, tops = result.token_ids, result.logprobs, result.top_logprobs
        t_host = time.monotonic()
        stats.t_forward = cur.t_launched - cur.t0 - stats.t_schedule
        stats.t_sample = t_host - t_wait
        if cur.gpu_events is not None:
            cur.gpu_events[1].synchronize()
            stats.gpu_ms = cur.gpu_events[0].elapsed_time(cur.gpu_events[1])
        unchanged = True
        for seq, n in cur.scheduled:
            if seq.is_finished:  # aborted while the step ran
                unchanged = False
                continue
            self.manager.commit(seq.seq_id, n)
            seq.num_computed_tokens += n
            if n == 1 and seq.output_token_ids:
                stats.num_decode_tokens += 1
            else:
                stats.num_prefill_tokens += n
        touched: dict[str, Request] = {}
        for j, seq in enumerate(cur.sample_seqs):
            if seq.is_finished:
                continue
            seq.request.metrics.token_at(t_host)
            seq.output_token_ids.append(tokens[j])
            if logprobs is not None:
                seq.logprobs.append(logprobs[j])
                seq.top_logprobs.append(tops[j])
            reason = self._why_finished(seq, tokens[j])
            if reason is not None:
                seq.finish_reason = reason
                self.scheduler.finish(seq)
                unchanged = False
            touched[seq.request.request_id] = seq.request
        outputs = []
        for request in touched.values():
            if request.is_finished:
                request.metrics.finished_time = t_host
                self.requests.pop(request.request_id, None)
            outputs.append(RequestOutput.of(request))
        done = time.monotonic()
        stats.num_seqs = len(cur.scheduled)
        stats.num_tokens = sum(n for _, n in cur.scheduled)
        stats.t_postprocess = done - t_host
        stats.step_time = done - cur.t0
        self.last_step = stats
        self.total_steps += 1
        return outputs, unchanged

    def _sample_row(self, seq: Sequence, ahead: int = 0) -> SampleRow:
        """``ahead`` = 1: the row of the token *after* the one that is being sampled right now."""
        p = seq.params
        n_out = len(seq.output_token_ids) + ahead
        banned = []
        if n_out < p.min_tokens:
            banned = sorted(self.eos_ids | set(p.stop_token_ids))
        held = self.manager.held.get(seq.seq_id) if p.has_penalties else None
        return SampleRow(p, seq.output_token_ids, seq.prompt_token_ids, seq.seed, banned,
                         draw=n_out if ahead else None,
                         slot=held.slot if held is not None else -1,
                         epoch=held.epoch if held is not None else 0)

    def _why_finished(self, seq: Sequence, token: int) -> str | None:
        """``seq`` has just received ``token``: bring its text up to date and say whether, and
        why, it ends here. Stops are looked for before the length limits, a stop token before a
        stop string (the order of src/llmserve/engine.py:475-491)."""
        p = seq.params
        fresh = ""
        if seq.text_stream is not None:
            fresh = seq.text_stream.push(seq.token_ids())
            seq.output_text += fresh
        if token in p.stop_token_ids or (token in self.eos_ids and not p.ignore_eos):
            seq.stop_reason = token
            return "stop"
        if fresh and p.stop:
            hit = find_stop(seq.output_text, len(fresh), p.stop)
            if hit is not None:
                begins, stop = hit
                keep = begins + len(stop) if p.include_stop_str_in_output else begins
                seq.output_text = seq.output_text[:keep]
                seq.stop_reason = stop
                return "stop"
        if len(seq.output_token_ids) >= p.max_tokens or seq.num_tokens >= self.cfg.max_model_len:
            return "length"
        return None

    def stats(self) -> dict:
        """Counters of the engine as it stands, and the kernel set that really runs."""
        sched = self.scheduler
        return dict(num_running=len(sched.running), num_waiting=len(sched.waiting),
                    num_preemptions=sched.num_preemptions, kv_cache_usage=self.manager.usage(),
                    num_kv_blocks=self.manager.num_pages(0), kernel_set=self.ops.name)


class LLM:
    """Offline use: ``LLM(model="random:smollm2-135m").generate(prompts, params)``
    (the entry point of src/llmserve/engine.py:536-577)."""

    def __init__(self, model: str = "smollm2-135m", ops=None, tokenizer=None, **kwargs) -> None:
        self.engine = LLMEngine(EngineConfig(model=model, **kwargs), ops=ops, tokenizer=tokenizer)
        self.tokenizer = self.engine.tokenizer

    def generate(self, prompts, params: SamplingParams | list[SamplingParams] | None = None,
                 use_tqdm: bool = False) -> list[RequestOutput]:
        """One output per prompt, in the order of the prompts. ``prompts``: a text, a list of
        token ids, or a list of either; ``params``: one for all, or one per prompt."""
        one = isinstance(prompts, str) or (len(prompts) > 0 and isinstance(prompts[0], int))
        batch = [prompts] if one else list(prompts)
        each = params if isinstance(params, list) else [params or SamplingParams()] * len(batch)
        if len(each) != len(batch):
            raise ValueError(f"{len(batch)} prompts but {len(each)} sampling parameters")
        order = [self.engine.add_request(p, sp) for p, sp in zip(batch, each)]
        finished: dict[str, RequestOutput] = {}
        while self.engine.has_unfinished_requests():
            finished.update((o.request_id, o) for o in self.engine.step() if o.finished)
        return [finished[rid] for rid in order]

    def chat(self, messages_list, params=None, **template_options) -> list[RequestOutput]:
        """``generate`` on conversations (lists of ``{"role", "content"}``), through the
        tokenizer's chat template with the turn of the assistant opened."""
        if self.tokenizer is None:
            raise ValueError("chat needs a tokenizer with a chat template")
        if messages_list and isinstance(messages_list[0], dict):
            messages_list = [messages_list]
        render = self.tokenizer.apply_chat_template
        return self.generate([render(m, tokenize=False, add_generation_prompt=True, **template_options)
                              for m in messages_list], params)
