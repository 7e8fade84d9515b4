"""The engine: request intake, the step loop, and the offline ``LLM`` API.

Names and meanings follow src/llmserve/engine.py (``EngineConfig`` :30-66, ``LLMEngine`` :83-533,
``LLM`` :536-577) where they apply to one GPU and unquantized weights.
"""

from __future__ import annotations

import itertools
import random
import time
from dataclasses import dataclass

from ..config.registry import architecture_for
from ..models.hub import preset_config_dict, resolve_model_path
from ..sampling import Sampler, SampleRow, SamplingParams
from ..weights.random_init import random_parameters
from .batch import StepEntry
from .detokenizer import IncrementalDetokenizer, find_stop
from .runner import ModelRunner, build_model, load_model, resolve_dtype
from .scheduler import Scheduler, SchedulerConfig
from .sequence import CompletionOutput, Request, RequestOutput, Sequence


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
    config_overrides: dict | None = None  # config.json keys to replace in a "random:<alias>" model

    def scheduler_config(self) -> SchedulerConfig:
        return SchedulerConfig(
            max_num_seqs=self.max_num_seqs,
            max_num_batched_tokens=self.max_num_batched_tokens,
            enable_chunked_prefill=self.enable_chunked_prefill,
            max_model_len=self.max_model_len,
        )


@dataclass
class StepStats:
    num_seqs: int = 0
    num_tokens: int = 0
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0
    num_preempted: int = 0
    step_time: float = 0.0
    t_schedule: float = 0.0
    t_forward: float = 0.0  # input preparation, model forward, sampling kernels, token read-back
    t_sample: float = 0.0
    t_postprocess: float = 0.0


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
        self.sampler = Sampler(ops, cfg.device)
        self.detok = IncrementalDetokenizer(tokenizer) if tokenizer is not None else None
        self.requests: dict[str, Request] = {}
        self._seq_ids = itertools.count()
        self._req_ids = itertools.count()
        self._seed_source = random.Random()
        self.eos_ids = set(getattr(mcfg, "eos_token_ids", ()))
        if tokenizer is not None and getattr(tokenizer, "eos_token_id", None) is not None:
            self.eos_ids.add(tokenizer.eos_token_id)
        self.last_step = StepStats()
        self.total_steps = 0

    # ------------------------------------------------------------------ intake
    def add_request(self, prompt: str | list[int], params: SamplingParams | None = None,
                    request_id: str | None = None, arrival_time: float | None = None) -> str:
        params = params or SamplingParams()
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("text prompts need a tokenizer")
            ids = list(self.tokenizer(prompt, add_special_tokens=False).input_ids)
            text = prompt
        else:
            ids, text = [int(t) for t in prompt], None
        if not ids:
            raise ValueError("empty prompt")
        if len(ids) >= self.cfg.max_model_len:
            raise ValueError(f"prompt has {len(ids)} tokens; max_model_len is {self.cfg.max_model_len}")
        v = self.model_cfg.vocab_size
        if min(ids) < 0 or max(ids) >= v:
            raise ValueError(f"prompt token ids must lie in [0, {v})")
        total = min(len(ids) + params.max_tokens, self.cfg.max_model_len)
        if not self.manager.fits_at_all(total, self.cfg.max_num_batched_tokens):
            raise ValueError("request can never fit in the KV cache; raise kv_cache_memory_gb")
        rid = request_id or f"req-{next(self._req_ids)}"
        if rid in self.requests:
            raise ValueError(f"duplicate request id {rid}")
        req = Request(rid, text, ids, params, arrival_time)
        seed = params.seed if params.seed is not None else self._seed_source.getrandbits(63)
        seq = Sequence(next(self._seq_ids), req, ids, seed)
        if self.detok is not None:
            seq.detok_state = self.detok.init_state(ids)
        req.seqs.append(seq)
        self.requests[rid] = req
        self.scheduler.add(seq)
        return rid

    def abort_request(self, request_id: str) -> None:
        req = self.requests.pop(request_id, None)
        if req is None:
            return
        for s in req.seqs:
            if not s.is_finished:
                s.finish_reason = "abort"
                self.scheduler.finish(s)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished()

    @property
    def num_unfinished_requests(self) -> int:
        return len(self.requests)

    # ------------------------------------------------------------------ step
    def step(self) -> list[RequestOutput]:
        t0 = time.monotonic()
        sched = self.scheduler.schedule()
        t1 = time.monotonic()
        stats = StepStats(num_preempted=len(sched.preempted), t_schedule=t1 - t0)
        if sched.is_empty:
            self.last_step = stats
            return []
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
        out = self.runner.step_and_sample(entries, self.sampler, rows, graphs=self.cfg.cuda_graphs)
        t2 = time.monotonic()
        stats.t_forward = t2 - t1
        for s in sched.scheduled:
            self.manager.commit(s.seq.seq_id, s.num_new_tokens)
            s.seq.num_computed_tokens += s.num_new_tokens
            if s.num_new_tokens == 1 and s.seq.output_token_ids:
                stats.num_decode_tokens += 1
            else:
                stats.num_prefill_tokens += s.num_new_tokens
        now = time.monotonic()
        touched: dict[str, Request] = {}
        for j, seq in enumerate(sample_seqs):
            self._append_token(
                seq, out.token_ids[j],
                None if out.logprobs is None else out.logprobs[j],
                None if out.top_logprobs is None else out.top_logprobs[j], now)
            touched[seq.request.request_id] = seq.request
        stats.num_seqs = len(sched.scheduled)
        stats.num_tokens = sched.num_tokens
        stats.step_time = time.monotonic() - t0
        stats.t_postprocess = stats.step_time - stats.t_schedule - stats.t_forward
        self.last_step = stats
        self.total_steps += 1
        outputs = []
        for req in touched.values():
            outputs.append(self._make_output(req))
            if req.is_finished:
                req.metrics.finished_time = now
                self.requests.pop(req.request_id, None)
        return outputs

    def _sample_row(self, seq: Sequence) -> SampleRow:
        p = seq.params
        banned = []
        if len(seq.output_token_ids) < p.min_tokens:
            banned = sorted(self.eos_ids | set(p.stop_token_ids))
        return SampleRow(p, seq.output_token_ids, seq.prompt_token_ids, seq.seed, banned)

    def _append_token(self, seq, token, logprob, top, now) -> None:
        req = seq.request
        if req.metrics.first_token_time is None:
            req.metrics.first_token_time = now
        req.metrics.last_token_time = now
        req.metrics.token_times.append(now)
        seq.output_token_ids.append(token)
        if logprob is not None:
            seq.logprobs.append(logprob)
            seq.top_logprobs.append(top)
        p = seq.params
        new_text = ""
        if self.detok is not None:
            new_text = self.detok.step(seq.token_ids(), seq.detok_state)
            seq.output_text += new_text
        # finish checks in the reference's order (src/llmserve/engine.py:475-491)
        reason = None
        if (not p.ignore_eos and token in self.eos_ids) or token in p.stop_token_ids:
            reason, seq.stop_reason = "stop", token
        elif p.stop and new_text:
            hit = find_stop(seq.output_text, len(new_text), p.stop)
            if hit is not None:
                idx, s = hit
                seq.output_text = seq.output_text[: idx + (len(s) if p.include_stop_str_in_output else 0)]
                reason, seq.stop_reason = "stop", s
        if reason is None and (len(seq.output_token_ids) >= p.max_tokens
                               or seq.num_tokens >= self.cfg.max_model_len):
            reason = "length"
        if reason is not None:
            seq.finish_reason = reason
            self.scheduler.finish(seq)

    def _make_output(self, req: Request) -> RequestOutput:
        outs = [
            CompletionOutput(
                index=s.index, text=s.output_text, token_ids=list(s.output_token_ids),
                finish_reason=s.finish_reason, stop_reason=s.stop_reason,
                logprobs=list(s.logprobs) if s.params.logprobs is not None else None,
                top_logprobs=list(s.top_logprobs) if s.params.logprobs is not None else None,
            )
            for s in req.seqs
        ]
        return RequestOutput(req.request_id, req.prompt, req.prompt_token_ids, outs,
                             req.is_finished, 0, req.metrics)

    def stats(self) -> dict:
        return {
            "num_running": len(self.scheduler.running),
            "num_waiting": len(self.scheduler.waiting),
            "kv_cache_usage": self.manager.usage(),
            "num_kv_blocks": self.manager.num_pages(0),
            "num_preemptions": self.scheduler.num_preemptions,
            "kernel_set": self.ops.name,
        }


class LLM:
    """Offline batch API: ``LLM(model="random:smollm2-135m").generate(prompts, params)``."""

    def __init__(self, model: str = "smollm2-135m", ops=None, tokenizer=None, **kwargs) -> None:
        self.engine = LLMEngine(EngineConfig(model=model, **kwargs), ops=ops, tokenizer=tokenizer)
        self.tokenizer = self.engine.tokenizer

    def generate(self, prompts, params: SamplingParams | list[SamplingParams] | None = None,
                 use_tqdm: bool = False) -> list[RequestOutput]:
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        if not isinstance(params, list):
            params = [params or SamplingParams()] * len(prompts)
        ids = [self.engine.add_request(p, sp) for p, sp in zip(prompts, params, strict=True)]
        done: dict[str, RequestOutput] = {}
        while self.engine.has_unfinished_requests():
            for o in self.engine.step():
                if o.finished:
                    done[o.request_id] = o
        return [done[i] for i in ids]

    def chat(self, messages_list, params=None, **kw) -> list[RequestOutput]:
        if self.tokenizer is None:
            raise ValueError("chat needs a tokenizer with a chat template")
        if messages_list and isinstance(messages_list[0], dict):
            messages_list = [messages_list]
        prompts = [
            self.tokenizer.apply_chat_template(m, tokenize=False, add_generation_prompt=True, **kw)
            for m in messages_list
        ]
        return self.generate(prompts, params)
