"""Request and sequence state (src/llmserve/sequence.py)."""

from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field

import numpy as np

from ..sampling.params import SamplingParams


class SeqStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class Sequence:
    """One generated continuation.

    ``num_computed_tokens`` counts tokens whose keys and values are in the cache. A sampled token
    is appended to ``output_token_ids`` and computed in the *next* step, so a decoding sequence
    always has exactly one token that is not computed yet (src/llmserve/sequence.py:23-26).
    """

    def __init__(self, seq_id: int, request: "Request", prompt_token_ids: list[int], seed: int) -> None:
        self.seq_id = seq_id
        self.request = request
        self.index = 0
        self.prompt_token_ids = prompt_token_ids
        self.output_token_ids: list[int] = []
        self.status = SeqStatus.WAITING
        self.num_computed_tokens = 0
        self.num_preemptions = 0
        self.finish_reason: str | None = None
        self.stop_reason: str | int | None = None
        self.logprobs: list[float] = []
        self.top_logprobs: list[list[tuple[int, float]]] = []
        self.output_text = ""
        self.detok_state = None
        self.seed = seed  # keys the device generator for this sequence
        self._prompt_array = None

    @property
    def params(self) -> SamplingParams:
        return self.request.params

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    def token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    def tokens_from(self, start: int, n: int):
        """Tokens ``start .. start+n-1``. A portion of the prompt comes as a slice of one int32
        array made once per sequence (a prompt is cut into portions many times; a list of a
        few thousand Python ints would be converted each time)."""
        p = len(self.prompt_token_ids)
        if start + n <= p:
            if n < 16:
                return self.prompt_token_ids[start : start + n]
            if self._prompt_array is None:
                self._prompt_array = np.asarray(self.prompt_token_ids, dtype=np.int32)
            return self._prompt_array[start : start + n]
        if start >= p:
            return self.output_token_ids[start - p : start - p + n]
        return self.prompt_token_ids[start:] + self.output_token_ids[: start + n - p]

    @property
    def is_finished(self) -> bool:
        return self.status == SeqStatus.FINISHED

    def __repr__(self) -> str:
        return (f"Seq({self.seq_id}, req={self.request.request_id}, {self.status.value}, "
                f"tok={self.num_tokens}, computed={self.num_computed_tokens})")


@dataclass
class RequestMetrics:
    arrival_time: float
    first_scheduled_time: float | None = None
    first_token_time: float | None = None
    last_token_time: float | None = None
    finished_time: float | None = None
    token_times: list[float] = field(default_factory=list)


class Request:
    def __init__(self, request_id: str, prompt: str | None, prompt_token_ids: list[int],
                 params: SamplingParams, arrival_time: float | None = None) -> None:
        self.request_id = request_id
        self.prompt = prompt
        self.prompt_token_ids = prompt_token_ids
        self.params = params
        self.seqs: list[Sequence] = []
        self.metrics = RequestMetrics(arrival_time or time.monotonic())

    @property
    def is_finished(self) -> bool:
        return all(s.is_finished for s in self.seqs)


@dataclass
class CompletionOutput:
    index: int
    text: str
    token_ids: list[int]
    finish_reason: str | None
    stop_reason: str | int | None = None
    logprobs: list[float] | None = None
    top_logprobs: list[list[tuple[int, float]]] | None = None


@dataclass
class RequestOutput:
    request_id: str
    prompt: str | None
    prompt_token_ids: list[int]
    outputs: list[CompletionOutput]
    finished: bool
    num_cached_tokens: int = 0
    metrics: RequestMetrics | None = None
