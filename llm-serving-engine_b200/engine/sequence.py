"""What the engine keeps per request while it runs, and what it hands back.

The public names (``Request``, ``Sequence``, ``RequestMetrics``, ``CompletionOutput``,
``RequestOutput`` and their fields) are the ones of src/llmserve/sequence.py, because they are the
entry point's output format (src/llmserve/sequence.py:126-145). A request here always has exactly
one sequence (parallel samples of one prompt are not built).
"""

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


class TokenLog:
    """A sequence's tokens: the prompt (fixed) and what has been generated (grows).

    Steps ask for runs of tokens ``start .. start+n-1``. A prompt is cut into portions many times,
    and a portion of a few thousand Python ints would be converted to an array on every step, so
    portions of the prompt come as slices of one int32 array that is made on first use.
    """

    SHORT = 16  # runs shorter than this are handed out as lists

    def __init__(self, prompt: list[int]) -> None:
        self.prompt = prompt
        self.generated: list[int] = []
        self._prompt_array: np.ndarray | None = None

    def __len__(self) -> int:
        return len(self.prompt) + len(self.generated)

    def everything(self) -> list[int]:
        return self.prompt + self.generated

    def run(self, start: int, n: int):
        p = len(self.prompt)
        end = start + n
        if start >= p:
            return self.generated[start - p : end - p]
        if end > p:
            return self.prompt[start:] + self.generated[: end - p]
        if n < self.SHORT:
            return self.prompt[start:end]
        if self._prompt_array is None:
            self._prompt_array = np.asarray(self.prompt, dtype=np.int32)
        return self._prompt_array[start:end]


@dataclass
class RequestMetrics:
    arrival_time: float
    first_scheduled_time: float | None = None
    first_token_time: float | None = None
    last_token_time: float | None = None
    finished_time: float | None = None
    token_times: list[float] = field(default_factory=list)

    def token_at(self, now: float) -> None:
        if self.first_token_time is None:
            self.first_token_time = now
        self.last_token_time = now
        self.token_times.append(now)


@dataclass
class Request:
    request_id: str
    prompt: str | None
    prompt_token_ids: list[int]
    params: SamplingParams
    arrival_time: float | None = None
    seqs: list["Sequence"] = field(default_factory=list)
    metrics: RequestMetrics = field(init=False)

    def __post_init__(self) -> None:
        self.metrics = RequestMetrics(self.arrival_time if self.arrival_time else time.monotonic())

    @property
    def is_finished(self) -> bool:
        return all(s.is_finished for s in self.seqs)


class Sequence:
    """One continuation of a request's prompt.

    ``num_computed_tokens`` counts the tokens whose keys and values are in the cache. A sampled
    token joins ``output_token_ids`` at once but is computed only in the *next* step, so a
    sequence that decodes always has exactly one token that is not computed yet
    (src/llmserve/sequence.py:23-26).
    """

    def __init__(self, seq_id: int, request: Request, prompt_token_ids: list[int], seed: int) -> None:
        self.seq_id = seq_id
        self.request = request
        self.index = 0  # among the request's sequences
        self.seed = seed  # keys the device generator for this sequence
        self.tokens = TokenLog(prompt_token_ids)
        self.status = SeqStatus.WAITING
        self.num_computed_tokens = 0
        self.num_preemptions = 0
        # results
        self.finish_reason: str | None = None
        self.stop_reason: str | int | None = None
        self.logprobs: list[float] = []
        self.top_logprobs: list[list[tuple[int, float]]] = []
        self.output_text = ""
        self.text_stream = None  # a detokenizer.TextStream when the engine has a tokenizer

    # the token lists under the names the rest of the engine and the outputs use
    @property
    def prompt_token_ids(self) -> list[int]:
        return self.tokens.prompt

    @property
    def output_token_ids(self) -> list[int]:
        return self.tokens.generated

    @property
    def params(self) -> SamplingParams:
        return self.request.params

    @property
    def num_tokens(self) -> int:
        return len(self.tokens)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.tokens.prompt)

    @property
    def is_finished(self) -> bool:
        return self.status is SeqStatus.FINISHED

    def token_ids(self) -> list[int]:
        return self.tokens.everything()

    def tokens_from(self, start: int, n: int):
        return self.tokens.run(start, n)

    def completion(self) -> "CompletionOutput":
        wants_logprobs = self.params.logprobs is not None
        return CompletionOutput(
            index=self.index, text=self.output_text, token_ids=list(self.output_token_ids),
            finish_reason=self.finish_reason, stop_reason=self.stop_reason,
            logprobs=list(self.logprobs) if wants_logprobs else None,
            top_logprobs=list(self.top_logprobs) if wants_logprobs else None,
        )

    def __repr__(self) -> str:
        return (f"Sequence(id={self.seq_id}, request={self.request.request_id!r}, {self.status.value}, "
                f"{self.num_computed_tokens}/{self.num_tokens} tokens computed)")


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

    @classmethod
    def of(cls, request: Request) -> "RequestOutput":
        """The request's state as an output object (a snapshot: lists are copied)."""
        return cls(request.request_id, request.prompt, request.prompt_token_ids,
                   [s.completion() for s in request.seqs], request.is_finished, 0, request.metrics)
