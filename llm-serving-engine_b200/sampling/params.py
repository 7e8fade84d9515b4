"""Sampling parameters of a request (names and meanings of src/llmserve/sampling.py:17-77).

Built: temperature, top_k, top_p, min_p, the three penalties, max_tokens, min_tokens,
stop_token_ids, stop strings, ignore_eos, seed, logprobs. Not built: ``n > 1`` (parallel samples
share prompt pages, which needs copy-on-write) and the ``guided_*`` options; both raise.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class SamplingParams:
    n: int = 1
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1  # -1 = disabled
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    max_tokens: int = 16
    min_tokens: int = 0
    stop: list[str] = field(default_factory=list)
    stop_token_ids: list[int] = field(default_factory=list)
    ignore_eos: bool = False
    seed: int | None = None
    logprobs: int | None = None  # number of top logprobs per token (0 = the sampled token only)
    include_stop_str_in_output: bool = False

    def __post_init__(self) -> None:
        if isinstance(self.stop, str):
            self.stop = [self.stop]
        # (what must hold, what to say if it does not); the ranges are the reference's
        # (src/llmserve/sampling.py:40-61), n > 1 is refused because it is not built
        rules = (
            (self.n == 1, "n must be 1: parallel samples of one prompt are not built"),
            (self.temperature >= 0, "temperature must be >= 0"),
            (0 < self.top_p <= 1, "top_p must be in (0, 1]"),
            (self.top_k == -1 or self.top_k >= 1, "top_k must be -1 (disabled) or >= 1"),
            (0 <= self.min_p <= 1, "min_p must be in [0, 1]"),
            (self.repetition_penalty > 0, "repetition_penalty must be > 0"),
            (self.max_tokens >= 1, "max_tokens must be >= 1"),
            (self.min_tokens >= 0, "min_tokens must be >= 0"),
            (self.logprobs is None or 0 <= self.logprobs <= 20, "logprobs must be between 0 and 20"),
        )
        for holds, message in rules:
            if not holds:
                raise ValueError(message)

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-5

    @property
    def has_cut(self) -> bool:
        """A sampled row whose candidates are cut by top-k, top-p or min-p (never a greedy row)."""
        return not self.greedy and (self.top_k > 0 or self.top_p < 1.0 or self.min_p > 0.0)

    @property
    def has_penalties(self) -> bool:
        return (self.presence_penalty != 0 or self.frequency_penalty != 0
                or self.repetition_penalty != 1.0)
