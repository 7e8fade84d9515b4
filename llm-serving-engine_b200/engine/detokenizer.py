"""Incremental detokenization and stop strings (behaviour of src/llmserve/detokenizer.py).

A character can span tokens, so a small window of tokens is decoded and only the new suffix is
emitted; text is held back while it ends in an incomplete UTF-8 sequence.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class DetokState:
    prefix_offset: int
    read_offset: int


class IncrementalDetokenizer:
    def __init__(self, tokenizer) -> None:
        self.tok = tokenizer

    def init_state(self, prompt_token_ids: list[int]) -> DetokState:
        n = len(prompt_token_ids)
        return DetokState(prefix_offset=max(0, n - 5), read_offset=n)

    def step(self, all_token_ids: list[int], state: DetokState) -> str:
        """The new text produced by the latest token(s)."""
        before = self.tok.decode(all_token_ids[state.prefix_offset : state.read_offset],
                                 skip_special_tokens=True)
        now = self.tok.decode(all_token_ids[state.prefix_offset :], skip_special_tokens=True)
        if len(now) > len(before) and not now.endswith("�"):
            state.prefix_offset = state.read_offset
            state.read_offset = len(all_token_ids)
            return now[len(before):]
        return ""


def find_stop(text: str, new_len: int, stops: list[str]) -> tuple[int, str] | None:
    """Earliest stop string that ends inside the last ``new_len`` characters: (start index, string)."""
    best = None
    for s in stops:
        if not s:
            continue
        i = text.find(s, max(0, len(text) - new_len - len(s) + 1))
        if i != -1 and (best is None or i < best[0]):
            best = (i, s)
    return best
