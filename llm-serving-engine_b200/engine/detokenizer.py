"""Text as it is generated: one :class:`TextStream` per sequence, and the search for stop strings.

Tokens do not map to characters one to one (a character may be spread over several byte tokens,
and many tokenizers print a token differently at the start of a text), so new text is never the
decoding of the new token alone. The stream decodes a short window of tokens twice, with and
without the tokens that arrived since the last text was shown, and shows the difference; while the
window ends inside a character nothing is shown. (What src/llmserve/detokenizer.py does with a
state object per sequence.)
"""

from __future__ import annotations

INCOMPLETE = "\N{REPLACEMENT CHARACTER}"  # what a decoder prints for a character that is cut short
CONTEXT_TOKENS = 5  # tokens before the first new one that are decoded along, for their spacing


class TextStream:
    def __init__(self, tokenizer, prompt_token_ids: list[int]) -> None:
        self._decode = lambda ids: tokenizer.decode(ids, skip_special_tokens=True)
        n = len(prompt_token_ids)
        self._window = max(0, n - CONTEXT_TOKENS)  # first token of the window
        self._shown = n  # tokens up to here have been turned into text

    def push(self, token_ids: list[int]) -> str:
        """``token_ids``: all of the sequence's tokens so far. Returns the text that is new."""
        window = token_ids[self._window :]
        old = self._decode(window[: self._shown - self._window])
        text = self._decode(window)
        if len(text) <= len(old) or text.endswith(INCOMPLETE):
            return ""  # the newest token has not completed a character yet
        self._window, self._shown = self._shown, len(token_ids)
        return text[len(old) :]


def find_stop(text: str, new_len: int, stops: list[str]) -> tuple[int, str] | None:
    """The stop string that begins first in ``text`` among those that reach into its last
    ``new_len`` characters (older text has been searched before): (where it begins, the string)."""
    found = None
    for stop in stops:
        if not stop:
            continue
        # a match may begin before the new text as long as it ends inside it
        at = text.find(stop, max(0, len(text) - new_len - len(stop) + 1))
        if at >= 0 and (found is None or at < found[0]):
            found = (at, stop)
    return found
