"""Text of a request's generated tokens, grown token by token, and stop strings.

A tokenizer cannot decode one token at a time: a character may span several tokens, and what a
token decodes to may depend on its neighbours (a leading space, a merged byte pair).  So the
text is grown by decoding a short tail of the tokens twice, with and without the new ones, and
appending what the longer decoding adds; text that ends in an unfinished character (the
replacement character U+FFFD) is held back until it completes or the request ends.
12vivi/tandem does the same per step (python/tandem/engine/detokenizer.py:29-52), as does its
model for this, vLLM's incremental detokenizer.
"""

from __future__ import annotations

from typing import Any, Sequence

CONTEXT_TOKENS = 6  # settled tokens decoded again in front of the new ones, so that they join as in the whole text


class OutputText:
    def __init__(self, tokenizer: Any, skip_special_tokens: bool = True, stop: Sequence[str] = ()) -> None:
        self.tokenizer, self.skip_special = tokenizer, skip_special_tokens
        self.stop = tuple(stop)
        self.text = ""
        self.settled = 0  # generated tokens whose text is in ``text``
        self.emitted = 0  # characters of ``text`` already handed out as deltas
        self.stopped = False

    def _decode(self, tokens: Sequence[int]) -> str:
        return self.tokenizer.decode(list(tokens), skip_special_tokens=self.skip_special)

    def feed(self, generated: Sequence[int], final: bool) -> str:
        """``generated``: all known generated tokens so far.  Returns the text that is new since
        the last call; while stop strings are set, a tail that could be the start of one is kept
        back until it is decided.  Sets ``stopped`` when a stop string has appeared: the text ends
        in front of its first occurrence and grows no more."""
        if self.stopped:
            return ""
        if len(generated) > self.settled:
            anchor = max(0, self.settled - CONTEXT_TOKENS)
            before = self._decode(generated[anchor: self.settled])
            after = self._decode(generated[anchor:])
            if len(after) > len(before) and (final or not after.endswith("�")):
                self.text += after[len(before):]
                self.settled = len(generated)
        if self.stop:
            hits = [at for at in (self.text.find(s) for s in self.stop) if at >= 0]
            if hits:
                self.text, self.stopped = self.text[: min(hits)], True
        upto = len(self.text)
        if self.stop and not final and not self.stopped:
            # a tail that may be the beginning of a stop string is not handed out yet
            held = max((k for s in self.stop for k in range(1, len(s)) if self.text.endswith(s[:k])), default=0)
            upto = max(self.emitted, upto - held)
        delta = self.text[self.emitted: upto]
        self.emitted = max(self.emitted, upto) if not self.stopped else len(self.text)
        return delta
