"""Token ids to text while they arrive, and stop strings.

The engine works on token ids.  A caller who has a tokenizer hands the engine a function
``token_bytes(token_id) -> bytes`` (for a byte-level BPE the text of a sequence is the
concatenation of its tokens' bytes); the engine then fills ``RequestOutput.text_delta`` and
honours ``SamplingParams.stop``.  Without such a function a request that sets ``stop`` is
refused when it is added.

The reference streams text the same way (src/minigpt_infer/tokenizer.py:49-97): a character
whose bytes are spread over several tokens is held back until it is whole; it decodes the whole
history at every token, here only the bytes not yet emitted are kept.  Stop strings follow
src/minigpt_infer/engine/engine.py:186-205: a request ends with reason "stop" once a stop
string appears in its text, and the text handed out ends where the stop string begins.
"""

from __future__ import annotations

from typing import Callable, Sequence


class IncrementalText:
    """Text of one request, token by token."""

    def __init__(self, token_bytes: Callable[[int], bytes]) -> None:
        self._token_bytes = token_bytes
        self._held = b""              # bytes of a character that is not whole yet (at most 3)
        self.text = ""                # everything emitted so far

    def add_token(self, token_id: int) -> str:
        """The text that this token completes (possibly empty)."""
        data = self._held + self._token_bytes(int(token_id))
        try:
            delta, self._held = data.decode("utf-8"), b""
        except UnicodeDecodeError as err:
            if err.end == len(data) and len(data) - err.start < 4 and err.reason.startswith("unexpected end"):
                # the tail is the beginning of a character: keep it for the next token
                delta, self._held = data[: err.start].decode("utf-8"), data[err.start:]
            else:
                delta, self._held = data.decode("utf-8", errors="replace"), b""
        self.text += delta
        return delta

    def finalize(self) -> str:
        """Bytes that never became a character, as replacement characters."""
        delta, self._held = self._held.decode("utf-8", errors="replace"), b""
        self.text += delta
        return delta


def cut_at_stop(text: str, delta: str, stops: Sequence[str]) -> tuple[str, str | None]:
    """``text`` ends with ``delta``.  If a stop string occurs in ``text``, return the part of
    ``delta`` that lies before the earliest occurrence, and that stop string; else
    ``(delta, None)``."""
    first, found = None, None
    for stop in stops:
        if not stop:
            continue
        at = text.find(stop)
        if at != -1 and (first is None or at < first):
            first, found = at, stop
    if found is None:
        return delta, None
    before_delta = len(text) - len(delta)
    return delta[: max(0, first - before_delta)], found
