"""Text of a request's growing output, piece by piece, and its stop strings.

``SamplingParams.stop`` ends a request when its text contains one of the strings
(``emberserve/tokenizer.py:88-190`` is the reference's incremental detokenizer; the engine
asks it after every token, ``emberserve/engine.py:1049-1057``).  Needs a tokenizer; without
one every piece is empty and stop strings never match.

Per request the state is: the text settled so far, how much of it has been handed out, and
two positions in the token list.  A step decodes only the tokens since the last settled one,
together with the few tokens before them (byte-level merges across the boundary then come
out as in a decode of the whole list), so its cost does not grow with the output.  A piece
that ends inside a multi-byte character (the tokenizer shows U+FFFD) is kept until the
character is complete.  Text that could still become a stop string, a trailing prefix of
one, is kept back too, so that a match never has to take back what was handed out; the stop
string itself is never part of the text.
"""

from __future__ import annotations

from dataclasses import dataclass

_INCOMPLETE = "�"


@dataclass
class _Progress:
    settled: str = ""   # all text decoded so far
    shown: int = 0      # characters of it handed out
    anchor: int = 0     # tokens [anchor, done) are decoded again as context of the next piece
    done: int = 0       # tokens whose text is in `settled`


def held_back(text: str, stop: list[str]) -> int:
    """How many trailing characters of `text` are the beginning (and not the whole) of a stop
    string."""
    most = 0
    for s in stop:
        for n in range(min(len(s) - 1, len(text)), most, -1):
            if text.endswith(s[:n]):
                most = n
                break
    return most


class Detokenizer:
    def __init__(self, tokenizer) -> None:
        self.tokenizer = tokenizer
        self._progress: dict[str, _Progress] = {}

    def drop(self, request_id: str) -> None:
        self._progress.pop(request_id, None)

    def text(self, request_id: str) -> str:
        """What has been handed out for the request so far."""
        st = self._progress.get(request_id)
        return "" if st is None else st.settled[:st.shown]

    def feed(self, request_id: str, output_ids: list[int], stop: list[str],
             final: bool = False) -> tuple[str, str | None]:
        """The new piece of text after `output_ids` (the request's whole output so far), and the
        stop string that the text has reached, if any.  `final` hands out what was kept back."""
        if self.tokenizer is None:
            return "", None
        st = self._progress.setdefault(request_id, _Progress())
        if len(output_ids) > st.done:
            context = self.tokenizer.decode(output_ids[st.anchor:st.done]) if st.done > st.anchor else ""
            both = self.tokenizer.decode(output_ids[st.anchor:])
            if both.endswith(_INCOMPLETE) and final:
                both = both[:-1]
            if len(both) > len(context) and not both.endswith(_INCOMPLETE):
                st.settled += both[len(context):]
                st.anchor, st.done = st.done, len(output_ids)
        visible, matched = st.settled, None
        if stop:
            where = -1
            for s in stop:  # a match can begin at most len(s) - 1 characters before what was handed out
                at = visible.find(s, max(0, st.shown - len(s) + 1))
                if at != -1 and (where == -1 or at < where):
                    where, matched = at, s
            if matched is not None:
                visible = visible[:where]
            elif not final:
                visible = visible[:len(visible) - held_back(visible, stop)]
        piece = visible[st.shown:] if len(visible) >= st.shown else ""
        st.shown = max(st.shown, len(visible))
        return piece, matched
