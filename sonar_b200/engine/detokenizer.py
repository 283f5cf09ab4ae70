"""Incremental detokenisation with stop-string matching.

Text is produced by decoding a sliding window of token ids and emitting only
what extends the previously decoded text, holding back while the tail is an
incomplete UTF-8 sequence.  Stop strings are searched in the newly produced
region (plus an overlap of the longest stop string); the last
``max(len(stop)) - 1`` characters are withheld from streaming until they can no
longer become part of a stop string.

Parity: ``aphrodite/v1/engine/detokenizer.py`` (353 lines).
"""
from __future__ import annotations

from sonar_b200.sampling_params import SamplingParams

_WINDOW = 6  # tokens of left context re-decoded each time


class IncrementalDetokenizer:
    def __init__(self, tokenizer, prompt_token_ids: list[int], params: SamplingParams) -> None:
        self.tokenizer = tokenizer
        self.params = params
        self.enabled = tokenizer is not None and params.detokenize
        self.token_ids: list[int] = list(prompt_token_ids[-_WINDOW:]) if self.enabled else []
        self.prefix_offset = 0
        self.read_offset = len(self.token_ids)
        self.text = ""
        self.stops = list(params.stop or [])
        self.hold_back = max((len(s) for s in self.stops), default=1) - 1
        if params.include_stop_str_in_output:
            self.hold_back = 0
        self._streamed = 0

    def update(self, new_token_ids: list[int], finished_by_engine: bool) -> str | None:
        """Feed tokens; returns the stop string that matched, if any."""
        if not self.enabled:
            return None
        skip = self.params.skip_special_tokens
        for tok in new_token_ids:
            self.token_ids.append(tok)
            prefix = self.tokenizer.decode(self.token_ids[self.prefix_offset:self.read_offset],
                                           skip_special_tokens=skip)
            full = self.tokenizer.decode(self.token_ids[self.prefix_offset:], skip_special_tokens=skip)
            if len(full) > len(prefix) and not full.endswith("�"):
                delta = full[len(prefix):]
                self.prefix_offset = max(self.read_offset - _WINDOW, self.prefix_offset)
                self.read_offset = len(self.token_ids)
                before = len(self.text)
                self.text += delta
                if self.stops:
                    hit = self._find_stop(before)
                    if hit is not None:
                        return hit
        return None

    def _find_stop(self, before: int) -> str | None:
        for s in self.stops:
            start = max(0, before - len(s) + 1)
            pos = self.text.find(s, start)
            if pos != -1:
                end = pos + len(s) if self.params.include_stop_str_in_output else pos
                self.text = self.text[:end]
                return s
        return None

    def get_next_text(self, finished: bool, delta: bool) -> str:
        """Text for the next update; streaming withholds a possible stop-string prefix."""
        end = len(self.text) if finished else max(len(self.text) - self.hold_back, self._streamed)
        if delta:
            out = self.text[self._streamed:end]
            self._streamed = end
            return out
        return self.text[:end]
