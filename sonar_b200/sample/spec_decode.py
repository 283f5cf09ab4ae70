"""Speculative decoding: n-gram (prompt-lookup) proposer.

Draft tokens are the continuation of the most recent earlier occurrence of the
sequence's last ``n`` tokens (longest ``n`` first, ``prompt_lookup_max`` down to
``prompt_lookup_min``).  The scheduler schedules the drafts as extra positions of
the next step; the runner verifies them greedily (keeps sampled tokens while they
agree with the drafts) and the scheduler rolls back the KV positions of rejected
drafts.  Matching is vectorised with numpy sliding windows.

Parity: ``aphrodite/v1/spec_decode/ngram_proposer.py`` (the reference also ships
EAGLE/Medusa/MTP draft-model proposers; those need trained draft heads).
"""
from __future__ import annotations

import numpy as np

from sonar_b200.config import SpeculativeConfig


class NgramProposer:
    def __init__(self, cfg: SpeculativeConfig) -> None:
        self.k = cfg.num_speculative_tokens
        self.max_n = cfg.prompt_lookup_max
        self.min_n = max(1, cfg.prompt_lookup_min)

    def propose(self, tokens: np.ndarray) -> list[int]:
        """``tokens``: every known token of the sequence (prompt + generated)."""
        n_tok = len(tokens)
        if self.k <= 0 or n_tok < self.min_n + 1:
            return []
        for n in range(min(self.max_n, n_tok - 1), self.min_n - 1, -1):
            tail = tokens[n_tok - n:]
            # windows of length n that end before the tail itself starts being its own match
            windows = np.lib.stride_tricks.sliding_window_view(tokens[: n_tok - 1], n)
            hits = np.nonzero((windows == tail).all(axis=1))[0]
            if len(hits) == 0:
                continue
            start = int(hits[-1]) + n           # most recent match; its continuation is the draft
            draft = tokens[start:start + self.k]
            if len(draft):
                return [int(t) for t in draft]
        return []
