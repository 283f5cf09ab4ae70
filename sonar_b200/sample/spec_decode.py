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


class _SuffixTrie:
    """Counts of every token sequence of length ≤ depth that occurred in the inserted text: node = dict
    token → [count, children].  ``extend`` adds the sequences that END in the newly appended tokens, so a text
    can grow token by token."""

    def __init__(self, depth: int) -> None:
        self.depth = depth
        self.root: dict[int, list] = {}
        self.size = 0

    def extend(self, tokens, start: int) -> None:
        """Account for ``tokens[start:]`` having been appended to ``tokens[:start]``."""
        n, d = len(tokens), self.depth
        for end in range(start, n):
            # every sequence tokens[b..end], b ≥ end-d+1: walk from each b (their prefixes exist already)
            for b in range(max(0, end - d + 1), end + 1):
                node = self.root
                for t in tokens[b:end]:
                    node = node[int(t)][1]
                ent = node.get(int(tokens[end]))
                if ent is None:
                    node[int(tokens[end])] = [1, {}]
                    self.size += 1
                else:
                    ent[0] += 1

    def match(self, context) -> tuple[int, dict]:
        """Longest suffix of ``context`` (≤ depth-1 tokens, so a continuation can follow) present in the trie:
        (its length, the node reached)."""
        for n in range(min(self.depth - 1, len(context)), 0, -1):
            node, ok = self.root, True
            for t in context[len(context) - n:]:
                ent = node.get(int(t))
                if ent is None:
                    ok = False
                    break
                node = ent[1]
            if ok and node:
                return n, node
        return 0, {}


class SuffixProposer:
    """Suffix decoding: drafts come from token sequences seen before — in this request's own prompt and
    output, and in the outputs of recently finished requests.  The longest suffix of the context found in
    either trie is continued along the most frequent path; a draft stops where the path's estimated
    probability (product of count ratios) falls under ``min_token_prob``, so its length adapts to how
    predictable the text is (at most ``max_spec_factor`` × match length + 1, and at most k).

    Parity: ``aphrodite/v1/spec_decode/suffix_decoding.py`` (per-request and global suffix trees, frequency
    walk, ``suffix_decoding_max_tree_depth / max_cached_requests / max_spec_factor / min_token_prob``).
    """

    def __init__(self, cfg: SpeculativeConfig) -> None:
        self.k = cfg.num_speculative_tokens
        self.depth = cfg.suffix_decoding_max_tree_depth
        self.max_cached = cfg.suffix_decoding_max_cached_requests
        self.factor = cfg.suffix_decoding_max_spec_factor
        self.min_prob = cfg.suffix_decoding_min_token_prob
        self.local: dict[str, tuple[_SuffixTrie, int]] = {}      # request → (trie, tokens inserted)
        self.shared = _SuffixTrie(self.depth)
        self.cached: list[str] = []

    def _walk(self, node: dict, limit: int) -> tuple[list[int], float]:
        out, prob = [], 1.0
        while node and len(out) < limit:
            total = sum(e[0] for e in node.values())
            tok, ent = max(node.items(), key=lambda kv: kv[1][0])
            prob *= ent[0] / total
            if prob < self.min_prob:
                break
            out.append(tok)
            node = ent[1]
        return out, prob

    def propose(self, tokens: np.ndarray, req_id: str | None = None) -> list[int]:
        if self.k <= 0 or len(tokens) < 2:
            return []
        best: list[int] = []
        tries = [self.shared]
        if req_id is not None:
            trie, done = self.local.get(req_id) or (_SuffixTrie(self.depth), 0)
            # the last token is left out so that the context's own ending is not its match
            trie.extend(tokens[:len(tokens) - 1], done)
            self.local[req_id] = (trie, max(done, len(tokens) - 1))
            tries.insert(0, trie)
        score = 0.0
        for trie in tries:
            n, node = trie.match(tokens)
            if n == 0:
                continue
            limit = min(self.k, int(self.factor * n) + 1)
            draft, prob = self._walk(node, limit)
            if len(draft) * prob > score:
                best, score = draft, len(draft) * prob
        return best

    def finish(self, req_id: str, tokens: np.ndarray, num_prompt: int) -> None:
        """The request is over: its output joins the shared trie, its own trie is dropped."""
        self.local.pop(req_id, None)
        if self.max_cached <= 0 or len(tokens) <= num_prompt:
            return
        self.shared.extend([int(t) for t in tokens[num_prompt:]], 0)
        self.cached.append(req_id)
        if len(self.cached) > self.max_cached:
            # bounded memory: start over rather than tracking per-response counts for removal
            self.shared = _SuffixTrie(self.depth)
            self.cached = []
