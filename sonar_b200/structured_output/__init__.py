"""Constrained decoding: grammars compiled per request, a packed token bitmask per step.

The engine core owns one ``StructuredOutputManager``.  A request that carries
``SamplingParams.structured_outputs`` gets a compiled grammar and a matcher when
it is added; after every ``schedule()`` the manager fills one row of a packed
``int32`` bitmask (bit ``t`` of word ``t // 32`` set = token ``t`` allowed) for
each structured request that will sample this step, the scheduler output carries
it to the workers, the worker masks the logits rows with it before sampling
(``ops.apply_token_bitmask``), and ``Scheduler.update_from_output`` advances the
matcher with the accepted tokens.

Two backends: ``xgrammar`` (JSON schema, regex, EBNF, choice, any-JSON) when the
package imports, and a built-in ``choice`` backend (a trie over the tokenised
alternatives) that needs nothing.

Parity: ``aphrodite/v1/structured_output/__init__.py`` (manager, ``grammar_bitmask``),
``backend_xgrammar.py``, and ``apply_grammar_bitmask`` used from
``v1/worker/gpu_model_runner.py:4246``.
"""
from __future__ import annotations

import json as _json
from typing import Any

import numpy as np

from sonar_b200.logger import init_logger
from sonar_b200.sampling_params import StructuredOutputsParams

logger = init_logger(__name__)

try:  # optional dependency
    import xgrammar as _xgr
except Exception:  # noqa: BLE001
    _xgr = None


def bitmask_words(vocab_size: int) -> int:
    return (vocab_size + 31) // 32


class Grammar:
    """Per-request matcher state."""

    def accept(self, token: int) -> bool:
        raise NotImplementedError

    def fill(self, row: np.ndarray) -> None:
        """Write the allowed-token bits of the next position into ``row`` (int32 words)."""
        raise NotImplementedError

    def terminated(self) -> bool:
        raise NotImplementedError


class XGrammar(Grammar):
    def __init__(self, compiled, vocab_size: int) -> None:
        self.matcher = _xgr.GrammarMatcher(compiled)
        self.vocab_size = vocab_size
        import torch
        self._buf = torch.zeros((1, bitmask_words(vocab_size)), dtype=torch.int32)

    def accept(self, token: int) -> bool:
        if self.matcher.is_terminated():
            return True
        return bool(self.matcher.accept_token(int(token)))

    def fill(self, row: np.ndarray) -> None:
        if self.matcher.is_terminated():
            row[:] = -1
            return
        self.matcher.fill_next_token_bitmask(self._buf, 0)
        row[:] = self._buf[0].numpy()

    def terminated(self) -> bool:
        return bool(self.matcher.is_terminated())


class ChoiceGrammar(Grammar):
    """One of a fixed list of token sequences, then end-of-sequence."""

    def __init__(self, alternatives: list[list[int]], eos: int | None, vocab_size: int) -> None:
        self.alts = [a for a in alternatives if a]
        self.eos = eos
        self.vocab_size = vocab_size
        self.prefix: list[int] = []
        self.done = False

    def _live(self) -> list[list[int]]:
        n = len(self.prefix)
        return [a for a in self.alts if a[:n] == self.prefix]

    def accept(self, token: int) -> bool:
        if self.done:
            return True
        n = len(self.prefix)
        live = self._live()
        if any(len(a) == n for a in live) and token == self.eos:
            self.done = True
            return True
        if not any(len(a) > n and a[n] == token for a in live):
            return False
        self.prefix.append(int(token))
        if self.eos is None and all(len(a) == n + 1 for a in self._live()):
            self.done = True
        return True

    def fill(self, row: np.ndarray) -> None:
        if self.done:
            row[:] = -1
            return
        row[:] = 0
        n = len(self.prefix)
        allowed = set()
        for a in self._live():
            if len(a) > n:
                allowed.add(a[n])
            elif self.eos is not None:
                allowed.add(self.eos)
        u = row.view(np.uint32)
        for t in allowed:
            u[t >> 5] |= np.uint32(1 << (t & 31))

    def terminated(self) -> bool:
        return self.done


class StructuredOutputManager:
    def __init__(self, tokenizer, vocab_size: int) -> None:
        self.tokenizer = tokenizer
        self.vocab_size = vocab_size
        self._compiler = None
        self._cache: dict[str, Any] = {}

    # -- backend -----------------------------------------------------------
    def _xgr_compiler(self):
        if self._compiler is None:
            tok = self.tokenizer
            if hasattr(tok, "get_vocab") and hasattr(tok, "backend_tokenizer"):
                info = _xgr.TokenizerInfo.from_huggingface(tok, vocab_size=self.vocab_size)
            else:
                pieces = tok.convert_ids_to_tokens(list(range(len(tok))), skip_special_tokens=False)
                pieces = [p if isinstance(p, str) else "" for p in pieces]
                pieces += [f"<unused{i}>" for i in range(len(pieces), self.vocab_size)]
                eos = getattr(tok, "eos_token_id", None)
                info = _xgr.TokenizerInfo(pieces, vocab_type=_xgr.VocabType.RAW, vocab_size=self.vocab_size,
                                          stop_token_ids=[eos] if eos is not None else None)
            self._compiler = _xgr.GrammarCompiler(info)
        return self._compiler

    def validate(self, p: StructuredOutputsParams) -> None:
        """Raise ``ValueError`` for a constraint no backend can serve (called by the frontend)."""
        if p.choice is not None:
            if not p.choice:
                raise ValueError("structured_outputs.choice is empty")
            return
        if _xgr is None:
            raise ValueError("json / regex / grammar constraints need the xgrammar package")

    def compile(self, p: StructuredOutputsParams, eos_token_id: int | None) -> Grammar:
        if p.choice is not None and (_xgr is None or self.tokenizer is None):
            alts = [self.tokenizer.encode(c, add_special_tokens=False) for c in p.choice]
            return ChoiceGrammar(alts, eos_token_id, self.vocab_size)
        if _xgr is None:
            raise ValueError("json / regex / grammar constraints need the xgrammar package")
        key = _json.dumps([p.json if not isinstance(p.json, dict) else _json.dumps(p.json, sort_keys=True),
                           p.regex, p.choice, p.grammar, p.json_object])
        compiled = self._cache.get(key)
        if compiled is None:
            c = self._xgr_compiler()
            try:
                if p.json is not None:
                    schema = p.json if isinstance(p.json, str) else _json.dumps(p.json)
                    compiled = c.compile_json_schema(schema)
                elif p.regex is not None:
                    compiled = c.compile_regex(p.regex)
                elif p.grammar is not None:
                    compiled = c.compile_grammar(p.grammar)
                elif p.choice is not None:
                    alts = " | ".join(_json.dumps(x) for x in p.choice)
                    compiled = c.compile_grammar(f"root ::= {alts}")
                else:
                    compiled = c.compile_builtin_json_grammar()
            except Exception as e:  # noqa: BLE001
                raise ValueError(f"invalid structured-output constraint: {e}") from e
            self._cache[key] = compiled
        return XGrammar(compiled, self.vocab_size)

    # -- per step ------------------------------------------------------------
    def bitmask(self, grammars: list[Grammar]) -> np.ndarray:
        out = np.empty((len(grammars), bitmask_words(self.vocab_size)), dtype=np.int32)
        for i, g in enumerate(grammars):
            g.fill(out[i])
        return out
