"""Per-request decoding controls.

The field set mirrors the public surface of ``aphrodite/sampling_params.py:235-432``
(OpenAI-style penalties, temperature/top-p/top-k/min-p, stops, logprobs) plus the
extended sampler family the reference adds on top of it (dynamic temperature,
top-a, tail-free, eta/epsilon cutoffs, typical-p, quadratic smoothing, XTC,
top-n-sigma, mirostat, DRY, skew, no-repeat-ngram).  Validation happens once in
``__post_init__``; the sampler reads plain attributes afterwards.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from enum import IntEnum
from typing import Any

_SAMPLING_EPS = 1e-5
_MAX_TEMP = 1e-2


class SamplingType(IntEnum):
    GREEDY = 0
    RANDOM = 1
    RANDOM_SEED = 2


class RequestOutputKind(IntEnum):
    CUMULATIVE = 0  # every update carries the whole output so far
    DELTA = 1       # every update carries only the new part
    FINAL_ONLY = 2  # a single update when the request finishes


@dataclass
class StructuredOutputsParams:
    """Constrained-decoding request: exactly one of the fields is set."""
    json: str | dict | None = None
    regex: str | None = None
    choice: list[str] | None = None
    grammar: str | None = None
    json_object: bool | None = None

    def __post_init__(self) -> None:
        count = sum(x is not None and x is not False for x in
                    (self.json, self.regex, self.choice, self.grammar, self.json_object))
        if count > 1:
            raise ValueError("only one structured-output constraint may be given")


@dataclass
class SamplingParams:
    n: int = 1
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    seed: int | None = None
    stop: str | list[str] | None = None
    stop_token_ids: list[int] | None = None
    ignore_eos: bool = False
    max_tokens: int | None = 16
    min_tokens: int = 0
    logprobs: int | None = None
    prompt_logprobs: int | None = None
    detokenize: bool = True
    skip_special_tokens: bool = True
    spaces_between_special_tokens: bool = True
    include_stop_str_in_output: bool = False
    output_kind: RequestOutputKind = RequestOutputKind.CUMULATIVE
    logit_bias: dict[int, float] | None = None
    allowed_token_ids: list[int] | None = None
    bad_words: list[str] | None = None
    structured_outputs: StructuredOutputsParams | None = None
    extra_args: dict[str, Any] | None = None
    # ---- extended sampler family ----
    no_repeat_ngram_size: int = 0
    dynatemp_min: float = 0.0
    dynatemp_max: float = 0.0
    dynatemp_exponent: float = 1.0
    temperature_last: bool = False
    top_a: float = 0.0
    tfs: float = 1.0
    eta_cutoff: float = 0.0
    epsilon_cutoff: float = 0.0
    typical_p: float = 1.0
    smoothing_factor: float = 0.0
    smoothing_curve: float = 1.0
    xtc_threshold: float = 0.1
    xtc_probability: float = 0.0
    nsigma: float = 0.0
    mirostat_mode: int = 0
    mirostat_tau: float = 0.0
    mirostat_eta: float = 0.0
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_sequence_breaker_ids: list[int] = field(default_factory=list)
    dry_range: int = 0
    skew: float = 0.0
    # filled by the engine from the model's generation config
    _eos_token_id: int | None = None
    _all_stop_token_ids: set[int] = field(default_factory=set)
    _bad_words_token_ids: list[list[int]] | None = None

    def __post_init__(self) -> None:
        if 0 < self.temperature < _MAX_TEMP:
            self.temperature = _MAX_TEMP
        if self.top_k is None or self.top_k < 0:
            self.top_k = 0
        if self.stop is None:
            self.stop = []
        elif isinstance(self.stop, str):
            self.stop = [self.stop]
        else:
            self.stop = list(self.stop)
        self.stop_token_ids = list(self.stop_token_ids or [])
        if self.logprobs is True:  # OpenAI-style boolean
            self.logprobs = 1
        self._verify()
        if self.temperature < _SAMPLING_EPS:
            # greedy: the truncation samplers cannot change the arg-max
            self.top_p, self.top_k, self.min_p = 1.0, 0, 0.0
        self._all_stop_token_ids = set(self.stop_token_ids)

    def _verify(self) -> None:
        if not isinstance(self.n, int) or self.n < 1:
            raise ValueError(f"n must be a positive integer, got {self.n}")
        for name, lo, hi in (("presence_penalty", -2.0, 2.0), ("frequency_penalty", -2.0, 2.0)):
            v = getattr(self, name)
            if not lo <= v <= hi:
                raise ValueError(f"{name} must be in [{lo}, {hi}], got {v}")
        if self.repetition_penalty <= 0.0:
            raise ValueError(f"repetition_penalty must be > 0, got {self.repetition_penalty}")
        if self.temperature < 0.0:
            raise ValueError(f"temperature must be non-negative, got {self.temperature}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if self.top_a < 0.0 or self.top_a > 1.0:
            raise ValueError(f"top_a must be in [0, 1], got {self.top_a}")
        if not 0.0 < self.tfs <= 1.0:
            raise ValueError(f"tfs must be in (0, 1], got {self.tfs}")
        if not 0.0 < self.typical_p <= 1.0:
            raise ValueError(f"typical_p must be in (0, 1], got {self.typical_p}")
        if self.eta_cutoff < 0 or self.epsilon_cutoff < 0:
            raise ValueError("eta_cutoff and epsilon_cutoff must be non-negative")
        if self.max_tokens is not None and self.max_tokens < 1:
            raise ValueError(f"max_tokens must be at least 1, got {self.max_tokens}")
        if self.min_tokens < 0:
            raise ValueError(f"min_tokens must be non-negative, got {self.min_tokens}")
        if self.max_tokens is not None and self.min_tokens > self.max_tokens:
            raise ValueError("min_tokens must not exceed max_tokens")
        if self.logprobs is not None and self.logprobs < -1:
            raise ValueError(f"logprobs must be >= -1, got {self.logprobs}")
        if self.prompt_logprobs is not None and self.prompt_logprobs < -1:
            raise ValueError(f"prompt_logprobs must be >= -1, got {self.prompt_logprobs}")
        if self.mirostat_mode not in (0, 2):
            raise ValueError("only mirostat mode 2 is implemented")
        if self.dynatemp_min < 0 or self.dynatemp_max < 0 or self.dynatemp_min > self.dynatemp_max:
            raise ValueError("dynatemp range must satisfy 0 <= min <= max")
        if self.stop and not self.detokenize:
            raise ValueError("stop strings need detokenize=True")
        if self.xtc_probability < 0 or self.xtc_probability > 1:
            raise ValueError("xtc_probability must be in [0, 1]")

    # ------------------------------------------------------------------
    @property
    def sampling_type(self) -> SamplingType:
        if self.temperature < _SAMPLING_EPS:
            return SamplingType.GREEDY
        if self.seed is not None:
            return SamplingType.RANDOM_SEED
        return SamplingType.RANDOM

    @property
    def all_stop_token_ids(self) -> set[int]:
        return self._all_stop_token_ids

    @property
    def needs_penalties(self) -> bool:
        return (self.presence_penalty != 0.0 or self.frequency_penalty != 0.0
                or self.repetition_penalty != 1.0)

    @property
    def needs_extended(self) -> bool:
        """True when any sampler beyond temperature/top-k/top-p/min-p is active."""
        return (self.top_a > 0 or self.tfs < 1.0 or self.eta_cutoff > 0 or self.epsilon_cutoff > 0
                or self.typical_p < 1.0 or self.smoothing_factor > 0 or self.xtc_probability > 0
                or self.nsigma > 0 or self.mirostat_mode != 0 or self.dry_multiplier > 0
                or self.skew != 0 or self.no_repeat_ngram_size > 0
                or self.dynatemp_max > 0 or self.temperature_last)

    def update_from_generation_config(self, eos_token_id: int | list[int] | None) -> None:
        """Attach the model's EOS ids: the first is *the* EOS (masked until
        ``min_tokens``), the others become extra stop tokens."""
        if eos_token_id is None:
            return
        ids = [eos_token_id] if isinstance(eos_token_id, int) else list(eos_token_id)
        if not ids:
            return
        self._eos_token_id = ids[0]
        if not self.ignore_eos:
            for t in ids:
                self._all_stop_token_ids.add(t)
                if t != ids[0] and t not in self.stop_token_ids:
                    self.stop_token_ids.append(t)

    def clone(self) -> "SamplingParams":
        return copy.deepcopy(self)


@dataclass
class BeamSearchParams:
    beam_width: int
    max_tokens: int
    ignore_eos: bool = False
    temperature: float = 0.0
    length_penalty: float = 1.0
    include_stop_str_in_output: bool = False


@dataclass
class PoolingParams:
    """Controls for embedding / classification requests."""
    task: str = "embed"
    normalize: bool = True
    dimensions: int | None = None
    truncate_prompt_tokens: int | None = None
