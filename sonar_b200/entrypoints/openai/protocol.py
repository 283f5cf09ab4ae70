"""Request / response schemas of the OpenAI-compatible API (pydantic v2).

The sampling fields a request may carry are the OpenAI ones plus the engine's
extended sampler family, mapped one-to-one onto ``SamplingParams``.
Parity: ``aphrodite/entrypoints/openai/chat_completion/protocol.py`` and
``completion/protocol.py``.
"""
from __future__ import annotations

import time
import uuid
from typing import Any, Literal

from pydantic import BaseModel, ConfigDict, Field

from sonar_b200.sampling_params import RequestOutputKind, SamplingParams


def _id(prefix: str) -> str:
    return f"{prefix}-{uuid.uuid4().hex}"


class _Base(BaseModel):
    model_config = ConfigDict(extra="allow")


class SamplingFields(_Base):
    n: int = 1
    max_tokens: int | None = None
    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    min_p: float | None = None
    presence_penalty: float | None = None
    frequency_penalty: float | None = None
    repetition_penalty: float | None = None
    seed: int | None = None
    stop: str | list[str] | None = None
    stop_token_ids: list[int] | None = None
    ignore_eos: bool = False
    min_tokens: int = 0
    skip_special_tokens: bool = True
    include_stop_str_in_output: bool = False
    logit_bias: dict[str, float] | None = None
    allowed_token_ids: list[int] | None = None
    bad_words: list[str] | None = None
    priority: int = 0
    # extended samplers
    top_a: float | None = None
    tfs: float | None = None
    eta_cutoff: float | None = None
    epsilon_cutoff: float | None = None
    typical_p: float | None = None
    smoothing_factor: float | None = None
    smoothing_curve: float | None = None
    xtc_threshold: float | None = None
    xtc_probability: float | None = None
    nsigma: float | None = None
    mirostat_mode: int | None = None
    mirostat_tau: float | None = None
    mirostat_eta: float | None = None
    dry_multiplier: float | None = None
    dry_base: float | None = None
    dry_allowed_length: int | None = None
    dry_sequence_breaker_ids: list[int] | None = None
    dynatemp_min: float | None = None
    dynatemp_max: float | None = None
    dynatemp_exponent: float | None = None
    temperature_last: bool | None = None
    skew: float | None = None
    no_repeat_ngram_size: int | None = None
    # constrained decoding
    response_format: dict[str, Any] | None = None
    structured_outputs: dict[str, Any] | None = None
    guided_json: str | dict[str, Any] | None = None
    guided_regex: str | None = None
    guided_choice: list[str] | None = None
    guided_grammar: str | None = None

    def structured_params(self):
        """``response_format`` / ``structured_outputs`` / legacy ``guided_*`` fields → StructuredOutputsParams."""
        from sonar_b200.sampling_params import StructuredOutputsParams
        if self.structured_outputs:
            return StructuredOutputsParams(**self.structured_outputs)
        if self.guided_json is not None:
            return StructuredOutputsParams(json=self.guided_json)
        if self.guided_regex is not None:
            return StructuredOutputsParams(regex=self.guided_regex)
        if self.guided_choice is not None:
            return StructuredOutputsParams(choice=self.guided_choice)
        if self.guided_grammar is not None:
            return StructuredOutputsParams(grammar=self.guided_grammar)
        rf = self.response_format
        if rf:
            kind = rf.get("type")
            if kind == "json_object":
                return StructuredOutputsParams(json_object=True)
            if kind == "json_schema":
                js = rf.get("json_schema") or {}
                return StructuredOutputsParams(json=js.get("schema", js))
        return None

    _PASS = ("top_p", "top_k", "min_p", "presence_penalty", "frequency_penalty", "repetition_penalty", "seed",
             "stop_token_ids", "allowed_token_ids", "bad_words", "top_a", "tfs", "eta_cutoff", "epsilon_cutoff",
             "typical_p", "smoothing_factor", "smoothing_curve", "xtc_threshold", "xtc_probability", "nsigma",
             "mirostat_mode", "mirostat_tau", "mirostat_eta", "dry_multiplier", "dry_base", "dry_allowed_length",
             "dry_sequence_breaker_ids", "dynatemp_min", "dynatemp_max", "dynatemp_exponent", "temperature_last",
             "skew", "no_repeat_ngram_size")

    def to_sampling_params(self, default_max_tokens: int | None, logprobs: int | None, stream: bool,
                           default_temperature: float = 1.0) -> SamplingParams:
        kw: dict[str, Any] = {k: getattr(self, k) for k in self._PASS if getattr(self, k) is not None}
        if self.logit_bias:
            kw["logit_bias"] = {int(k): float(v) for k, v in self.logit_bias.items()}
        so = self.structured_params()
        if so is not None:
            kw["structured_outputs"] = so
        return SamplingParams(
            n=self.n, max_tokens=self.max_tokens if self.max_tokens is not None else default_max_tokens,
            temperature=self.temperature if self.temperature is not None else default_temperature,
            stop=self.stop, ignore_eos=self.ignore_eos, min_tokens=self.min_tokens,
            skip_special_tokens=self.skip_special_tokens,
            include_stop_str_in_output=self.include_stop_str_in_output, logprobs=logprobs,
            output_kind=RequestOutputKind.DELTA if stream else RequestOutputKind.FINAL_ONLY, **kw)


class StreamOptions(_Base):
    include_usage: bool = False


class CompletionRequest(SamplingFields):
    model: str | None = None
    prompt: str | list[str] | list[int] | list[list[int]]
    stream: bool = False
    stream_options: StreamOptions | None = None
    logprobs: int | None = None
    echo: bool = False
    suffix: str | None = None


class ChatMessage(_Base):
    role: str
    content: str | list[dict[str, Any]] | None = None
    name: str | None = None
    tool_calls: list[dict[str, Any]] | None = None
    tool_call_id: str | None = None


class ChatCompletionRequest(SamplingFields):
    model: str | None = None
    messages: list[ChatMessage]
    stream: bool = False
    stream_options: StreamOptions | None = None
    logprobs: bool = False
    top_logprobs: int | None = None
    max_completion_tokens: int | None = None
    tools: list[dict[str, Any]] | None = None
    tool_choice: str | dict[str, Any] | None = None
    chat_template: str | None = None
    add_generation_prompt: bool = True


class UsageInfo(_Base):
    prompt_tokens: int = 0
    completion_tokens: int = 0
    total_tokens: int = 0
    prompt_tokens_details: dict[str, int] | None = None


class CompletionLogprobs(_Base):
    text_offset: list[int] = Field(default_factory=list)
    token_logprobs: list[float | None] = Field(default_factory=list)
    tokens: list[str] = Field(default_factory=list)
    top_logprobs: list[dict[str, float] | None] = Field(default_factory=list)


class CompletionChoice(_Base):
    index: int
    text: str
    logprobs: CompletionLogprobs | None = None
    finish_reason: str | None = None
    stop_reason: int | str | None = None


class CompletionResponse(_Base):
    id: str = Field(default_factory=lambda: _id("cmpl"))
    object: str = "text_completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str
    choices: list[CompletionChoice]
    usage: UsageInfo | None = None


class ChatLogprobEntry(_Base):
    token: str
    logprob: float
    bytes: list[int] | None = None
    top_logprobs: list[dict[str, Any]] = Field(default_factory=list)


class ChatLogprobs(_Base):
    content: list[ChatLogprobEntry] = Field(default_factory=list)


class ChatResponseMessage(_Base):
    role: str = "assistant"
    content: str | None = None
    reasoning_content: str | None = None
    tool_calls: list[dict[str, Any]] | None = None


class ChatChoice(_Base):
    index: int
    message: ChatResponseMessage
    logprobs: ChatLogprobs | None = None
    finish_reason: str | None = None
    stop_reason: int | str | None = None


class ChatCompletionResponse(_Base):
    id: str = Field(default_factory=lambda: _id("chatcmpl"))
    object: str = "chat.completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str
    choices: list[ChatChoice]
    usage: UsageInfo | None = None


class TokenizeRequest(_Base):
    model: str | None = None
    prompt: str | None = None
    messages: list[ChatMessage] | None = None
    add_special_tokens: bool = True
    add_generation_prompt: bool = True


class DetokenizeRequest(_Base):
    model: str | None = None
    tokens: list[int]


class EmbeddingRequest(_Base):
    model: str | None = None
    input: str | list[str] | list[int] | list[list[int]]
    encoding_format: Literal["float", "base64"] = "float"
    dimensions: int | None = None


class ErrorResponse(_Base):
    object: str = "error"
    message: str
    type: str
    param: str | None = None
    code: int
