"""User-facing result objects (parity: ``aphrodite/outputs.py:22,83``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass
class Logprob:
    logprob: float
    rank: int | None = None
    decoded_token: str | None = None


@dataclass
class CompletionOutput:
    index: int
    text: str
    token_ids: list[int]
    cumulative_logprob: float | None = None
    logprobs: list[dict[int, Logprob]] | None = None
    finish_reason: str | None = None
    stop_reason: int | str | None = None

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None


@dataclass
class RequestMetrics:
    arrival_time: float = 0.0
    first_token_time: float | None = None
    finished_time: float | None = None
    num_cached_tokens: int = 0
    num_generation_tokens: int = 0


@dataclass
class RequestOutput:
    request_id: str
    prompt: str | None
    prompt_token_ids: list[int] | None
    outputs: list[CompletionOutput]
    finished: bool
    prompt_logprobs: list[dict[int, Logprob] | None] | None = None
    metrics: RequestMetrics | None = None
    num_cached_tokens: int = 0
    kv_transfer_params: dict[str, Any] | None = None

    def add(self, nxt: "RequestOutput", aggregate: bool) -> None:
        """Merge a later update into this one (used when a consumer is slower
        than the producer and several updates are pending)."""
        self.finished |= nxt.finished
        for comp in nxt.outputs:
            for mine in self.outputs:
                if mine.index == comp.index:
                    if aggregate:
                        mine.text += comp.text
                        mine.token_ids = list(mine.token_ids) + list(comp.token_ids)
                        if comp.logprobs:
                            mine.logprobs = (mine.logprobs or []) + comp.logprobs
                        mine.cumulative_logprob = comp.cumulative_logprob
                        mine.finish_reason = comp.finish_reason
                        mine.stop_reason = comp.stop_reason
                    else:
                        self.outputs[self.outputs.index(mine)] = comp
                    break
            else:
                self.outputs.append(comp)


@dataclass
class PoolingOutput:
    data: Any


@dataclass
class PoolingRequestOutput:
    request_id: str
    outputs: PoolingOutput
    prompt_token_ids: list[int]
    finished: bool = True


@dataclass
class BeamSearchSequence:
    tokens: list[int]
    cum_logprob: float = 0.0
    text: str | None = None
    finish_reason: str | None = None


@dataclass
class BeamSearchOutput:
    sequences: list[BeamSearchSequence] = field(default_factory=list)
