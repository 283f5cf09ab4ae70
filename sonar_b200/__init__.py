"""sonar_b200 — a Blackwell-native LLM inference engine.

Public surface: ``LLM`` (offline generation), ``SamplingParams``, the result
types, ``EngineArgs`` and the async engine used by the OpenAI-compatible
server (``python -m sonar_b200.entrypoints.cli serve``).
"""
from sonar_b200.version import __version__  # noqa: F401
from sonar_b200.sampling_params import (BeamSearchParams, PoolingParams, RequestOutputKind,  # noqa: F401
                                        SamplingParams, StructuredOutputsParams)
from sonar_b200.outputs import CompletionOutput, PoolingRequestOutput, RequestOutput  # noqa: F401
from sonar_b200.config import EngineArgs  # noqa: F401


def __getattr__(name: str):
    if name == "LLM":
        from sonar_b200.entrypoints.llm import LLM
        return LLM
    if name == "LLMEngine":
        from sonar_b200.engine.llm_engine import LLMEngine
        return LLMEngine
    if name == "AsyncLLM":
        from sonar_b200.engine.async_llm import AsyncLLM
        return AsyncLLM
    raise AttributeError(name)
