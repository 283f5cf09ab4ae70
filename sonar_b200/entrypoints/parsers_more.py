"""More tool-call and reasoning formats, registered into the tables of ``parsers.py`` on import.

Tool calls:

* ``deepseek_v3`` — ``<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>NAME`` + a fenced JSON block +
  ``<｜tool▁call▁end｜>`` … ``<｜tool▁calls▁end｜>``;
* ``qwen3_coder`` (alias ``qwen3_xml``) — ``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>…</function></tool_call>``;
* ``glm45`` — ``<tool_call>NAME`` followed by ``<arg_key>k</arg_key><arg_value>v</arg_value>`` pairs, ``</tool_call>``;
* ``granite`` — ``<|tool_call|>`` or ``<tool_call>`` followed by a JSON list of calls;
* ``phi4_mini_json`` — ``functools[{…}, …]``;
* ``kimi_k2`` — ``<|tool_calls_section_begin|><|tool_call_begin|>functions.NAME:IDX<|tool_call_argument_begin|>{json}<|tool_call_end|>…``.

Reasoning: ``glm45``, ``ernie45`` (``<think>``), ``seed_oss`` (``<seed:think>``), ``mistral`` (``[THINK]``),
``hunyuan_a13b`` (``<think>`` / ``<answer>`` wrappers).

Values of XML-style parameters are JSON-decoded when they parse (numbers, booleans, objects) and kept as strings
otherwise.  Text before the first call marker is the visible content; an unfinished call is withheld while
streaming (the generic ``extract_streaming`` re-parses the text so far).

Parity: ``aphrodite/tool_parsers/{deepseekv3,qwen3coder,glm4_moe,granite,phi4mini,kimi_k2}_tool_parser.py`` and
``aphrodite/reasoning/{glm4_moe,ernie45,seedoss,mistral,hunyuan_a13b}_reasoning_parser.py`` (formats only).
"""
from __future__ import annotations

import json
import re

from sonar_b200.entrypoints.parsers import (ExtractedTools, ReasoningParser, ToolCall, ToolParser, _call_from_obj,
                                            register_reasoning_parser, register_tool_parser)


def _value(text: str):
    t = text.strip()
    try:
        return json.loads(t)
    except (json.JSONDecodeError, ValueError):
        return t


def _split(text: str, marker: str) -> tuple[str | None, str]:
    """(content before the marker — also hiding a marker that is only half there —, rest from the marker on)."""
    i = text.find(marker)
    if i >= 0:
        return (text[:i] or None), text[i:]          # not stripped: streamed content must only ever grow
    for k in range(len(marker) - 1, 0, -1):
        if text.endswith(marker[:k]):
            return (text[:-k] or None), ""
    return (text or None), ""


class DeepSeekV3ToolParser(ToolParser):
    _call = re.compile(r"<｜tool▁call▁begin｜>(?P<type>.*?)<｜tool▁sep｜>(?P<name>.*?)\n```json\n(?P<args>.*?)\n```\s*<｜tool▁call▁end｜>", re.S)

    def extract(self, text: str) -> ExtractedTools:
        content, rest = _split(text, "<｜tool▁calls▁begin｜>")
        calls = [ToolCall(m.group("name").strip(), m.group("args").strip()) for m in self._call.finditer(rest)]
        return ExtractedTools(content, calls)


class Qwen3CoderToolParser(ToolParser):
    _block = re.compile(r"<tool_call>\s*(.*?)\s*</tool_call>", re.S)
    _fn = re.compile(r"<function=([^>\n]+)>(.*?)</function>", re.S)
    _param = re.compile(r"<parameter=([^>\n]+)>\n?(.*?)\n?</parameter>", re.S)

    def extract(self, text: str) -> ExtractedTools:
        content, rest = _split(text, "<tool_call>")
        calls = []
        for b in self._block.finditer(rest):
            for f in self._fn.finditer(b.group(1)):
                args = {k.strip(): _value(v) for k, v in self._param.findall(f.group(2))}
                calls.append(ToolCall(f.group(1).strip(), json.dumps(args, ensure_ascii=False)))
        return ExtractedTools(content, calls)


class Glm45ToolParser(ToolParser):
    _block = re.compile(r"<tool_call>\s*([^\n<]+)\s*(.*?)</tool_call>", re.S)
    _pair = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)

    def extract(self, text: str) -> ExtractedTools:
        content, rest = _split(text, "<tool_call>")
        calls = []
        for b in self._block.finditer(rest):
            args = {k.strip(): _value(v) for k, v in self._pair.findall(b.group(2))}
            calls.append(ToolCall(b.group(1).strip(), json.dumps(args, ensure_ascii=False)))
        return ExtractedTools(content, calls)


class _JsonListAfterMarker(ToolParser):
    markers: tuple[str, ...] = ()

    def extract(self, text: str) -> ExtractedTools:
        for mk in self.markers:
            if mk in text:
                content, rest = _split(text, mk)
                payload = rest[len(mk):].strip()
                try:
                    objs, _ = json.JSONDecoder().raw_decode(payload)
                except (json.JSONDecodeError, ValueError):
                    return ExtractedTools(content, [])            # the list is still being written
                objs = objs if isinstance(objs, list) else [objs]
                return ExtractedTools(content, [c for c in map(_call_from_obj, objs) if c])
        content, _ = _split(text, self.markers[0])
        return ExtractedTools(content, [])


class GraniteToolParser(_JsonListAfterMarker):
    markers = ("<|tool_call|>", "<tool_call>")


class Phi4MiniToolParser(_JsonListAfterMarker):
    markers = ("functools",)


class KimiK2ToolParser(ToolParser):
    _call = re.compile(r"<\|tool_call_begin\|>\s*(?P<id>[\w.\-]+:\d+)\s*<\|tool_call_argument_begin\|>\s*(?P<args>.*?)\s*<\|tool_call_end\|>", re.S)

    def extract(self, text: str) -> ExtractedTools:
        content, rest = _split(text, "<|tool_calls_section_begin|>")
        calls = []
        for m in self._call.finditer(rest):
            full = m.group("id")
            name = full.split(":")[0].split(".", 1)[-1]               # "functions.get_weather:0" → get_weather
            calls.append(ToolCall(name, m.group("args"), id=full))
        return ExtractedTools(content, calls)


class SeedOssReasoningParser(ReasoningParser):
    start, end = "<seed:think>", "</seed:think>"


class MistralReasoningParser(ReasoningParser):
    start, end = "[THINK]", "[/THINK]"


class Glm45ReasoningParser(ReasoningParser):
    """``<think>…</think>``; the template may already have opened the block."""


class HunyuanReasoningParser(ReasoningParser):
    """``<think>…</think><answer>…</answer>``: the answer wrapper is dropped from the visible content."""

    def extract(self, text: str):
        reasoning, content = super().extract(text)
        if content:
            content = content.replace("<answer>", "").replace("</answer>", "").strip() or None
        return reasoning, content


for _name, _cls in (("deepseek_v3", DeepSeekV3ToolParser), ("qwen3_coder", Qwen3CoderToolParser),
                    ("qwen3_xml", Qwen3CoderToolParser), ("glm45", Glm45ToolParser), ("granite", GraniteToolParser),
                    ("phi4_mini_json", Phi4MiniToolParser), ("kimi_k2", KimiK2ToolParser)):
    register_tool_parser(_name, _cls)
for _name, _cls in (("glm45", Glm45ReasoningParser), ("ernie45", Glm45ReasoningParser), ("seed_oss", SeedOssReasoningParser),
                    ("mistral", MistralReasoningParser), ("hunyuan_a13b", HunyuanReasoningParser)):
    register_reasoning_parser(_name, _cls)
