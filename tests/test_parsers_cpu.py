"""Tool-call and reasoning parsers: whole-text and streamed extraction."""
import json

import pytest

from sonar_b200.entrypoints.parsers import get_reasoning_parser, get_tool_parser


def _stream(parser, text, step=3):
    prev, r_acc, c_acc = "", "", ""
    for i in range(0, len(text), step):
        d = text[i:i + step]
        r, c = parser.extract_streaming(prev, d)
        r_acc += r or ""
        c_acc += c or ""
        prev += d
    return r_acc, c_acc


def test_reasoning_qwen3_and_deepseek():
    q = get_reasoning_parser("qwen3")
    assert q.extract("<think>plan it</think>answer") == ("plan it", "answer")
    assert q.extract("no markers") == (None, "no markers")
    assert q.extract("<think>unfinished") == ("unfinished", None)
    d = get_reasoning_parser("deepseek_r1")
    assert d.extract("thinking...</think>final") == ("thinking...", "final")
    assert d.extract("still thinking") == ("still thinking", None)
    for step in (1, 2, 5, 50):
        assert _stream(q, "<think>plan it</think>answer here", step) == ("plan it", "answer here")
        assert _stream(d, "abc def</think>the answer", step) == ("abc def", "the answer")
    with pytest.raises(ValueError):
        get_reasoning_parser("nope")


def test_tool_parsers():
    h = get_tool_parser("hermes")
    txt = 'Let me check.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>'
    out = h.extract(txt)
    assert out.content == "Let me check." and len(out.tool_calls) == 1
    assert out.tool_calls[0].name == "get_weather" and json.loads(out.tool_calls[0].arguments) == {"city": "Paris"}
    assert h.extract("plain text").tool_calls == []
    # streaming: text first, the call once complete, nothing of the raw markup leaks
    prev, content, calls = "", "", []
    for i in range(0, len(txt), 4):
        c, new = h.extract_streaming(prev, txt[i:i + 4])
        content += c or ""
        calls += new
        prev += txt[i:i + 4]
    assert len(calls) == 1 and "<tool" not in content and content.startswith("Let me check.")

    l3 = get_tool_parser("llama3_json")
    out = l3.extract('{"name": "f", "parameters": {"x": 1}}; {"name": "g", "parameters": {}}')
    assert [c.name for c in out.tool_calls] == ["f", "g"] and out.content is None
    assert l3.extract("hello").content == "hello"

    m = get_tool_parser("mistral")
    out = m.extract('[TOOL_CALLS] [{"name": "f", "arguments": {"a": "b"}}]')
    assert out.tool_calls[0].name == "f" and json.loads(out.tool_calls[0].arguments) == {"a": "b"}

    p = get_tool_parser("pythonic")
    out = p.extract('[get_weather(city="Paris", days=3), ping()]')
    assert [c.name for c in out.tool_calls] == ["get_weather", "ping"]
    assert json.loads(out.tool_calls[0].arguments) == {"city": "Paris", "days": 3}
    assert p.extract("[1, 2]").tool_calls == []
    assert out.tool_calls[0].to_openai()["type"] == "function"
