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


def test_more_tool_call_formats():
    import json

    from sonar_b200.entrypoints.parsers import get_tool_parser
    ds = ("Let me check.<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>get_weather\n```json\n"
          '{"city": "Paris"}\n```<｜tool▁call▁end｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>get_time\n```json\n{"tz": "CET"}\n```'
          "<｜tool▁call▁end｜><｜tool▁calls▁end｜>")
    r = get_tool_parser("deepseek_v3").extract(ds)
    assert r.content == "Let me check." and [(c.name, json.loads(c.arguments)) for c in r.tool_calls] == [
        ("get_weather", {"city": "Paris"}), ("get_time", {"tz": "CET"})]
    qc = ("I will call it.\n<tool_call>\n<function=search>\n<parameter=query>\nblackwell tcgen05\n</parameter>\n"
          "<parameter=limit>\n5\n</parameter>\n<parameter=exact>\ntrue\n</parameter>\n</function>\n</tool_call>")
    r = get_tool_parser("qwen3_coder").extract(qc)
    assert r.content.strip() == "I will call it." and r.tool_calls[0].name == "search"
    assert json.loads(r.tool_calls[0].arguments) == {"query": "blackwell tcgen05", "limit": 5, "exact": True}
    glm = "<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Beijing</arg_value>\n<arg_key>days</arg_key>\n<arg_value>3</arg_value>\n</tool_call>"
    r = get_tool_parser("glm45").extract(glm)
    assert r.content is None and json.loads(r.tool_calls[0].arguments) == {"city": "Beijing", "days": 3}
    r = get_tool_parser("granite").extract('<|tool_call|>[{"name": "f", "arguments": {"x": 1}}, {"name": "g", "arguments": {}}]')
    assert [c.name for c in r.tool_calls] == ["f", "g"]
    r = get_tool_parser("phi4_mini_json").extract('functools[{"name": "add", "arguments": {"a": 1, "b": 2}}]')
    assert r.tool_calls[0].name == "add" and json.loads(r.tool_calls[0].arguments) == {"a": 1, "b": 2}
    kimi = ("ok<|tool_calls_section_begin|><|tool_call_begin|>functions.get_weather:0<|tool_call_argument_begin|>"
            '{"city": "Oslo"}<|tool_call_end|><|tool_calls_section_end|>')
    r = get_tool_parser("kimi_k2").extract(kimi)
    assert r.content == "ok" and r.tool_calls[0].name == "get_weather" and r.tool_calls[0].id == "functions.get_weather:0"
    # streaming: text flows until a call opens, a half-written marker is held back, each call is emitted once
    p = get_tool_parser("qwen3_coder")
    sent, calls, prev = "", [], ""
    for ch in [qc[i:i + 7] for i in range(0, len(qc), 7)]:
        d, new = p.extract_streaming(prev, ch)
        prev += ch
        sent += d or ""
        calls += new
    assert sent.strip() == "I will call it." and len(calls) == 1 and "<tool" not in sent
    # an unfinished JSON list yields no call yet
    assert get_tool_parser("granite").extract('<|tool_call|>[{"name": "f", "argu').tool_calls == []


def test_more_reasoning_formats():
    from sonar_b200.entrypoints.parsers import get_reasoning_parser
    assert get_reasoning_parser("seed_oss").extract("<seed:think>plan</seed:think>answer") == ("plan", "answer")
    assert get_reasoning_parser("mistral").extract("[THINK]a[/THINK]b") == ("a", "b")
    assert get_reasoning_parser("glm45").extract("<think>x</think>y") == ("x", "y")
    assert get_reasoning_parser("hunyuan_a13b").extract("<think>r</think><answer>42</answer>") == ("r", "42")
