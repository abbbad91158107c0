"""Protocol normalisation, chat template and streaming tool-call / reasoning parser."""
import json

import pytest

from titanic_flash_41_b200.api import protocol as P


def tool_request():
    return {"max_tokens": 128, "messages": [
        {"role": "user", "content": "Read both files. Literal <think> and </think>."},
        {"role": "assistant", "content": "", "reasoning_content": "Read each file independently.",
         "tool_calls": [
             {"id": "call_a", "type": "function", "function": {"name": "read", "arguments": "{\"path\":\"a.rs\"}"}},
             {"id": "call_b", "type": "function", "function": {"name": "read", "arguments": "{\"path\":\"b.rs\"}"}}]},
        {"role": "tool", "tool_call_id": "call_a", "content": "fn a() {}"},
        {"role": "tool", "tool_call_id": "call_b", "content": "fn b() {}"}],
        "tools": [{"type": "function", "function": {"name": "read", "parameters": {
            "type": "object", "properties": {"path": {"type": "string"}}, "required": ["path"]}}}]}


def test_unknown_and_unsupported_fields_are_rejected():
    with pytest.raises(P.ProtocolError, match="unsupported native chat field: foo"):
        P.normalize_chat_request({"messages": [{"role": "user", "content": "x"}], "foo": 1})
    base = {"messages": [{"role": "user", "content": "x"}]}
    for bad in ({"presence_penalty": 0.5}, {"logprobs": True}, {"n": 2}, {"stop": ["a"]}, {"top_k": 5},
                {"response_format": {"type": "json_object"}}, {"tool_choice": "required"},
                {"max_tokens": 1, "max_completion_tokens": 1}, {"thinking": {"budget_tokens": 5}},
                {"tools": [{"type": "function", "function": {"name": "f", "strict": True}}]}):
        with pytest.raises(P.ProtocolError):
            P.normalize_chat_request({**base, **bad})
    r = P.normalize_chat_request(base)
    assert (r.temperature, r.top_p, r.reasoning_effort, r.model) == (1.0, 1.0, "high", P.DEFAULT_MODEL)
    with pytest.raises(P.ProtocolError):
        P.normalize_chat_request({**base, "temperature": 0.6}, allow_sampling=False)
    assert P.normalize_chat_request({**base, "temperature": 0.6, "top_p": 0.95}).top_p == 0.95


def test_max_tokens_resolution():
    assert P.resolve_max_tokens(None, 100, 1000) == 900
    assert P.resolve_max_tokens(50, 100, 1000) == 50
    assert P.resolve_max_tokens(None, 100, 10 ** 7) == P.DEFAULT_MAX_NEW_TOKENS
    with pytest.raises(P.ProtocolError) as e:
        P.resolve_max_tokens(5, 1000, 1000)
    assert e.value.code == "context_length_exceeded"


def test_tool_order_effort_and_adjacent_users():
    req = tool_request()
    texts = {}
    for effort, score in (("high", 75), ("max", 100)):
        req["reasoning_effort"] = effort
        t = P.render_chat(P.normalize_chat_request(req))
        assert f"Reasoning Effort: {score} (range 1-100" in t
        assert "Read each file independently." in t
        rev = json.loads(json.dumps(req))
        rev["messages"][2], rev["messages"][3] = rev["messages"][3], rev["messages"][2]
        assert P.render_chat(P.normalize_chat_request(rev)) == t     # arrival order normalises to call order
        texts[effort] = t
    assert texts["high"] != texts["max"]
    sep = {"messages": [{"role": "user", "content": "First 😀"}, {"role": "user", "content": "Second 中文"}]}
    mer = {"messages": [{"role": "user", "content": "First 😀\n\nSecond 中文"}]}
    assert P.render_chat(P.normalize_chat_request(sep)) == P.render_chat(P.normalize_chat_request(mer))


def test_assistant_prefix_continuation():
    for content, reasoning, suffix in (("Draft answer: ", "Prepared reasoning.", "Draft answer: "),
                                       ("", "Continue reasoning here", "Continue reasoning here")):
        req = {"messages": [{"role": "user", "content": "Continue."},
                            {"role": "assistant", "content": content, "reasoning_content": reasoning, "prefix": True}]}
        assert P.render_chat(P.normalize_chat_request(req)).endswith(suffix)


@pytest.mark.parametrize("width", [1, 3, 17, 256])
def test_parallel_tool_stream_preserves_typed_arguments(width):
    D = P.DSML
    text = ("Choose both.</think>\n\n<%s calls>\n<%s invoke name=\"read\">\n<%s parameter name=\"path\" "
            "string=\"true\">目录/😀.rs</%s parameter>\n</%s invoke>\n<%s invoke name=\"read\">\n"
            "<%s parameter name=\"path\" string=\"true\">b.rs</%s parameter>\n<%s parameter name=\"options\" "
            "string=\"false\">{\"lines\": [1, 3], \"raw\": true, \"end\": null}</%s parameter>\n</%s invoke>\n"
            "</%s calls>") % ((D,) * 12)
    r = P.parse_completion(text, True, True, "stop", 10, 99, width=width)
    ch = r["choices"][0]
    assert ch["finish_reason"] == "tool_calls"
    assert ch["message"]["reasoning_content"] == "Choose both."
    calls = ch["message"]["tool_calls"]
    assert len(calls) == 2 and calls[0]["id"] != calls[1]["id"]
    args = [json.loads(c["function"]["arguments"]) for c in calls]
    assert args == [{"path": "目录/😀.rs"}, {"path": "b.rs", "options": {"lines": [1, 3], "raw": True, "end": None}}]
    assert r["usage"]["completion_tokens"] == 99


def test_stream_deltas_concatenate_to_the_whole():
    text = "think hard</think>\n\nThe answer is 4."
    p = P.StreamParser(True, True)
    deltas = []
    for ch in text:
        deltas += p.feed(ch)
    deltas += p.feed("", final=True)
    assert "".join(d.get("reasoning_content", "") for d in deltas) == "think hard"
    assert "".join(d.get("content", "") for d in deltas) == "The answer is 4."
    assert p.result() == {"role": "assistant", "content": "The answer is 4.", "reasoning_content": "think hard"}


def test_render_round_trip_of_tool_calls():
    calls = [{"id": "x", "type": "function", "function": {"name": "f", "arguments": json.dumps({"a": "s", "b": [1, 2]})}}]
    parsed = P.parse_tool_calls(P.render_tool_calls(calls))
    assert json.loads(parsed[0]["function"]["arguments"]) == {"a": "s", "b": [1, 2]}
