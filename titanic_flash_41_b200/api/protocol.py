"""OpenAI-compatible chat protocol: request normalisation, chat template, and the streaming
parser that turns generated text into reasoning / content / tool-call deltas.

Behavioural contract (reference: src/protocol.rs:184-326 normalize_chat_request, :315 max-token
resolution; the chat recipe exercised by src/protocol_recipe_tests.rs:35-101):

* only an allow-list of chat fields is accepted; controls the engine cannot honour are rejected
  with a 400 naming the field;
* tool calls are written by the model as DSML blocks

      <｜DSML｜ calls>
      <｜DSML｜ invoke name="read">
      <｜DSML｜ parameter name="path" string="true">a.rs</｜DSML｜ parameter>
      </｜DSML｜ invoke>
      </｜DSML｜ calls>

  ``string="true"`` parameters are literal strings, ``string="false"`` parameters are JSON;
* reasoning precedes ``</think>``; "Reasoning Effort: N (range 1-100 ...)" is a system line
  (75 for "high", 100 for "max");
* tool results are re-ordered to the order of the calls they answer; adjacent user messages
  merge with a blank line.
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Tuple

DEFAULT_MODEL = "DeepSeek-V4.1-Flash-1017"
DEFAULT_MAX_NEW_TOKENS = 262144

ALLOWED_FIELDS = {
    "messages", "model", "frequency_penalty", "presence_penalty", "logprobs", "top_logprobs", "max_tokens",
    "max_completion_tokens", "n", "seed", "stop", "stream", "stream_options", "temperature", "top_p", "top_k",
    "response_format", "tools", "tool_choice", "reasoning_effort", "thinking", "chat_template_kwargs",
    "parallel_tool_calls",
}

BOS, EOS = "<｜begin▁of▁sentence｜>", "<｜end▁of▁sentence｜>"
USER, ASSISTANT = "<｜User｜>", "<｜Assistant｜>"
THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
DSML = "｜DSML｜"
EFFORT_SCORES = {"low": 25, "medium": 50, "high": 75, "max": 100}


class ProtocolError(ValueError):
    """A request the server answers with 4xx; ``code`` is the machine-readable error code."""

    def __init__(self, message: str, status: int = 400, code: str = "invalid_request_error"):
        super().__init__(message)
        self.status, self.code = status, code


@dataclass
class ChatRequest:
    messages: List[Dict[str, Any]]
    model: str = DEFAULT_MODEL
    stream: bool = False
    include_usage: bool = False
    temperature: float = 1.0
    top_p: float = 1.0
    seed: Optional[int] = None
    max_new_tokens: Optional[int] = None
    tools: List[Dict[str, Any]] = field(default_factory=list)
    tool_choice: str = "auto"
    reasoning_effort: str = "high"
    thinking: bool = True
    background: bool = False


def _num(body, key, default):
    v = body.get(key, default)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ProtocolError(f"{key} must be a number")
    return v


def normalize_chat_request(body: Dict[str, Any], allow_sampling: bool = True) -> ChatRequest:
    """Validate and canonicalise a /v1/chat/completions body.

    ``allow_sampling`` False reproduces the reference's restriction to T in {0, 1}, top_p = 1
    (src/protocol.rs:253-262); this engine's verifier is exact for any temperature / nucleus, so
    the default accepts them."""
    if not isinstance(body, dict):
        raise ProtocolError("request body must be a JSON object")
    for k in body:
        if k not in ALLOWED_FIELDS:
            raise ProtocolError(f"unsupported native chat field: {k}")
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise ProtocolError("messages must be a non-empty array")
    for m in msgs:
        if not isinstance(m, dict) or m.get("role") not in ("system", "developer", "user", "assistant", "tool"):
            raise ProtocolError("every message needs a role of system, developer, user, assistant or tool")
    if _num(body, "frequency_penalty", 0) != 0 or _num(body, "presence_penalty", 0) != 0:
        raise ProtocolError("frequency_penalty and presence_penalty are not supported")
    if body.get("logprobs") not in (None, False) or body.get("top_logprobs") not in (None, 0):
        raise ProtocolError("logprobs are not supported")
    if _num(body, "n", 1) != 1:
        raise ProtocolError("n must be 1")
    stop = body.get("stop")
    if stop not in (None, [], ""):
        raise ProtocolError("stop sequences are not supported")
    if _num(body, "top_k", -1) not in (-1, 0):
        raise ProtocolError("top_k is not supported")
    rf = body.get("response_format")
    if rf is not None and (not isinstance(rf, dict) or rf.get("type", "text") != "text"):
        raise ProtocolError("response_format.type must be text")
    tc = body.get("tool_choice", "auto")
    if tc not in ("auto", "none"):
        raise ProtocolError("tool_choice must be auto or none")
    tools = body.get("tools") or []
    if not isinstance(tools, list):
        raise ProtocolError("tools must be an array")
    for t in tools:
        fn = t.get("function") if isinstance(t, dict) else None
        if not isinstance(fn, dict) or not isinstance(fn.get("name"), str):
            raise ProtocolError("every tool needs function.name")
        if fn.get("strict"):
            raise ProtocolError("strict tools are not supported")
    if "max_tokens" in body and "max_completion_tokens" in body:
        raise ProtocolError("give max_tokens or max_completion_tokens, not both")
    mx = body.get("max_tokens", body.get("max_completion_tokens"))
    if mx is not None and (isinstance(mx, bool) or not isinstance(mx, int) or mx < 1):
        raise ProtocolError("max_tokens must be a positive integer")
    temperature, top_p = float(_num(body, "temperature", 1.0)), float(_num(body, "top_p", 1.0))
    if temperature < 0 or temperature > 2 or not (0 < top_p <= 1):
        raise ProtocolError("temperature must be in [0, 2] and top_p in (0, 1]")
    if not allow_sampling and (temperature not in (0.0, 1.0) or top_p != 1.0):
        raise ProtocolError("only temperature 0 or 1 with top_p 1 is supported")
    effort = body.get("reasoning_effort", "high")
    if effort not in EFFORT_SCORES:
        raise ProtocolError("reasoning_effort must be low, medium, high or max")
    thinking = body.get("thinking")
    think_on = True
    if isinstance(thinking, dict):
        if "budget_tokens" in thinking:
            raise ProtocolError("thinking budgets are not supported")
        think_on = thinking.get("type", "enabled") != "disabled"
    elif isinstance(thinking, bool):
        think_on = thinking
    kw = body.get("chat_template_kwargs") or {}
    if isinstance(kw, dict) and "thinking" in kw:
        think_on = bool(kw["thinking"])
    seed = body.get("seed")
    if seed is not None and (isinstance(seed, bool) or not isinstance(seed, int)):
        raise ProtocolError("seed must be an integer")
    so = body.get("stream_options") or {}
    return ChatRequest(messages=msgs, model=body.get("model") or DEFAULT_MODEL, stream=bool(body.get("stream")),
                       include_usage=bool(isinstance(so, dict) and so.get("include_usage")),
                       temperature=temperature, top_p=top_p, seed=seed, max_new_tokens=mx, tools=tools,
                       tool_choice=tc, reasoning_effort=effort, thinking=think_on)


def resolve_max_tokens(requested: Optional[int], prompt_tokens: int, context: int,
                       default: int = DEFAULT_MAX_NEW_TOKENS) -> int:
    """Default 262,144 new tokens clipped to the remaining context; a prompt that already fills
    the context is an error before any GPU admission (src/protocol.rs:315-326)."""
    remaining = context - prompt_tokens
    if remaining < 1:
        raise ProtocolError(f"prompt of {prompt_tokens} tokens does not fit the {context}-token context",
                            400, "context_length_exceeded")
    return min(requested if requested is not None else default, remaining)


# ---------------------------------------------------------------------------------------------
# chat template
# ---------------------------------------------------------------------------------------------
def _text_of(content: Any) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    if isinstance(content, list):
        parts = []
        for p in content:
            if isinstance(p, dict) and p.get("type") in ("text", "input_text"):
                parts.append(p.get("text", ""))
            elif isinstance(p, dict) and p.get("type") in ("image_url", "input_image", "image"):
                parts.append("<｜image｜>")
        return "".join(parts)
    raise ProtocolError("message content must be a string or an array of parts")


def image_parts(messages: List[Dict[str, Any]]) -> List[str]:
    """URLs / data URIs of every image part, in prompt order."""
    out = []
    for m in messages:
        c = m.get("content")
        if isinstance(c, list):
            for p in c:
                if isinstance(p, dict) and p.get("type") in ("image_url", "input_image", "image"):
                    u = p.get("image_url", p.get("url"))
                    out.append(u.get("url") if isinstance(u, dict) else u)
    return out


def render_tool_calls(calls: List[Dict[str, Any]]) -> str:
    lines = [f"<{DSML} calls>"]
    for c in calls:
        fn = c.get("function", {})
        args = fn.get("arguments", "{}")
        if isinstance(args, str):
            try:
                args = json.loads(args) if args.strip() else {}
            except json.JSONDecodeError:
                raise ProtocolError("tool call arguments must be JSON")
        lines.append(f"<{DSML} invoke name=\"{fn.get('name', '')}\">")
        for k, v in (args or {}).items():
            if isinstance(v, str):
                lines.append(f"<{DSML} parameter name=\"{k}\" string=\"true\">{v}</{DSML} parameter>")
            else:
                lines.append(f"<{DSML} parameter name=\"{k}\" string=\"false\">"
                             f"{json.dumps(v, ensure_ascii=False)}</{DSML} parameter>")
        lines.append(f"</{DSML} invoke>")
    lines.append(f"</{DSML} calls>")
    return "\n".join(lines)


def _tools_block(tools: List[Dict[str, Any]]) -> str:
    specs = [json.dumps(t["function"], ensure_ascii=False, sort_keys=True) for t in tools]
    return ("## Tools\nYou may call the functions below. To call, write a DSML block: "
            f"<{DSML} calls> containing one <{DSML} invoke name=\"...\"> per call with "
            f"<{DSML} parameter name=\"...\" string=\"true|false\"> children.\n" + "\n".join(specs))


def render_chat(req: ChatRequest) -> str:
    """Messages -> prompt text ending where the assistant's turn starts."""
    msgs = [dict(m) for m in req.messages]
    # tool results answer calls in call order, whatever order they arrived in
    ordered: List[Dict[str, Any]] = []
    i = 0
    while i < len(msgs):
        m = msgs[i]
        ordered.append(m)
        i += 1
        if m["role"] == "assistant" and m.get("tool_calls"):
            ids = [c.get("id") for c in m["tool_calls"]]
            j = i
            results = []
            while j < len(msgs) and msgs[j]["role"] == "tool":
                results.append(msgs[j])
                j += 1
            results.sort(key=lambda r: ids.index(r.get("tool_call_id")) if r.get("tool_call_id") in ids else len(ids))
            ordered += results
            i = j
    system = [_text_of(m.get("content")) for m in ordered if m["role"] in ("system", "developer")]
    sys_lines = [s for s in system if s]
    if req.thinking:
        sys_lines.append(f"Reasoning Effort: {EFFORT_SCORES[req.reasoning_effort]} (range 1-100, higher means "
                         "more thorough reasoning)")
    if req.tools and req.tool_choice != "none":
        sys_lines.append(_tools_block(req.tools))
    out = [BOS, "\n\n".join(sys_lines)]
    prev_user = False
    last_prefix = None
    turns = [m for m in ordered if m["role"] not in ("system", "developer")]
    for k, m in enumerate(turns):
        role = m["role"]
        if role == "user":
            text = _text_of(m.get("content"))
            out.append(("\n\n" + text) if prev_user else (USER + text))
            prev_user = True
            continue
        prev_user = False
        if role == "assistant":
            body = ""
            rc = m.get("reasoning_content")
            is_prefix = bool(m.get("prefix")) and k == len(turns) - 1
            content = _text_of(m.get("content"))
            if is_prefix:
                # continuation of an unfinished assistant turn: stop inside reasoning when there is no
                # content yet, else inside the content
                body = (THINK_OPEN + (rc or "")) if (rc and not content) else \
                    ((THINK_OPEN + rc + THINK_CLOSE if rc else THINK_CLOSE) + content)
                last_prefix = body
                out.append(ASSISTANT + body)
                continue
            if rc and m.get("tool_calls"):
                body += THINK_OPEN + rc + THINK_CLOSE     # reasoning is kept only next to tool calls
            else:
                body += THINK_CLOSE
            body += content
            if m.get("tool_calls"):
                body += ("\n\n" if content else "") + render_tool_calls(m["tool_calls"])
            out.append(ASSISTANT + body + EOS)
        elif role == "tool":
            out.append(f"<｜tool▁output｜>{_text_of(m.get('content'))}<｜tool▁output▁end｜>")
    if last_prefix is None:
        out.append(ASSISTANT + (THINK_OPEN if req.thinking else THINK_CLOSE))
    return "".join(out)


# ---------------------------------------------------------------------------------------------
# streaming parser: generated text -> reasoning / content / tool-call deltas
# ---------------------------------------------------------------------------------------------
_CALLS_OPEN, _CALLS_CLOSE = f"<{DSML} calls>", f"</{DSML} calls>"
_INVOKE_RE = re.compile(rf"<{DSML} invoke name=\"([^\"]*)\">(.*?)</{DSML} invoke>", re.S)
_PARAM_RE = re.compile(rf"<{DSML} parameter name=\"([^\"]*)\" string=\"(true|false)\">(.*?)</{DSML} parameter>", re.S)


def parse_tool_calls(block: str) -> List[Dict[str, Any]]:
    """DSML calls block -> OpenAI tool_calls (arguments as a JSON string, typed per parameter)."""
    calls = []
    for name, body in _INVOKE_RE.findall(block):
        args: Dict[str, Any] = {}
        for pname, is_str, val in _PARAM_RE.findall(body):
            if is_str == "true":
                args[pname] = val
            else:
                try:
                    args[pname] = json.loads(val)
                except json.JSONDecodeError:
                    args[pname] = val
        calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                      "function": {"name": name, "arguments": json.dumps(args, ensure_ascii=False)}})
    return calls


class StreamParser:
    """Incremental parser.  ``feed(text)`` returns a list of deltas
    ({"reasoning_content": ..} | {"content": ..} | {"tool_calls": [..]}); text that might be the
    start of a marker is held back until it is disambiguated, so a marker split across pieces of
    any width parses the same (reference test: widths 1, 3, 17, 256)."""

    def __init__(self, thinking: bool = True, tools: bool = True):
        self.state = "reasoning" if thinking else "content"
        self.tools = tools
        self.buf = ""
        self.reasoning, self.content = [], []
        self.tool_calls: List[Dict[str, Any]] = []
        self._call_index = 0
        self._skip_nl = 0        # newlines of the separator after </think> still to swallow

    def _markers(self) -> Tuple[str, ...]:
        if self.state == "reasoning":
            return (THINK_CLOSE,)
        if self.state == "content":
            return (_CALLS_OPEN,) if self.tools else ()
        return (_CALLS_CLOSE,)

    @staticmethod
    def _holdback(buf: str, markers: Iterable[str]) -> int:
        """Length of the longest suffix of buf that is a proper prefix of a marker."""
        best = 0
        for m in markers:
            for n in range(min(len(m) - 1, len(buf)), 0, -1):
                if buf.endswith(m[:n]):
                    best = max(best, n)
                    break
        return best

    def _emit(self, text: str, out: List[Dict[str, Any]]) -> None:
        if not text:
            return
        if self.state == "reasoning":
            self.reasoning.append(text)
            out.append({"reasoning_content": text})
        elif self.state == "content":
            while self._skip_nl and text.startswith("\n"):
                text, self._skip_nl = text[1:], self._skip_nl - 1
            if not text:
                return
            self._skip_nl = 0
            self.content.append(text)
            out.append({"content": text})

    def feed(self, text: str, final: bool = False) -> List[Dict[str, Any]]:
        out: List[Dict[str, Any]] = []
        self.buf += text
        while True:
            markers = self._markers()
            hit, pos = None, -1
            for m in markers:
                p = self.buf.find(m)
                if p >= 0 and (pos < 0 or p < pos):
                    hit, pos = m, p
            if hit is None:
                keep = 0 if final else self._holdback(self.buf, markers)
                if self.state == "calls":
                    if final:
                        self._finish_calls(self.buf, out)
                        self.buf = ""
                    break
                emit = self.buf[: len(self.buf) - keep]
                self.buf = self.buf[len(self.buf) - keep:]
                self._emit(emit, out)
                break
            before, self.buf = self.buf[:pos], self.buf[pos + len(hit):]
            if self.state == "reasoning":
                self._emit(before, out)
                self.state = "content"
                self._skip_nl = 2
            elif self.state == "content":
                self._emit(before.rstrip("\n") if before.strip() == "" else before, out)
                self.state = "calls"
            else:
                self._finish_calls(before, out)
                self.state = "content"
        return out

    def _finish_calls(self, block: str, out: List[Dict[str, Any]]) -> None:
        calls = parse_tool_calls(block)
        for c in calls:
            c["index"] = self._call_index
            self._call_index += 1
        if calls:
            self.tool_calls += calls
            out.append({"tool_calls": calls})

    def result(self) -> Dict[str, Any]:
        content = "".join(self.content)
        if content.startswith("\n\n"):
            content = content[2:]
        msg: Dict[str, Any] = {"role": "assistant", "content": content.rstrip("\n") if self.tool_calls else content}
        r = "".join(self.reasoning)
        if r:
            msg["reasoning_content"] = r
        if self.tool_calls:
            msg["tool_calls"] = [{k: v for k, v in c.items() if k != "index"} for c in self.tool_calls]
        return msg


def parse_completion(text: str, thinking: bool, tools: bool, finish: str, prompt_tokens: int,
                     completion_tokens: int, model: str = DEFAULT_MODEL, width: int = 0) -> Dict[str, Any]:
    """Whole completion text -> chat.completion object (reference: Frontend::parse_completion,
    src/protocol.rs:518).  ``width`` > 0 feeds the parser in pieces of that many characters."""
    p = StreamParser(thinking, tools)
    if width > 0:
        for i in range(0, len(text), width):
            p.feed(text[i:i + width])
        p.feed("", final=True)
    else:
        p.feed(text, final=True)
    msg = p.result()
    if msg.get("tool_calls"):
        finish = "tool_calls"
    return {"id": "chatcmpl-" + uuid.uuid4().hex, "object": "chat.completion", "model": model,
            "choices": [{"index": 0, "message": msg, "finish_reason": finish}],
            "usage": {"prompt_tokens": prompt_tokens, "completion_tokens": completion_tokens,
                      "total_tokens": prompt_tokens + completion_tokens}}
