"""Tool-call extraction from generated text (whole text and streaming) for the chat route.

Every supported syntax is described by a begin marker, an end marker and a body decoder that
turns the text between them into (name, json-arguments) pairs.  The streaming parser withholds
text from the first (possibly partial) begin marker on.  For the JSON-bodied syntaxes (a single
`{"name": ..., "arguments": {...}}` object per call) a call is streamed the way OpenAI clients expect:
one delta with the function name and empty arguments as soon as the name is complete, then the
argument text piece by piece as it is generated (deltas without a name, same tool index).  Bodies
of any other shape (lists of calls, arguments given as a string, the tag-based syntaxes) are
emitted once complete: one delta with the name and the full argument string.

Reference: lightllm/server/function_call_parser.py (qwen25, llama3, mistral, deepseekv3/v31/v32,
glm47, kimi_k2, qwen3_coder).
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple


@dataclass
class ToolCallItem:
    tool_index: int
    name: Optional[str]
    parameters: str


def _json_calls(body: str) -> List[Tuple[str, str]]:
    body = body.strip()
    if not body:
        return []
    try:
        obj = json.loads(body)
    except json.JSONDecodeError:
        # several objects separated by newlines / semicolons
        out = []
        for part in re.split(r"\n+|;", body):
            part = part.strip()
            if part:
                try:
                    out += _json_calls(part)
                except Exception:
                    pass
        return out
    objs = obj if isinstance(obj, list) else [obj]
    out = []
    for o in objs:
        if isinstance(o, dict) and "name" in o:
            args = o.get("arguments", o.get("parameters", {}))
            out.append((o["name"], args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)))
    return out


def _deepseek_v3_calls(body: str):
    out = []
    for m in re.finditer(r"<｜tool▁call▁begin｜>(?:function)?<｜tool▁sep｜>(.*?)\n```json\n(.*?)\n```<｜tool▁call▁end｜>", body, re.S):
        out.append((m.group(1).strip(), m.group(2).strip()))
    return out


def _deepseek_v31_calls(body: str):
    return [(m.group(1).strip(), m.group(2).strip())
            for m in re.finditer(r"<｜tool▁call▁begin｜>(.*?)<｜tool▁sep｜>(.*?)<｜tool▁call▁end｜>", body, re.S)]


def _deepseek_v32_calls(body: str):
    out = []
    for m in re.finditer(r"<｜DSML｜invoke name=\"(.*?)\">(.*?)</｜DSML｜invoke>", body, re.S):
        args = {}
        for p in re.finditer(r"<｜DSML｜parameter name=\"(.*?)\"(?: string=\"(true|false)\")?>(.*?)</｜DSML｜parameter>", m.group(2), re.S):
            val = p.group(3)
            if p.group(2) == "true":
                args[p.group(1)] = val
            else:
                try:
                    args[p.group(1)] = json.loads(val)
                except Exception:
                    args[p.group(1)] = val
        out.append((m.group(1), json.dumps(args, ensure_ascii=False)))
    return out


def _glm_calls(body: str):
    lines = body.strip().split("\n", 1)
    name = lines[0].strip()
    rest = lines[1] if len(lines) > 1 else ""
    args = {}
    for m in re.finditer(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", rest, re.S):
        v = m.group(2).strip()
        try:
            args[m.group(1).strip()] = json.loads(v)
        except Exception:
            args[m.group(1).strip()] = v
    return [(name, json.dumps(args, ensure_ascii=False))] if name else []


def _kimi_calls(body: str):
    out = []
    for m in re.finditer(r"<\|tool_call_begin\|>\s*(?:functions\.)?([\w\.\-]+?)(?::\d+)?\s*<\|tool_call_argument_begin\|>(.*?)<\|tool_call_end\|>", body, re.S):
        out.append((m.group(1), m.group(2).strip()))
    return out


def _qwen3_coder_calls(body: str):
    out = []
    for m in re.finditer(r"<function=(.*?)>(.*?)</function>", body, re.S):
        args = {}
        for p in re.finditer(r"<parameter=(.*?)>\n?(.*?)\n?</parameter>", m.group(2), re.S):
            v = p.group(2)
            try:
                args[p.group(1).strip()] = json.loads(v)
            except Exception:
                args[p.group(1).strip()] = v
        out.append((m.group(1).strip(), json.dumps(args, ensure_ascii=False)))
    return out


_JSON_HEAD = re.compile(r'\s*\{\s*"name"\s*:\s*"((?:[^"\\]|\\.)*)"\s*,\s*"(?:arguments|parameters)"\s*:\s*')


class _JsonArgStream:
    """Incremental view of one `{"name": "f", "arguments": {...}}` body: `feed(body)` is called with everything
    received so far and returns (name or None on later calls, new piece of the argument text).  `usable` turns
    False as soon as the body cannot be streamed this way (the caller then waits for the whole body)."""

    def __init__(self):
        self.usable = True
        self.name_sent = False
        self.val_start = -1
        self.emitted = 0          # characters of the argument value handed out
        self.complete = False     # the argument value has been closed
        # scanner state inside the value
        self._pos, self._depth, self._in_str, self._esc = 0, 0, False, False

    def feed(self, body: str):
        if not self.usable or self.complete:
            return None, ""
        if self.val_start < 0:
            m = _JSON_HEAD.match(body)
            if m is None:
                head = body.lstrip()
                # still a prefix of what the pattern wants?  (a '{', then "name", its string, a comma, the key)
                probe = '{"name":'
                compact = re.sub(r"\s+", "", head[:64])
                if compact and not (probe.startswith(compact[:len(probe)]) or compact.startswith(probe)):
                    self.usable = False
                return None, ""
            if m.end() >= len(body):
                return None, ""
            if body[m.end()] not in "{[":
                self.usable = False      # arguments given as a string or a scalar: decode at the end
                return None, ""
            self.val_start = self._pos = m.end()
            self._name = json.loads('"' + m.group(1) + '"')
        # advance the scanner to find the end of the value (if it is there yet)
        i = self._pos
        while i < len(body) and not self.complete:
            ch = body[i]
            if self._in_str:
                if self._esc:
                    self._esc = False
                elif ch == "\\":
                    self._esc = True
                elif ch == '"':
                    self._in_str = False
            elif ch == '"':
                self._in_str = True
            elif ch in "{[":
                self._depth += 1
            elif ch in "}]":
                self._depth -= 1
                if self._depth == 0:
                    self.complete = True
            i += 1
        self._pos = i
        piece = body[self.val_start + self.emitted:i]
        self.emitted += len(piece)
        name = None
        if not self.name_sent:
            self.name_sent = True
            name = self._name
        return name, piece


@dataclass
class CallFormat:
    begin: str
    end: Optional[str]          # None: the call runs to the end of the text
    decode: Callable[[str], List[Tuple[str, str]]]
    keep_markers: bool = False  # the decoder wants begin/end included in the body


_FORMATS: Dict[str, CallFormat] = {
    "qwen25": CallFormat("<tool_call>", "</tool_call>", _json_calls),
    "qwen": CallFormat("<tool_call>", "</tool_call>", _json_calls),
    "llama3": CallFormat("<|python_tag|>", None, _json_calls),
    "mistral": CallFormat("[TOOL_CALLS]", None, _json_calls),
    "deepseekv3": CallFormat("<｜tool▁calls▁begin｜>", "<｜tool▁calls▁end｜>", _deepseek_v3_calls),
    "deepseekv31": CallFormat("<｜tool▁calls▁begin｜>", "<｜tool▁calls▁end｜>", _deepseek_v31_calls),
    "deepseekv32": CallFormat("<｜DSML｜function_calls>", "</｜DSML｜function_calls>", _deepseek_v32_calls),
    "glm47": CallFormat("<tool_call>", "</tool_call>", _glm_calls),
    "kimi_k2": CallFormat("<|tool_calls_section_begin|>", "<|tool_calls_section_end|>", _kimi_calls),
    "qwen3_coder": CallFormat("<tool_call>", "</tool_call>", _qwen3_coder_calls),
}


class FunctionCallParser:
    def __init__(self, tools: Optional[List[Any]], tool_call_parser: str):
        if tool_call_parser not in _FORMATS:
            raise ValueError(f"unknown tool call parser {tool_call_parser!r}; known: {sorted(_FORMATS)}")
        self.fmt = _FORMATS[tool_call_parser]
        # with LIGHTLLM_ENABLE_TOOL_NAME_CHECK=1 calls to functions that the request did not declare are dropped
        self.check_names = os.getenv("LIGHTLLM_ENABLE_TOOL_NAME_CHECK", "False").upper() in ("ON", "TRUE", "1")
        self.tool_names = set()
        for t in tools or []:
            fn = getattr(t, "function", None) or (t.get("function") if isinstance(t, dict) else None)
            name = getattr(fn, "name", None) or (fn.get("name") if isinstance(fn, dict) else None)
            if name:
                self.tool_names.add(name)
        self._buf = ""
        self._index = 0
        self._in_call = False
        self._json_stream: Optional[_JsonArgStream] = None   # per call, JSON-bodied syntaxes only

    def has_tool_call(self, text: str) -> bool:
        return self.fmt.begin in text

    def _items(self, body: str) -> List[ToolCallItem]:
        out = []
        for name, args in self.fmt.decode(body):
            if self.check_names and self.tool_names and name not in self.tool_names:
                continue
            out.append(ToolCallItem(self._index, name, args))
            self._index += 1
        return out

    def parse_non_stream(self, text: str) -> Tuple[str, List[ToolCallItem]]:
        f = self.fmt
        normal, calls = [], []
        pos = 0
        while True:
            i = text.find(f.begin, pos)
            if i < 0:
                normal.append(text[pos:])
                break
            normal.append(text[pos:i])
            if f.end is None:
                calls += self._items(text[i + len(f.begin):])
                break
            j = text.find(f.end, i + len(f.begin))
            if j < 0:
                calls += self._items(text[i + len(f.begin):])
                break
            calls += self._items(text[i + len(f.begin):j])
            pos = j + len(f.end)
        return "".join(normal).strip("\n"), calls

    def _stream_json_body(self, body: str, calls: List[ToolCallItem]) -> bool:
        """Feeds the body received so far to the incremental JSON view; returns True while that view is in charge
        of this call (False: the body has to be decoded as a whole)."""
        js = self._json_stream
        if js is None or not js.usable:
            return False
        name, piece = js.feed(body)
        if not js.usable:
            return False
        if name is not None:
            if self.check_names and self.tool_names and name not in self.tool_names:
                js.usable = False          # not one of the declared tools: dropped like in the whole-body path
                js.dropped = True
                return True
            calls.append(ToolCallItem(self._index, name, ""))
        if piece and not getattr(js, "dropped", False):
            calls.append(ToolCallItem(self._index, None, piece))
        return True

    def parse_stream_chunk(self, chunk: str) -> Tuple[str, List[ToolCallItem]]:
        f = self.fmt
        self._buf += chunk
        normal, calls = "", []
        while True:
            if not self._in_call:
                i = self._buf.find(f.begin)
                if i >= 0:
                    normal += self._buf[:i]
                    self._buf = self._buf[i + len(f.begin):]
                    self._in_call = True
                    self._json_stream = _JsonArgStream() if f.decode is _json_calls else None
                    continue
                keep = 0
                for n in range(min(len(f.begin) - 1, len(self._buf)), 0, -1):
                    if f.begin.startswith(self._buf[-n:]):
                        keep = n
                        break
                normal += self._buf[:len(self._buf) - keep]
                self._buf = self._buf[len(self._buf) - keep:]
                break
            js = self._json_stream
            if f.end is None:
                # body runs to the end of generation
                if getattr(self, "_swallow", False):  # the call was streamed to its end: drop what follows it
                    self._buf = ""
                    break
                if self._stream_json_body(self._buf, calls) or getattr(js, "dropped", False):
                    if js.complete and js.name_sent and not getattr(js, "dropped", False):
                        self._index += 1
                        self._swallow = True
                    break
                if js is not None and js.name_sent:
                    break                             # already handed out incrementally
                items = self._items(self._buf)        # decode what we have once it parses as JSON
                if items:
                    calls += items
                    self._buf = ""
                break
            j = self._buf.find(f.end)
            if j < 0:
                # keep a possible partial end marker out of the incremental view
                hold = 0
                for n in range(min(len(f.end) - 1, len(self._buf)), 0, -1):
                    if f.end.startswith(self._buf[-n:]):
                        hold = n
                        break
                self._stream_json_body(self._buf[:len(self._buf) - hold], calls)
                break
            streamed = self._stream_json_body(self._buf[:j], calls)
            if streamed or (js is not None and js.name_sent):
                if js.name_sent and not getattr(js, "dropped", False):
                    self._index += 1
            else:
                calls += self._items(self._buf[:j])
            self._buf = self._buf[j + len(f.end):]
            self._in_call = False
            self._json_stream = None
        return normal, calls
