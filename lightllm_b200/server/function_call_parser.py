"""Tool-call extraction from generated text (whole text and streaming) for the chat route.

Every supported syntax is described by a begin marker, an end marker and a body decoder that
turns the text between them into (name, json-arguments) pairs.  The streaming parser withholds
text from the first (possibly partial) begin marker on and emits each call once its body is
complete: one delta with the function name and the full argument string.

Reference: lightllm/server/function_call_parser.py (qwen25, llama3, mistral, deepseekv3/v31/v32,
glm47, kimi_k2, qwen3_coder).
"""
from __future__ import annotations

import json
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
        self.tool_names = set()
        for t in tools or []:
            fn = getattr(t, "function", None) or (t.get("function") if isinstance(t, dict) else None)
            name = getattr(fn, "name", None) or (fn.get("name") if isinstance(fn, dict) else None)
            if name:
                self.tool_names.add(name)
        self._buf = ""
        self._index = 0
        self._in_call = False

    def has_tool_call(self, text: str) -> bool:
        return self.fmt.begin in text

    def _items(self, body: str) -> List[ToolCallItem]:
        out = []
        for name, args in self.fmt.decode(body):
            if self.tool_names and name not in self.tool_names:
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
                    continue
                keep = 0
                for n in range(min(len(f.begin) - 1, len(self._buf)), 0, -1):
                    if f.begin.startswith(self._buf[-n:]):
                        keep = n
                        break
                normal += self._buf[:len(self._buf) - keep]
                self._buf = self._buf[len(self._buf) - keep:]
                break
            if f.end is None:
                # body runs to the end of generation: try to decode what we have when it parses as JSON
                items = self._items(self._buf)
                if items:
                    calls += items
                    self._buf = ""
                break
            j = self._buf.find(f.end)
            if j < 0:
                break
            calls += self._items(self._buf[:j])
            self._buf = self._buf[j + len(f.end):]
            self._in_call = False
        return normal, calls
