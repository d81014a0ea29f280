"""Prompt format of DeepSeek-V3.2, rendered in Python: the model ships no Jinja chat template.

`render(messages, thinking)` turns an OpenAI-style conversation (system / developer / user / assistant / tool
messages, tool definitions and assistant tool calls) into the prompt string; `parse_completion(text, thinking)`
turns a completed answer back into a message (reasoning, content, tool calls).  `DeepSeekV32Tokenizer` wraps a
Hugging Face tokenizer so that `apply_chat_template` goes through `render`.

The wire format: `<｜User｜>…<｜Assistant｜>` turns, a `<think>` opener after the last user turn in thinking mode and
a `</think>` closer everywhere else, assistant turns closed by the end-of-sentence token, tool calls as
`<｜DSML｜function_calls>` blocks of `invoke` / `parameter` elements (string parameters verbatim, everything else as
JSON) and tool outputs as `<function_results><result>…</result></function_results>`.

Reference: lightllm/models/deepseek3_2/encoding_dsv32.py (encode_messages, render_message,
parse_message_from_completion_text) and lightllm/models/deepseek3_2/model.py:24-108 (DeepSeekV32Tokenizer).
"""
from __future__ import annotations

import copy
import json
import re
from typing import Any, Dict, List, Optional

BOS = "<｜begin▁of▁sentence｜>"
EOS = "<｜end▁of▁sentence｜>"
THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
DSML = "｜DSML｜"
USER_TAG, ASSISTANT_TAG = "<｜User｜>", "<｜Assistant｜>"
CALLS_OPEN, CALLS_CLOSE = f"<{DSML}function_calls>", f"</{DSML}function_calls>"

# the tool preamble the model was trained with; {D} the DSML marker, {tools} one JSON schema per line
_TOOLS_PREAMBLE = (
    "## Tools\n"
    "You have access to a set of tools you can use to answer the user's question.\n"
    'You can invoke functions by writing a "<{D}function_calls>" block like the following as part of your reply '
    "to the user:\n"
    "<{D}function_calls>\n"
    '<{D}invoke name="$FUNCTION_NAME">\n'
    '<{D}parameter name="$PARAMETER_NAME" string="true|false">$PARAMETER_VALUE</{D}parameter>\n'
    "...\n"
    "</{D}invoke>\n"
    '<{D}invoke name="$FUNCTION_NAME2">\n'
    "...\n"
    "</{D}invoke>\n"
    "</{D}function_calls>\n"
    "String and scalar parameters should be specified as is without any escaping or quotes, while lists and objects "
    'should use JSON format. The "string" attribute should be set to "true" for string type parameters and "false" '
    "for other types (numbers, booleans, arrays, objects).\n"
    "If the thinking_mode is enabled, then after function results you should strongly consider outputting a thinking "
    "block. Here is an example:\n"
    "<{D}function_calls>\n"
    "...\n"
    "</{D}function_calls>\n"
    "<function_results>\n"
    "...\n"
    "</function_results>\n"
    "{TO}...thinking about results{TC}\n"
    "Here are the functions available in JSONSchema format:\n"
    "<functions>\n"
    "{tools}\n"
    "</functions>\n"
)
_FORMAT_PREAMBLE = "## Response Format:\n\nYou MUST strictly adhere to the following schema to reply:\n"


def _json(v: Any) -> str:
    try:
        return json.dumps(v, ensure_ascii=False)
    except (TypeError, ValueError):
        return json.dumps(v, ensure_ascii=True, default=str)


def _function_of(tool: dict) -> dict:
    return tool["function"] if "function" in tool else tool


def tools_section(tools: List[dict]) -> str:
    """The system-prompt section that lists the callable functions (OpenAI wrappers or bare function dicts)."""
    return _TOOLS_PREAMBLE.format(D=DSML, TO=THINK_OPEN, TC=THINK_CLOSE,
                                  tools="\n".join(_json(_function_of(t)) for t in tools))


def _call_block(call: dict) -> str:
    fn = call.get("function", call)
    args = fn.get("arguments") or {}
    if isinstance(args, str):
        args = json.loads(args) if args.strip() else {}
    lines = [f'<{DSML}invoke name="{fn.get("name")}">']
    for k, v in args.items():
        is_str = isinstance(v, str)
        lines.append(f'<{DSML}parameter name="{k}" string="{"true" if is_str else "false"}">'
                     f'{v if is_str else _json(v)}</{DSML}parameter>')
    lines.append(f"</{DSML}invoke>")
    return "\n".join(lines)


def _last_user(messages: List[dict]) -> int:
    for i in range(len(messages) - 1, -1, -1):
        if messages[i].get("role") in ("user", "developer"):
            return i
    return -1


def _extras(msg: dict) -> str:
    out = ""
    if msg.get("tools"):
        out += "\n\n" + tools_section(msg["tools"])
    if msg.get("response_format"):
        out += "\n\n" + _FORMAT_PREAMBLE + _json(msg["response_format"])
    return out


class _Renderer:
    def __init__(self, messages: List[dict], thinking: bool):
        self.m, self.thinking, self.last_user = messages, thinking, _last_user(messages)

    def _turn_end(self, opens: bool) -> str:
        return THINK_OPEN if (opens and self.thinking) else THINK_CLOSE

    def one(self, i: int) -> str:
        msg = self.m[i]
        role = msg.get("role")
        fn = getattr(self, f"_{role}", None) if isinstance(role, str) else None
        if fn is None:
            raise ValueError(f"message {i}: unknown role {role!r}")
        return fn(i, msg)

    def _system(self, i, msg):
        return (msg.get("content") or "") + _extras(msg)

    def _user(self, i, msg):
        return f"{USER_TAG}{msg.get('content')}{ASSISTANT_TAG}" + self._turn_end(i == self.last_user)

    def _developer(self, i, msg):
        if not msg.get("content"):
            raise ValueError(f"message {i}: a developer message needs content")
        body = _extras(msg) + f"\n\n# The user's message is: {msg['content']}"
        return f"{USER_TAG}{body}{ASSISTANT_TAG}" + self._turn_end(i == self.last_user)

    def _assistant(self, i, msg):
        calls = msg.get("tool_calls") or []
        text = msg.get("content") or ""
        if msg.get("prefix") and not calls:
            return text                    # a prefix to be continued: left open
        think = ""
        if self.thinking and i > self.last_user:
            reasoning = msg.get("reasoning") or msg.get("reasoning_content")
            if not (reasoning or calls):
                raise ValueError(f"message {i}: in thinking mode an assistant message after the last user turn needs "
                                 "reasoning or tool calls")
            think = (reasoning or "") + THINK_CLOSE
        block = ""
        if calls:
            block = "\n\n" + CALLS_OPEN + "\n" + "\n".join(_call_block(c) for c in calls) + "\n" + CALLS_CLOSE
        return think + text + block + EOS

    def _tool(self, i, msg):
        j = i - 1
        while j >= 0 and self.m[j].get("role") == "tool":
            j -= 1
        if j < 0 or self.m[j].get("role") != "assistant":
            raise ValueError(f"message {i}: a tool output without the assistant message that called it")
        calls = self.m[j].get("tool_calls") or []
        k = i - j                                   # 1-based position among this assistant turn's outputs
        if len(calls) < k:
            raise ValueError(f"message {i}: more tool outputs than tool calls")
        out = "\n\n<function_results>" if k == 1 else ""
        out += f"\n<result>{msg.get('content')}</result>"
        if k == len(calls):
            out += "\n</function_results>\n\n" + self._turn_end(i >= self.last_user)
        return out


def _without_old_reasoning(messages: List[dict]) -> List[dict]:
    """Reasoning of assistant turns before the last user turn is not fed back.  Developer messages before the last
    user turn are left out as well: the model's published encoder does so, and prompts should look as in training."""
    last = _last_user(messages)
    out = []
    for i, m in enumerate(messages):
        if i < last:
            role = m.get("role")
            if role == "assistant":
                m = {k: v for k, v in m.items() if k not in ("reasoning", "reasoning_content")}
            elif role not in ("user", "system", "tool"):
                continue
        out.append(m)
    return out


def render(messages: List[dict], thinking: bool = False, context: Optional[List[dict]] = None,
           drop_thinking: bool = True, add_bos: bool = True) -> str:
    """Prompt for `messages`; with `context` (earlier messages already rendered) only the new ones are emitted."""
    context = list(context or [])
    full = context + list(messages)
    if thinking and drop_thinking:
        full = _without_old_reasoning(full)
    r = _Renderer(full, thinking)
    head = BOS if (add_bos and not context) else ""
    return head + "".join(r.one(len(context) + i) for i in range(len(messages)))


# ------------------------------------------------------------------ completion -> message
_INVOKE = re.compile(rf'<{DSML}invoke name="(.*?)">\n(.*?)</{DSML}invoke>\n', re.S)
_PARAM = re.compile(rf'<{DSML}parameter name="(.*?)" string="(true|false)">(.*?)</{DSML}parameter>\n', re.S)


def _parse_calls(block: str) -> List[dict]:
    """`block` is what stands between the opening and closing function_calls markers."""
    if not block.startswith("\n"):
        raise ValueError("tool call block: missing line break after the opening marker")
    pos, calls = 1, []
    while pos < len(block):
        m = _INVOKE.match(block, pos)
        if m is None:
            raise ValueError("tool call block: malformed invoke element")
        args, p = {}, 0
        body = m.group(2)
        while p < len(body):
            pm = _PARAM.match(body, p)
            if pm is None:
                raise ValueError("tool call block: malformed parameter element")
            name, is_str, val = pm.groups()
            if name in args:
                raise ValueError(f"tool call block: parameter {name!r} given twice")
            args[name] = _json(val) if is_str == "true" else val
            p = pm.end()
        arguments = "{" + ", ".join(f"{_json(k)}: {v}" for k, v in args.items()) + "}"
        calls.append({"type": "function", "function": {"name": m.group(1), "arguments": arguments}})
        pos = m.end()
    return calls


def parse_completion(text: str, thinking: bool = False) -> Dict[str, Any]:
    """Splits a well-formed completion (as the model writes it after the prompt) into reasoning, content and tool
    calls.  Raises ValueError on anything else; it does not repair."""
    reasoning = ""
    calls_start = "\n\n" + CALLS_OPEN
    if thinking:
        end = text.find(THINK_CLOSE)
        early_calls = text.find(calls_start)
        if end < 0 or (0 <= early_calls < end):
            raise ValueError("thinking mode: no closing think marker before the answer")
        reasoning, text = text[:end], text[end + len(THINK_CLOSE):]
    calls: List[dict] = []
    at = text.find(calls_start)
    if at < 0:
        if not text.endswith(EOS):
            raise ValueError("the completion does not end with the end-of-sentence token")
        content = text[: -len(EOS)]
    else:
        content, rest = text[:at], text[at + len(calls_start):]
        close = rest.find(CALLS_CLOSE)
        if close < 0:
            raise ValueError("tool call block is not closed")
        if rest[close + len(CALLS_CLOSE):] not in ("", EOS):
            raise ValueError("text after the tool call block")
        calls = _parse_calls(rest[:close])
    for marker in (BOS, EOS, THINK_OPEN, THINK_CLOSE, DSML):
        if marker in content or marker in reasoning:
            raise ValueError(f"marker {marker!r} inside the text")
    return {"role": "assistant", "content": content, "reasoning": reasoning, "tool_calls": calls}


# ------------------------------------------------------------------ tokenizer wrapper
class DeepSeekV32Tokenizer:
    """A Hugging Face tokenizer whose `apply_chat_template` renders with this module.  Everything else is the inner
    tokenizer's."""

    def __init__(self, tokenizer):
        self.tokenizer = tokenizer
        self._added_vocab = None

    def __getattr__(self, name):
        return getattr(self.tokenizer, name)

    def __len__(self):
        return len(self.tokenizer)

    def get_added_vocab(self):
        if self._added_vocab is None:
            self._added_vocab = self.tokenizer.get_added_vocab()
        return self._added_vocab

    @property
    def chat_template(self):
        return "deepseek_v32"     # not Jinja: tells callers that a template exists

    def apply_chat_template(self, conversation=None, messages=None, tools=None, tokenize=False,
                            add_generation_prompt=True, thinking=None, enable_thinking=None, **kw):
        msgs = conversation if conversation is not None else messages
        if msgs is None:
            raise ValueError("apply_chat_template needs the conversation")
        if kw.get("chat_template"):       # an explicit Jinja template wins
            return self.tokenizer.apply_chat_template(msgs, tools=tools, tokenize=tokenize,
                                                      add_generation_prompt=add_generation_prompt, **kw)
        msgs = copy.deepcopy(list(msgs))
        if tools:
            wrapped = [t if "function" in t else {"type": "function", "function": t} for t in tools]
            sys_msg = next((m for m in msgs if m.get("role") == "system"), None)
            if sys_msg is None:
                msgs.insert(0, {"role": "system", "content": "", "tools": wrapped})
            else:
                sys_msg["tools"] = list(sys_msg.get("tools") or []) + wrapped
        think = bool(thinking if thinking is not None else enable_thinking)
        prompt = render(msgs, thinking=think, drop_thinking=kw.get("drop_thinking", True),
                        add_bos=kw.get("add_default_bos_token", True))
        if tokenize:
            return self.tokenizer.encode(prompt, add_special_tokens=False)
        return prompt
