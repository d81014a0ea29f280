"""Splits model output into reasoning content and the final answer, for whole texts and for
streams.  Each model family is described by its opening / closing markers and whether generation
starts inside the reasoning block (the chat template already emitted the opening marker).

Reference: lightllm/server/reasoning_parser.py (detectors for deepseek-r1, qwen3, gpt-oss, glm45,
kimi, minimax, step3, nano_v3, interns1, gemma4).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass
class ThinkFormat:
    start: str
    end: str
    force_reasoning: bool = False   # output begins inside the block even without the start marker
    strip_prefix: str = ""          # text to drop from the start of the answer (e.g. a channel header)


_FORMATS = {
    "deepseek-r1": ThinkFormat("<think>", "</think>", force_reasoning=True),
    "deepseek-v3": ThinkFormat("<think>", "</think>"),
    "qwen3": ThinkFormat("<think>", "</think>"),
    "qwen3-thinking": ThinkFormat("<think>", "</think>", force_reasoning=True),
    "glm45": ThinkFormat("<think>", "</think>"),
    "kimi": ThinkFormat("◁think▷", "◁/think▷"),
    "kimi_k2": ThinkFormat("<think>", "</think>"),
    "minimax": ThinkFormat("<think>", "</think>"),
    "minimax-append-think": ThinkFormat("<think>", "</think>", force_reasoning=True),
    "step3": ThinkFormat("<think>", "</think>", force_reasoning=True),
    "nano_v3": ThinkFormat("<think>", "</think>", force_reasoning=True),
    "interns1": ThinkFormat("<think>", "</think>", force_reasoning=True),
    "gemma4": ThinkFormat("<think>", "</think>"),
    "gpt-oss": ThinkFormat("<|channel|>analysis<|message|>", "<|end|>",
                           strip_prefix="<|start|>assistant<|channel|>final<|message|>"),
}


class ReasoningParser:
    def __init__(self, model_type: str, stream_reasoning: bool = True, force_reasoning: Optional[bool] = None):
        if model_type not in _FORMATS:
            raise ValueError(f"unknown reasoning parser {model_type!r}; known: {sorted(_FORMATS)}")
        self.fmt = _FORMATS[model_type]
        self.stream_reasoning = stream_reasoning
        self.in_reasoning = self.fmt.force_reasoning if force_reasoning is None else force_reasoning
        self.done = False
        self._buf = ""
        self._held_reasoning = ""

    # ---- whole text ----
    def parse_non_stream(self, text: str) -> Tuple[Optional[str], str]:
        f = self.fmt
        in_r = self.in_reasoning
        if f.start in text:
            before, _, rest = text.partition(f.start)
            in_r = True
            text = before + rest if not before.strip() else rest
        if not in_r:
            return None, self._clean(text)
        if f.end in text:
            reasoning, _, answer = text.partition(f.end)
            return reasoning.strip() or None, self._clean(answer)
        return text.strip() or None, ""  # truncated inside the block

    def _clean(self, answer: str) -> str:
        a = answer
        if self.fmt.strip_prefix and a.lstrip().startswith(self.fmt.strip_prefix):
            a = a.lstrip()[len(self.fmt.strip_prefix):]
        return a.lstrip("\n") if a.startswith("\n\n") else a

    # ---- stream ----
    @staticmethod
    def _partial_suffix(buf: str, marker: str) -> int:
        """Length of the longest suffix of `buf` that is a proper prefix of `marker`."""
        for n in range(min(len(marker) - 1, len(buf)), 0, -1):
            if marker.startswith(buf[-n:]):
                return n
        return 0

    def parse_stream_chunk(self, chunk: str) -> Tuple[Optional[str], str]:
        """Returns (reasoning delta or None, answer delta)."""
        f = self.fmt
        self._buf += chunk
        reasoning_out, answer_out = "", ""
        while True:
            if self.done:
                answer_out += self._buf
                self._buf = ""
                break
            if not self.in_reasoning:
                i = self._buf.find(f.start)
                if i >= 0:
                    answer_out += self._buf[:i]
                    self._buf = self._buf[i + len(f.start):]
                    self.in_reasoning = True
                    continue
                keep = self._partial_suffix(self._buf, f.start)
                answer_out += self._buf[:len(self._buf) - keep]
                self._buf = self._buf[len(self._buf) - keep:]
                break
            # inside the block
            if self._buf.startswith(f.start):
                self._buf = self._buf[len(f.start):]
                continue
            i = self._buf.find(f.end)
            if i >= 0:
                reasoning_out += self._buf[:i]
                self._buf = self._buf[i + len(f.end):]
                self.in_reasoning = False
                self.done = True
                if f.strip_prefix and self._buf.startswith(f.strip_prefix):
                    self._buf = self._buf[len(f.strip_prefix):]
                continue
            keep = max(self._partial_suffix(self._buf, f.end), self._partial_suffix(self._buf, f.start))
            reasoning_out += self._buf[:len(self._buf) - keep]
            self._buf = self._buf[len(self._buf) - keep:]
            break
        if not self.stream_reasoning:
            self._held_reasoning += reasoning_out
            if self.done and self._held_reasoning:
                reasoning_out, self._held_reasoning = self._held_reasoning, ""
            else:
                reasoning_out = ""
        return (reasoning_out or None), answer_out
