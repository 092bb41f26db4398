"""Reasoning/content separation for DeepSeek-V4 output.

In thinking mode the prompt ends with ``<think>``, so the completion is reasoning up to the
first ``</think>`` and content after it; in chat mode (also reasoning_effort="none", whose
prompt pre-closes the block) everything is content.  Mirrors the delegation in
overlay/reasoning_deepseek_v3.py:20-46 and its thinking-by-default variant (:90-103).  A tool-call
block that opens before ``</think>`` (the model forgot to close its reasoning) ends the reasoning
there, so the call is not lost (overlay/tool_parser_deepseekv32.py:58-62).
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

from .tool_parser import BLOCK_OPENS, held_back

THINK_OPEN = "<think>"
THINK_CLOSE = "</think>"


def thinking_enabled(chat_template_kwargs: Optional[Dict[str, Any]], default: bool = False) -> bool:
    kw = chat_template_kwargs or {}
    if kw.get("reasoning_effort") == "none":
        return False
    t, e = kw.get("thinking"), kw.get("enable_thinking")
    if t is None and e is None:
        return default
    return bool(t) or bool(e)


class ReasoningSplitter:
    """Incremental splitter: `push(text)` -> (reasoning_delta, content_delta)."""

    def __init__(self, thinking: bool, recover_tool_calls: bool = True):
        self.in_reasoning = thinking
        self.buf = ""
        self.at_start = True
        self._stops = (THINK_CLOSE,) + (tuple(BLOCK_OPENS) if recover_tool_calls else ())

    def push(self, text: str) -> Tuple[str, str]:
        if not self.in_reasoning:
            return "", text
        self.buf += text
        if self.at_start:
            if THINK_OPEN.startswith(self.buf):
                return "", ""                               # may still be the echo of the opening tag
            if self.buf.startswith(THINK_OPEN):
                self.buf = self.buf[len(THINK_OPEN):]
            self.at_start = False
        hits = [(self.buf.find(s), s) for s in self._stops if s in self.buf]
        if hits:
            pos, stop = min(hits)
            reasoning = self.buf[:pos]
            rest = self.buf[pos + len(stop):] if stop == THINK_CLOSE else self.buf[pos:]
            self.buf, self.in_reasoning = "", False
            return reasoning, rest
        n = len(self.buf) - held_back(self.buf, self._stops)
        out, self.buf = self.buf[:n], self.buf[n:]
        return out, ""

    def flush(self) -> Tuple[str, str]:
        out, self.buf = self.buf, ""
        return (out, "") if self.in_reasoning else ("", out)


def split_reasoning(text: str, thinking: bool) -> Tuple[Optional[str], Optional[str]]:
    """Complete output -> (reasoning or None, content or None)."""
    s = ReasoningSplitter(thinking)
    r, c = s.push(text)
    r2, c2 = s.flush()
    r, c = r + r2, c + c2
    if not thinking:
        return None, c
    return (r or None), (c or None)
