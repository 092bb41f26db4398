"""Tokenizer front end: chat requests -> prompt token ids with the DeepSeek-V4 encoding.

`ChatTokenizer` wraps any object with `encode(str) -> ids` / `decode(ids) -> str` (a
`tokenizers.Tokenizer`, a transformers tokenizer, or the byte-level stand-in below) and applies
the request-level rules of overlay/tok_deepseek_v4.py:27-84: `thinking`/`enable_thinking`
select thinking mode; tools ride on the leading system message (inserted when absent);
reasoning_effort "none" forces chat mode, "max"/"xhigh" -> max, "high" -> high, anything else
renders no preamble.  `IncrementalDetokenizer` turns a growing id list into text deltas that
never split a multi-byte character.
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

from . import encoding as E

SPECIAL_TOKENS = [E.BOS, E.EOS, E.THINK_OPEN, E.THINK_CLOSE, E.USER, E.ASSISTANT, E.LATEST_REMINDER,
                  E.DSML] + list(E.TASK_TOKENS.values())


def chat_encode_config(kwargs: Dict[str, Any]) -> Dict[str, Any]:
    """Request chat-template kwargs -> arguments of `encode_messages`."""
    thinking = bool(kwargs.get("thinking", False)) or bool(kwargs.get("enable_thinking", False))
    mode = "thinking" if thinking else "chat"
    effort = kwargs.get("reasoning_effort")
    if not isinstance(effort, str):
        effort = None
    elif effort == "none":
        mode, effort = "chat", None
    elif effort in ("max", "xhigh"):
        effort = "max"
    elif effort != "high":
        effort = None
    return {"thinking_mode": mode, "drop_thinking": kwargs.get("drop_thinking", True), "reasoning_effort": effort}


def attach_tools(messages: Sequence[Dict[str, Any]], tools: Optional[Sequence[Dict[str, Any]]]) -> List[Dict[str, Any]]:
    msgs = list(messages)
    if tools:
        if msgs and msgs[0].get("role") == "system":
            msgs[0] = {**msgs[0], "tools": list(tools)}
        else:
            msgs.insert(0, {"role": "system", "tools": list(tools)})
    return msgs


def render_chat(messages: Sequence[Dict[str, Any]], tools: Optional[Sequence[Dict[str, Any]]] = None, **kwargs) -> str:
    return E.encode_messages(attach_tools(messages, tools), **chat_encode_config(kwargs))


class ByteTokenizer:
    """Stand-in vocabulary for tests and random-weight serving: special tokens get ids 0..S-1,
    UTF-8 bytes follow.  Round-trips any string; needs vocab_size >= S + 256."""

    def __init__(self, vocab_size: int = 512):
        self.specials = list(SPECIAL_TOKENS)
        self.base = len(self.specials)
        if vocab_size < self.base + 256:
            raise ValueError(f"vocab_size {vocab_size} < {self.base + 256}")
        self.vocab_size = vocab_size
        self.eos_token_id = self.specials.index(E.EOS)
        self.bos_token_id = self.specials.index(E.BOS)

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        i = 0
        while i < len(text):
            for k, sp in enumerate(self.specials):
                if text.startswith(sp, i):
                    ids.append(k)
                    i += len(sp)
                    break
            else:
                ids.extend(self.base + b for b in text[i].encode("utf-8"))
                i += 1
        return ids

    def decode_bytes(self, ids: Sequence[int]) -> bytes:
        out = bytearray()
        for t in ids:
            if t < self.base:
                out += self.specials[t].encode("utf-8")
            elif t < self.base + 256:
                out.append(t - self.base)
        return bytes(out)

    def decode(self, ids: Sequence[int]) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")


class HFTokenizer:
    """`tokenizers.Tokenizer` loaded from a checkpoint directory's tokenizer.json."""

    def __init__(self, path: str):
        from tokenizers import Tokenizer
        f = os.path.join(path, "tokenizer.json") if os.path.isdir(path) else path
        self.tk = Tokenizer.from_file(f)
        self.vocab_size = self.tk.get_vocab_size(with_added_tokens=True)
        self.eos_token_id = self.tk.token_to_id(E.EOS)
        self.bos_token_id = self.tk.token_to_id(E.BOS)

    def encode(self, text: str) -> List[int]:
        return self.tk.encode(text, add_special_tokens=False).ids

    def decode(self, ids: Sequence[int]) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=False)


class ChatTokenizer:
    def __init__(self, base):
        self.base = base
        self.eos_token_id = getattr(base, "eos_token_id", None)
        self.vocab_size = getattr(base, "vocab_size", None)

    def apply_chat_template(self, messages, tools=None, tokenize: bool = True, max_length: Optional[int] = None, **kwargs):
        prompt = render_chat(messages, tools, **kwargs)
        if not tokenize:
            return prompt
        ids = self.base.encode(prompt)
        return ids[:max_length] if max_length else ids

    def encode(self, text: str) -> List[int]:
        return self.base.encode(text)

    def decode(self, ids: Sequence[int]) -> str:
        return self.base.decode(ids)


class IncrementalDetokenizer:
    """Text deltas from a growing token list.  Decodes a short window before the emitted prefix so
    that merges across token boundaries come out right, and holds back an incomplete UTF-8 tail."""

    WINDOW = 6

    def __init__(self, tokenizer, stop_strings: Sequence[str] = ()):
        self.tk = tokenizer
        self.ids: List[int] = []
        self.prefix_start = 0
        self.read = 0

    def push(self, new_ids: Sequence[int]) -> str:
        self.ids.extend(new_ids)
        old = self.tk.decode(self.ids[self.prefix_start:self.read])
        new = self.tk.decode(self.ids[self.prefix_start:])
        if new.endswith("�") or len(new) <= len(old):
            return ""
        delta = new[len(old):]
        self.read = len(self.ids)
        self.prefix_start = max(self.read - self.WINDOW, 0)
        return delta
