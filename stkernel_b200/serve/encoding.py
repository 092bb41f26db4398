"""DeepSeek-V4 chat encoding: messages -> prompt string, completion text -> assistant message.

The wire format (special tokens, DSML tool-call markup, tool-section text, reasoning-effort
preambles) is the checkpoint's protocol and is reproduced exactly; the implementation is a
small renderer class per concern.  Behaviour follows overlay/tok_deepseek_v4_encoding.py
(render rules :258-436, tool-message merging :443-541, encode :548-615, completion parser
:650-793):

* no standalone tool role: tool results become ``<tool_result>`` blocks of a user turn, ordered
  like the assistant's tool calls;
* thinking mode: earlier assistant turns lose their reasoning unless tools are declared; the
  prompt ends with ``<think>`` (thinking) or ``</think>`` (chat);
* reasoning effort ``high``/``max`` prepends a fixed preamble to the first message;
* quick-instruction "task" tokens for internal classification turns.
"""
from __future__ import annotations

import copy
import json
import re
from typing import Any, Dict, List, Optional, Sequence, Tuple

BOS = "<｜begin▁of▁sentence｜>"
EOS = "<｜end▁of▁sentence｜>"
THINK_OPEN = "<think>"
THINK_CLOSE = "</think>"
DSML = "｜DSML｜"
USER = "<｜User｜>"
ASSISTANT = "<｜Assistant｜>"
LATEST_REMINDER = "<｜latest_reminder｜>"
TASK_TOKENS = {name: f"<｜{name}｜>" for name in ("action", "query", "authority", "domain", "title", "read_url")}
TOOL_CALLS_BLOCK = "tool_calls"

EFFORT_PREAMBLE: Dict[str, str] = {
    "low": "",
    "high": (
        "Reasoning Effort: Absolute maximum with no shortcuts permitted.\n"
        "You MUST be very thorough in your thinking and comprehensively decompose the problem to resolve the root "
        "cause, rigorously stress-testing your logic against all potential paths, edge cases, and adversarial "
        "scenarios.\n"
        "Explicitly write out your entire deliberation process, documenting every intermediate step, considered "
        "alternative, and rejected hypothesis to ensure absolutely no assumption is left unchecked.\n\n"
    ),
    "max": (
        "Reasoning Effort: Beyond maximum — exhaustive, relentless, and uncompromising.\n"
        "You MUST reason with the utmost depth and rigor, leaving absolutely nothing to chance: exhaustively "
        "decompose the problem into its most fundamental components, trace every causal chain to its root, and "
        "resolve the underlying cause rather than any surface symptom.\n"
        "Do not stop reasoning until you have independently verified the solution from multiple angles and are "
        "certain that no assumption remains unchecked and no error remains undiscovered.\n\n"
    ),
}

_TOOLS_SECTION = (
    "## Tools\n\n"
    "You have access to a set of tools to help answer the user's question. You can invoke tools by writing a "
    "\"<{d}tool_calls>\" block like the following:\n\n"
    "<{d}tool_calls>\n"
    "<{d}invoke name=\"$TOOL_NAME\">\n"
    "<{d}parameter name=\"$PARAMETER_NAME\" string=\"true|false\">$PARAMETER_VALUE</{d}parameter>\n"
    "...\n"
    "</{d}invoke>\n"
    "<{d}invoke name=\"$TOOL_NAME2\">\n"
    "...\n"
    "</{d}invoke>\n"
    "</{d}tool_calls>\n\n"
    "String parameters should be specified as is and set `string=\"true\"`. For all other types (numbers, booleans, "
    "arrays, objects), pass the value in JSON format and set `string=\"false\"`.\n\n"
    "If thinking_mode is enabled (triggered by {to}), you MUST output your complete reasoning inside {to}...{tc} "
    "BEFORE any tool calls or final response.\n\n"
    "Otherwise, output directly after {tc} with tool calls or final response.\n\n"
    "### Available Tool Schemas\n\n"
    "{schemas}\n\n"
    "You MUST strictly follow the above defined tool name and parameter schemas to invoke tool calls.\n"
)
_RESPONSE_FORMAT = "## Response Format:\n\nYou MUST strictly adhere to the following schema to reply:\n{schema}"


def dumps(value: Any) -> str:
    try:
        return json.dumps(value, ensure_ascii=False)
    except Exception:
        return json.dumps(value, ensure_ascii=True)


# ---------------------------------------------------------------------------------------
# tool calls <-> DSML
# ---------------------------------------------------------------------------------------
def _call_arguments(arguments: Any) -> Dict[str, Any]:
    """Arguments of a tool call as a dict; anything that is not a JSON object is wrapped as
    {"arguments": original} so that resent histories with "" or "null" still encode."""
    raw = arguments
    if isinstance(arguments, str):
        try:
            arguments = json.loads(arguments)
        except Exception:
            return {"arguments": raw}
    if not isinstance(arguments, dict):
        return {"arguments": raw if isinstance(raw, str) else dumps(arguments)}
    return arguments


def dsml_parameters(arguments: Any) -> str:
    lines = []
    for key, val in _call_arguments(arguments).items():
        is_str = isinstance(val, str)
        lines.append(f'<{DSML}parameter name="{key}" string="{"true" if is_str else "false"}">'
                     f'{val if is_str else dumps(val)}</{DSML}parameter>')
    return "\n".join(lines)


def dsml_tool_calls(tool_calls: Sequence[Dict[str, Any]]) -> str:
    """OpenAI-format tool calls -> the DSML block that follows an assistant turn's content."""
    invokes = []
    for tc in tool_calls:
        fn = tc["function"]
        invokes.append(f'<{DSML}invoke name="{fn["name"]}">\n{dsml_parameters(fn["arguments"])}\n</{DSML}invoke>')
    body = "\n".join(invokes)
    return f"\n\n<{DSML}{TOOL_CALLS_BLOCK}>\n{body}\n</{DSML}{TOOL_CALLS_BLOCK}>"


def tools_section(tools: Sequence[Dict[str, Any]]) -> str:
    schemas = "\n".join(dumps(t["function"]) for t in tools)
    return _TOOLS_SECTION.format(d=DSML, to=THINK_OPEN, tc=THINK_CLOSE, schemas=schemas)


# ---------------------------------------------------------------------------------------
# preprocessing
# ---------------------------------------------------------------------------------------
def merge_tool_messages(messages: Sequence[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """role=tool messages (and adjacent user text) fold into user turns made of content blocks."""
    out: List[Dict[str, Any]] = []
    for m in messages:
        m = copy.deepcopy(m)
        role = m.get("role")
        prev = out[-1] if out else None
        prev_is_block_user = prev is not None and prev.get("role") == "user" and "content_blocks" in prev
        if role == "tool":
            block = {"type": "tool_result", "tool_use_id": m.get("tool_call_id", ""), "content": m.get("content", "")}
            if prev_is_block_user:
                prev["content_blocks"].append(block)
            else:
                out.append({"role": "user", "content_blocks": [block]})
        elif role == "user":
            block = {"type": "text", "text": m.get("content", "")}
            if prev_is_block_user and prev.get("task") is None:
                prev["content_blocks"].append(block)
            else:
                new = {"role": "user", "content": m.get("content", ""), "content_blocks": [block]}
                for key in ("task", "wo_eos", "mask"):
                    if key in m:
                        new[key] = m[key]
                out.append(new)
        else:
            out.append(m)
    return out


def order_tool_results(messages: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """Within a user turn, tool_result blocks follow the order of the preceding assistant's calls."""
    order: Dict[str, int] = {}
    for m in messages:
        role = m.get("role")
        if role == "assistant" and m.get("tool_calls"):
            order = {}
            for i, tc in enumerate(m["tool_calls"]):
                cid = tc.get("id") or tc.get("function", {}).get("id", "")
                if cid:
                    order[cid] = i
        elif role == "user" and m.get("content_blocks"):
            results = [b for b in m["content_blocks"] if b.get("type") == "tool_result"]
            if len(results) > 1 and order:
                ranked = iter(sorted(results, key=lambda b: order.get(b.get("tool_use_id", ""), 0)))
                m["content_blocks"] = [next(ranked) if b.get("type") == "tool_result" else b for b in m["content_blocks"]]
    return messages


def last_user_index(messages: Sequence[Dict[str, Any]]) -> int:
    for i in range(len(messages) - 1, -1, -1):
        if messages[i].get("role") in ("user", "developer"):
            return i
    return -1


def strip_old_reasoning(messages: Sequence[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """Before the last user turn: assistants lose their reasoning, developer turns disappear."""
    last = last_user_index(messages)
    keep_roles = {"user", "system", "tool", "latest_reminder", "direct_search_results"}
    out = []
    for i, m in enumerate(messages):
        role = m.get("role")
        if role in keep_roles or i >= last:
            out.append(m)
        elif role == "assistant":
            m = copy.copy(m)
            m.pop("reasoning", None)
            m.pop("reasoning_content", None)
            out.append(m)
    return out


# ---------------------------------------------------------------------------------------
# rendering
# ---------------------------------------------------------------------------------------
class Renderer:
    def __init__(self, messages: List[Dict[str, Any]], thinking_mode: str, drop_thinking: bool, effort: Optional[str]):
        if thinking_mode not in ("chat", "thinking"):
            raise ValueError(f"Invalid thinking_mode `{thinking_mode}`")
        effort = effort or "low"
        if effort not in EFFORT_PREAMBLE:
            raise ValueError(f"Invalid reasoning effort: {effort}, expected one of {list(EFFORT_PREAMBLE)}")
        self.messages = messages
        self.thinking = thinking_mode == "thinking"
        self.drop_thinking = drop_thinking
        self.effort = effort
        self.last_user = last_user_index(messages)

    # -- per-role bodies ---------------------------------------------------------
    def _extras(self, m: Dict[str, Any]) -> str:
        out = ""
        if m.get("tools"):
            out += "\n\n" + tools_section(m["tools"])
        if m.get("response_format"):
            out += "\n\n" + _RESPONSE_FORMAT.format(schema=dumps(m["response_format"]))
        return out

    def _user_body(self, m: Dict[str, Any]) -> str:
        blocks = m.get("content_blocks")
        if not blocks:
            return m.get("content") or ""
        parts = []
        for b in blocks:
            kind = b.get("type")
            if kind == "text":
                parts.append(b.get("text", ""))
            elif kind == "tool_result":
                content = b.get("content", "")
                if isinstance(content, list):
                    content = "\n\n".join(c.get("text", "") if c.get("type") == "text" else f"[Unsupported {c.get('type')}]"
                                          for c in content)
                parts.append(f"<tool_result>{content}</tool_result>")
            else:
                parts.append(f"[Unsupported {kind}]")
        return "\n\n".join(parts)

    def _assistant_body(self, i: int, m: Dict[str, Any]) -> str:
        reasoning = m.get("reasoning")
        if reasoning is None:
            reasoning = m.get("reasoning_content")
        after_task = i >= 1 and self.messages[i - 1].get("task") is not None
        think = ""
        if self.thinking and not after_task and (not self.drop_thinking or i > self.last_user):
            think = (reasoning or "") + THINK_CLOSE
        calls = dsml_tool_calls(m["tool_calls"]) if m.get("tool_calls") else ""
        return think + (m.get("content") or "") + calls + ("" if m.get("wo_eos", False) else EOS)

    # -- one message -------------------------------------------------------------------
    def render(self, i: int) -> str:
        m = self.messages[i]
        role = m.get("role")
        out = EFFORT_PREAMBLE[self.effort] if (i == 0 and self.thinking) else ""
        if role == "system":
            out += (m.get("content") or "") + self._extras(m)
        elif role == "developer":
            if not m.get("content"):
                raise ValueError(f"Invalid message for role `{role}`: {m}")
            out += USER + m["content"] + self._extras(m)
        elif role == "user":
            out += USER + self._user_body(m)
        elif role == "latest_reminder":
            out += LATEST_REMINDER + str(m.get("content"))
        elif role == "assistant":
            out += self._assistant_body(i, m)
        elif role == "tool":
            raise NotImplementedError("tool messages must be merged into user turns first (merge_tool_messages)")
        else:
            raise NotImplementedError(f"Unknown role: {role}")

        # what follows decides whether the generation prefix is appended
        nxt = self.messages[i + 1].get("role") if i + 1 < len(self.messages) else None
        if nxt is not None and nxt not in ("assistant", "latest_reminder"):
            return out
        task = m.get("task")
        if task is not None:
            if task not in TASK_TOKENS:
                raise ValueError(f"Invalid task: '{task}'. Valid tasks are: {list(TASK_TOKENS)}")
            if task == "action":
                out += ASSISTANT + (THINK_OPEN if self.thinking else THINK_CLOSE) + TASK_TOKENS[task]
            else:
                out += TASK_TOKENS[task]
        elif role in ("user", "developer"):
            opens = self.thinking and (not self.drop_thinking or i >= self.last_user)
            out += ASSISTANT + (THINK_OPEN if opens else THINK_CLOSE)
        return out


def encode_messages(messages: Sequence[Dict[str, Any]], thinking_mode: str,
                    context: Optional[Sequence[Dict[str, Any]]] = None, drop_thinking: bool = True,
                    add_default_bos_token: bool = True, reasoning_effort: Optional[str] = None) -> str:
    """Encode `messages` (continuing an already-encoded `context`, if any) into the prompt string."""
    context = list(context) if context else []
    new = merge_tool_messages(messages)
    new = order_tool_results(context + new)[len(context):]
    if context:
        context = order_tool_results(merge_tool_messages(context))
    full = context + new
    prompt = BOS if (add_default_bos_token and not context) else ""
    drop = drop_thinking and not any(m.get("tools") for m in full)
    if thinking_mode == "thinking" and drop:
        full = strip_old_reasoning(full)
        n_render = len(full) - len(strip_old_reasoning(context))
    else:
        n_render = len(new)
    first = len(full) - n_render
    r = Renderer(full, thinking_mode, drop, reasoning_effort)
    for i in range(first, len(full)):
        prompt += r.render(i)
    return prompt


# ---------------------------------------------------------------------------------------
# completion parsing
# ---------------------------------------------------------------------------------------
def _scan(text: str, start: int, stops: Sequence[str]) -> Tuple[int, str, Optional[str]]:
    """Text from `start` up to the earliest stop string -> (index after the stop, text, stop or None)."""
    best, which = len(text), None
    for s in stops:
        p = text.find(s, start)
        if p != -1 and p < best:
            best, which = p, s
    if which is None:
        return len(text), text[start:], None
    return best + len(which), text[start:best], which


_INVOKE_NAME = re.compile(r'^\s*name="(.*?)">\n$', re.DOTALL)
_PARAM = re.compile(r'^ name="(.*?)" string="(true|false)">(.*?)<$', re.DOTALL)


def parse_tool_calls(index: int, text: str) -> Tuple[int, Optional[str], List[Dict[str, str]]]:
    """Parse the body of a DSML tool_calls block starting right after its opening tag name."""
    close_block = f"</{DSML}{TOOL_CALLS_BLOCK}>"
    open_invoke, close_invoke = f"<{DSML}invoke", f"</{DSML}invoke"
    open_param, close_param = f"<{DSML}parameter", f"/{DSML}parameter"
    calls: List[Dict[str, str]] = []
    stop = None
    while index < len(text):
        index, gap, stop = _scan(text, index, [open_invoke, close_block])
        if gap != ">\n":
            raise ValueError(f"Tool call format error: expected '>\\n' but got '{gap}'")
        if stop == close_block:
            break
        if stop is None:
            raise ValueError("Missing special token in tool calls")
        index, head, stop = _scan(text, index, [open_param, close_invoke])
        names = _INVOKE_NAME.findall(head)
        if len(names) != 1:
            raise ValueError(f"Tool name format error: '{head}'")
        args: Dict[str, Tuple[str, str]] = {}
        while stop == open_param:
            index, body, stop = _scan(text, index, [close_param])
            found = _PARAM.findall(body)
            if len(found) != 1:
                raise ValueError(f"Parameter format error: '{body}'")
            pname, is_str, pval = found[0]
            if pname in args:
                raise ValueError(f"Duplicate parameter name: '{pname}'")
            args[pname] = (pval, is_str)
            index, gap, stop = _scan(text, index, [open_param, close_invoke])
            if gap != ">\n":
                raise ValueError(f"Parameter format error: expected '>\\n' but got '{gap}'")
        fields = ", ".join(f"{dumps(k)}: {dumps(v) if s == 'true' else v}" for k, (v, s) in args.items())
        calls.append({"name": names[0], "arguments": "{" + fields + "}"})
    return index, stop, calls


def parse_message_from_completion_text(text: str, thinking_mode: str) -> Dict[str, Any]:
    """One assistant turn of raw model output (with its EOS) -> {role, content, reasoning, tool_calls}.
    Raises ValueError on malformed output."""
    open_calls = f"\n\n<{DSML}{TOOL_CALLS_BLOCK}"
    index, reasoning = 0, ""
    if thinking_mode == "thinking":
        index, reasoning, stop = _scan(text, index, [THINK_CLOSE, open_calls])
        if stop != THINK_CLOSE:
            raise ValueError("Invalid thinking format: missing </think>")
    index, content, stop = _scan(text, index, [EOS, open_calls])
    calls: List[Dict[str, str]] = []
    if stop == open_calls:
        index, stop, calls = parse_tool_calls(index, text)
        index, tail, stop = _scan(text, index, [EOS])
        if tail:
            raise ValueError("Unexpected content after tool calls")
    elif stop != EOS:
        raise ValueError("Invalid format: missing EOS token")
    if index != len(text) or stop not in (EOS, None):
        raise ValueError("Unexpected content at end")
    for tok in (BOS, EOS, THINK_OPEN, THINK_CLOSE, DSML):
        if tok in content or tok in reasoning:
            raise ValueError(f"Unexpected special token '{tok}' in content")
    return {"role": "assistant", "content": content, "reasoning": reasoning,
            "tool_calls": [{"type": "function", "function": {"name": c["name"], "arguments": c["arguments"]}} for c in calls]}
