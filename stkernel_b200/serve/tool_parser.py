"""DSML tool-call extraction from model output, whole or streamed.

One incremental lexer (`DsmlLexer`) turns text fed in arbitrary pieces into events
(content, invoke open/close, parameter open/text/close, block close); `ToolCallParser`
folds those events into OpenAI tool calls.  The complete-output path feeds the lexer once,
so both paths share one grammar and one coercion rule.  Semantics follow
overlay/tool_parser_deepseekv32.py:

* block markers ``<｜DSML｜function_calls>`` (V3.2) and ``<｜DSML｜tool_calls>`` (V4) are both
  accepted; text before the first block is content (:189-229);
* ``string="true"`` parameters are strings as written; others are coerced by the tool's JSON
  schema type, falling back to JSON then to the raw string (:152-167);
* a lone ``arguments`` / ``input`` parameter that the schema does not declare, holding an
  object whose keys the schema does declare, is unwrapped (:128-150);
* streaming emits the call id/name once, then argument JSON fragments: string parameters as
  they arrive (JSON-escaped), object/array parameters raw, scalars and unions only when
  complete (:350-368, :421-537); a stream never emits a key that the OpenAI wire omits.
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

DSML = "｜DSML｜"
BLOCK_NAMES = ("function_calls", "tool_calls")
# The V4 encoder separates content from the block by a blank line, which belongs to the markup.
BLOCK_OPENS = tuple(f"\n\n<{DSML}{n}>" for n in BLOCK_NAMES) + tuple(f"<{DSML}{n}>" for n in BLOCK_NAMES)
INVOKE_CLOSE = f"</{DSML}invoke>"
PARAM_CLOSE = f"</{DSML}parameter>"
_INVOKE_OPEN = re.compile(rf'<{DSML}invoke\s+name="([^"]+)"\s*>')
_PARAM_OPEN = re.compile(rf'<{DSML}parameter\s+name="([^"]+)"\s+string="(true|false)"\s*>')


def held_back(text: str, tags: Sequence[str]) -> int:
    """Length of the longest suffix of `text` that is a proper prefix of one of `tags`."""
    best = 0
    for tag in tags:
        for k in range(min(len(tag) - 1, len(text)), best, -1):
            if text.endswith(tag[:k]):
                best = k
                break
    return best


# ---------------------------------------------------------------------------------------
# schema helpers
# ---------------------------------------------------------------------------------------
def tool_properties(tools: Optional[Sequence[Dict[str, Any]]], name: Optional[str]) -> Dict[str, Any]:
    for t in tools or ():
        fn = t.get("function", t) if isinstance(t, dict) else {}
        if fn.get("name") == name:
            params = fn.get("parameters") or {}
            props = params.get("properties") if isinstance(params, dict) else None
            return props if isinstance(props, dict) else {}
    return {}


def schema_types(schema: Any) -> List[str]:
    """JSON-schema type names a property admits; "string" when the schema says nothing."""
    if not isinstance(schema, dict):
        return ["string"]
    out: List[str] = []
    t = schema.get("type")
    if isinstance(t, str):
        out.append(t)
    elif isinstance(t, list):
        out.extend(x for x in t if isinstance(x, str))
    for key in ("anyOf", "oneOf"):
        for sub in schema.get(key) or ():
            out.extend(schema_types(sub) if isinstance(sub, dict) and sub else [])
    if not out and "enum" in schema:
        for v in schema["enum"]:
            out.append("null" if v is None else "boolean" if isinstance(v, bool) else "integer" if isinstance(v, int)
                       else "number" if isinstance(v, float) else "string" if isinstance(v, str)
                       else "array" if isinstance(v, list) else "object")
    if not out and ("properties" in schema or "items" in schema):
        out.append("object" if "properties" in schema else "array")
    seen: List[str] = []
    for x in out or ["string"]:
        if x not in seen:
            seen.append(x)
    return seen


def coerce(value: str, types: Sequence[str]) -> Any:
    """A raw parameter body as the first schema type that accepts it; else JSON; else the text."""
    text = value.strip()
    for t in types:
        if t == "null" and text.lower() in ("null", "none", ""):
            return None
        if t == "integer":
            try:
                return int(text)
            except ValueError:
                pass
        if t == "number":
            try:
                f = float(text)
                return int(f) if f.is_integer() and re.fullmatch(r"[+-]?\d+", text) else f
            except ValueError:
                pass
        if t == "boolean" and text.lower() in ("true", "false"):
            return text.lower() == "true"
        if t in ("object", "array"):
            try:
                v = json.loads(text)
                if isinstance(v, dict if t == "object" else list):
                    return v
            except ValueError:
                pass
        if t == "string":
            return value
    try:
        return json.loads(text)
    except ValueError:
        return value


def unwrap(params: Dict[str, Any], props: Dict[str, Any]) -> Dict[str, Any]:
    for wrapper in ("arguments", "input"):
        if set(params) != {wrapper} or wrapper in props:
            continue
        inner = params[wrapper]
        if isinstance(inner, str):
            try:
                inner = json.loads(inner)
            except ValueError:
                return params
        if isinstance(inner, dict) and set(inner) <= set(props):
            return inner
    return params


# ---------------------------------------------------------------------------------------
# lexer
# ---------------------------------------------------------------------------------------
@dataclass
class Event:
    kind: str                   # content | invoke | param | text | param_end | invoke_end | block_end
    a: str = ""
    b: str = ""


class DsmlLexer:
    """Incremental DSML scanner.  `feed` returns the events that the text so far determines;
    an incomplete tag stays buffered until more text arrives."""

    def __init__(self):
        self.buf = ""
        self.state = "content"          # content | block | invoke | param

    def feed(self, text: str) -> List[Event]:
        self.buf += text
        out: List[Event] = []
        while self._advance(out):
            pass
        return out

    def _take(self, n: int) -> str:
        head, self.buf = self.buf[:n], self.buf[n:]
        return head

    def _advance(self, out: List[Event]) -> bool:
        b = self.buf
        if self.state == "content":
            hits = [(b.find(t), t) for t in BLOCK_OPENS if t in b]
            if hits:
                pos, tag = min(hits)
                if pos:
                    out.append(Event("content", self._take(pos)))
                self._take(len(tag))
                self.state = "block"
                return True
            n = len(b) - held_back(b, BLOCK_OPENS)
            if n > 0:
                out.append(Event("content", self._take(n)))
            return False
        if self.state == "param":
            pos = b.find(PARAM_CLOSE)
            if pos >= 0:
                if pos:
                    out.append(Event("text", self._take(pos)))
                self._take(len(PARAM_CLOSE))
                out.append(Event("param_end"))
                self.state = "invoke"
                return True
            n = len(b) - held_back(b, (PARAM_CLOSE,))
            if n > 0:
                out.append(Event("text", self._take(n)))
            return False
        # between tags: whitespace is insignificant
        stripped = b.lstrip()
        if len(stripped) != len(b):
            self.buf = b = stripped
        if self.state == "block":
            for name in BLOCK_NAMES:
                close = f"</{DSML}{name}>"
                if b.startswith(close):
                    self._take(len(close))
                    out.append(Event("block_end"))
                    self.state = "content"
                    return True
            m = _INVOKE_OPEN.match(b)
            if m:
                self._take(m.end())
                out.append(Event("invoke", m.group(1)))
                self.state = "invoke"
                return True
            return False
        if b.startswith(INVOKE_CLOSE):
            self._take(len(INVOKE_CLOSE))
            out.append(Event("invoke_end"))
            self.state = "block"
            return True
        m = _PARAM_OPEN.match(b)
        if m:
            self._take(m.end())
            out.append(Event("param", m.group(1), m.group(2)))
            self.state = "param"
            return True
        return False


# ---------------------------------------------------------------------------------------
# parser
# ---------------------------------------------------------------------------------------
@dataclass
class ToolCallDelta:
    index: int
    id: Optional[str] = None
    name: Optional[str] = None
    arguments: Optional[str] = None

    def to_openai(self) -> Dict[str, Any]:
        fn: Dict[str, Any] = {}
        if self.name is not None:
            fn["name"] = self.name
        if self.arguments is not None:
            fn["arguments"] = self.arguments
        d: Dict[str, Any] = {"index": self.index, "function": fn}
        if self.id is not None:
            d["id"] = self.id
            d["type"] = "function"
        return d


@dataclass
class Delta:
    content: str = ""
    tool_calls: List[ToolCallDelta] = field(default_factory=list)

    def __bool__(self) -> bool:
        return bool(self.content or self.tool_calls)


def new_call_id() -> str:
    return f"call_{uuid.uuid4().hex[:24]}"


def _escape(text: str) -> str:
    return json.dumps(text, ensure_ascii=False)[1:-1]


class ToolCallParser:
    """Streaming state over one response.  `push(delta_text)` returns what can go on the wire."""

    def __init__(self, tools: Optional[Sequence[Dict[str, Any]]] = None):
        self.tools = list(tools or ())
        self.lexer = DsmlLexer()
        self.calls: List[Dict[str, Any]] = []       # {"id", "name", "arguments" (streamed JSON text)}
        self._open = False
        self._mode: Optional[str] = None            # string | raw | held
        self._pname = ""
        self._pstring = ""
        self._held: List[str] = []
        self._started = False
        self._props: Dict[str, Any] = {}

    # -- emit helpers -----------------------------------------------------------------
    def _emit(self, delta: Delta, **kw) -> None:
        idx = len(self.calls) - 1
        args = kw.get("arguments")
        if args:
            self.calls[idx]["arguments"] += args
        for d in delta.tool_calls:
            if d.index == idx:
                for k, v in kw.items():
                    if k == "arguments":
                        d.arguments = (d.arguments or "") + v
                    else:
                        setattr(d, k, v)
                return
        delta.tool_calls.append(ToolCallDelta(index=idx, **kw))

    def _key(self, delta: Delta, key: str, as_string: bool) -> None:
        lead = "," if self._started else "{"
        self._started = True
        self._emit(delta, arguments=lead + json.dumps(key, ensure_ascii=False) + ":" + ('"' if as_string else ""))

    def _convert(self, raw: Dict[str, Tuple[str, str]]) -> Dict[str, Any]:
        vals = {k: (v if s == "true" else coerce(v, schema_types(self._props.get(k, {})))) for k, (v, s) in raw.items()}
        return unwrap(vals, self._props)

    # -- events -----------------------------------------------------------------------
    def _on(self, ev: Event, delta: Delta) -> None:
        if ev.kind == "content":
            delta.content += ev.a
        elif ev.kind == "invoke":
            self.calls.append({"id": new_call_id(), "name": ev.a, "arguments": ""})
            self._open, self._started = True, False
            self._props = tool_properties(self.tools, ev.a)
            self._emit(delta, id=self.calls[-1]["id"], name=ev.a, arguments="")
        elif ev.kind == "param":
            self._pname, self._pstring, self._held = ev.a, ev.b, []
            wrapper = (not self._started and bool(self._props) and ev.a in ("arguments", "input")
                       and ev.a not in self._props)
            if wrapper:
                self._mode = "held"
            elif ev.b == "true":
                self._key(delta, ev.a, True)
                self._mode = "string"
            elif ev.a in self._props and set(schema_types(self._props[ev.a])) <= {"object", "array"}:
                self._key(delta, ev.a, False)
                self._mode = "raw"
            else:
                self._mode = "held"
        elif ev.kind == "text":
            if self._mode == "string":
                self._emit(delta, arguments=_escape(ev.a))
            elif self._mode == "raw":
                self._emit(delta, arguments=ev.a)
            else:
                self._held.append(ev.a)
        elif ev.kind == "param_end":
            if self._mode == "string":
                self._emit(delta, arguments='"')
            elif self._mode == "held":
                for k, v in self._convert({self._pname: ("".join(self._held), self._pstring)}).items():
                    self._key(delta, k, False)
                    self._emit(delta, arguments=json.dumps(v, ensure_ascii=False))
            self._mode = None
        elif ev.kind == "invoke_end":
            self._emit(delta, arguments="}" if self._started else "{}")
            self._open = False

    def push(self, text: str) -> Delta:
        delta = Delta()
        for ev in self.lexer.feed(text):
            self._on(ev, delta)
        return delta

    def flush(self) -> Delta:
        """End of stream: text held back as a possible tag prefix is content after all."""
        delta = Delta()
        if self.lexer.state == "content" and self.lexer.buf:
            delta.content, self.lexer.buf = self.lexer.buf, ""
        return delta

    @property
    def complete_calls(self) -> List[Dict[str, Any]]:
        n = len(self.calls) - (1 if self._open else 0)
        return self.calls[:n]


def extract_tool_calls(text: str, tools: Optional[Sequence[Dict[str, Any]]] = None
                       ) -> Tuple[Optional[str], List[Dict[str, Any]]]:
    """Complete output -> (content before the first block or None, OpenAI tool calls).
    Output without a well-formed call is returned whole as content."""
    if not any(t in text for t in BLOCK_OPENS):
        return text, []
    p = ToolCallParser(tools)
    d = p.push(text)
    calls = []
    for c in p.complete_calls:
        try:
            args = json.dumps(json.loads(c["arguments"]), ensure_ascii=False)
        except ValueError:
            continue
        calls.append({"id": c["id"], "type": "function", "function": {"name": c["name"], "arguments": args}})
    if not calls:
        return text, []
    first = min(text.find(t) for t in BLOCK_OPENS if t in text)
    return (text[:first] if first > 0 else None), calls
