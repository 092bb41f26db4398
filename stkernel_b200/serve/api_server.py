"""HTTP front end: OpenAI chat/completions, Anthropic messages, metrics, profiling, cache reset.

The endpoints are the ones the reference's launcher, supervisor and bench clients use
(launchers/start-hy4-tp4.sh:354-392 serve flags; launchers/dsv4-tp4-supervisor.sh:45-54,117-132
health probe and prefix-cache reset; bench/bench-dec.py:60-119 `/metrics`; bench/profile-step.py:49-57
`/start_profile` + `/stop_profile`; bench/bench-ctx.py:28-82 streaming with usage):

    GET  /health, /v1/models, /metrics
    POST /v1/chat/completions   (stream or not; stream_options.include_usage; tools; thinking kwargs; n choices)
    POST /v1/completions        (raw prompt or token ids)
    POST /v1/messages           (Anthropic wire: text / thinking / tool_use blocks, SSE events)
    POST /v1/messages/count_tokens, /tokenize, /detokenize
    POST /start_profile, /stop_profile, /reset_prefix_cache

`AsyncEngine` owns the engine on one worker thread (the thread that owns the CUDA context and
replays the decode graphs); HTTP handlers talk to it through thread-safe queues, so a slow client
never stalls a step.
"""
from __future__ import annotations

import asyncio
import dataclasses
import json
import queue
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, AsyncIterator, Dict, List, Optional, Sequence, Tuple

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..runtime.engine import Engine, SamplingParams
from .reasoning import ReasoningSplitter, thinking_enabled
from .tokenizer import ChatTokenizer, IncrementalDetokenizer
from .tool_parser import ToolCallParser, BLOCK_OPENS


# ---------------------------------------------------------------------------------------
# engine driver
# ---------------------------------------------------------------------------------------
@dataclass
class TokenEvent:
    tokens: List[int]
    finished: bool
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    logprobs: Optional[List[Any]] = None          # per token: (log-probability, [(id, log-probability), ...]) when asked for


class AsyncEngine:
    """Runs `engine.step()` on a worker thread; per-request asyncio queues carry the tokens out."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self._inbox: "queue.Queue[Tuple[str, Any]]" = queue.Queue()
        self._streams: Dict[int, Tuple[asyncio.AbstractEventLoop, asyncio.Queue]] = {}
        self._wake = threading.Event()
        self._stop = False
        self._profiler = None
        self.last_trace: Optional[str] = None
        self._thread = threading.Thread(target=self._run, name="stk-engine", daemon=True)
        self._thread.start()

    # -- worker thread --------------------------------------------------------------------
    def _post(self, rid: int, ev: TokenEvent) -> None:
        target = self._streams.get(rid)
        if target is not None:
            loop, q = target
            loop.call_soon_threadsafe(q.put_nowait, ev)

    def _drain_inbox(self) -> None:
        while True:
            try:
                kind, payload = self._inbox.get_nowait()
            except queue.Empty:
                return
            if kind == "add":
                prompt, params, loop, q, fut = payload
                try:
                    rid = self.engine.add_request(prompt, params)
                    self._streams[rid] = (loop, q)
                    self._on_add(rid, prompt, params)
                    loop.call_soon_threadsafe(fut.set_result, rid)
                except Exception as e:                       # rejected request (too long, ...)
                    loop.call_soon_threadsafe(fut.set_exception, e)
            elif kind == "abort":
                if self.engine.abort(payload):
                    self._on_abort(payload)
                    self._post(payload, TokenEvent([], True, "abort"))
                self._streams.pop(payload, None)
                self.engine.release(payload)
            elif kind == "call":
                fn, loop, fut = payload
                try:
                    res = fn()
                    loop.call_soon_threadsafe(fut.set_result, res)
                except Exception as e:
                    loop.call_soon_threadsafe(fut.set_exception, e)

    def _publish(self, produced: Sequence[Tuple[int, int]]) -> None:
        """One event per request and step: a speculative step yields several tokens for a request, and the finished flag
        must arrive with the last of them, not the first."""
        eng = self.engine
        by_req: Dict[int, List[int]] = {}
        for rid, tok in produced:
            by_req.setdefault(rid, []).append(tok)
        for rid, toks in by_req.items():
            r = eng.requests.get(rid)
            done = r is not None and r.finished
            lps = None
            if r is not None and getattr(r.params, "logprobs", None) is not None:
                lps = list(getattr(r, "logprobs", [])[-len(toks):])
            self._post(rid, TokenEvent(toks, done, r.finish_reason if done else None, logprobs=lps))
            if done:
                self._streams.pop(rid, None)
                eng.release(rid)

    def _on_add(self, rid: int, prompt: List[int], params: SamplingParams) -> None:
        """Hook: a request entered the engine (multi-rank leaders mirror it to the followers)."""

    def _on_abort(self, rid: int) -> None:
        """Hook: a live request was aborted."""

    def _run(self) -> None:
        eng = self.engine
        while not self._stop:
            self._drain_inbox()
            if not eng.has_work():
                self._wake.wait(timeout=0.05)
                self._wake.clear()
                continue
            try:
                self._publish(eng.step())
            except Exception as e:                           # a failed step fails every open stream; the loop lives on
                for rid in list(self._streams):
                    self._post(rid, TokenEvent([], True, "error", error=f"{type(e).__name__}: {e}"))
                    eng.abort(rid)
                self._streams.clear()
                continue

    # -- asyncio side ------------------------------------------------------------------------
    async def generate(self, prompt: Sequence[int], params: SamplingParams) -> AsyncIterator[TokenEvent]:
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        fut = loop.create_future()
        self._inbox.put(("add", (list(prompt), params, loop, q, fut)))
        self._wake.set()
        rid = await fut
        try:
            while True:
                ev = await q.get()
                yield ev
                if ev.finished:
                    return
        finally:
            self._inbox.put(("abort", rid))                    # no-op for a finished request
            self._wake.set()

    async def call(self, fn):
        """Run `fn()` on the engine thread between steps."""
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        self._inbox.put(("call", (fn, loop, fut)))
        self._wake.set()
        return await fut

    def shutdown(self) -> None:
        self._stop = True
        self._wake.set()
        self._thread.join(timeout=5)

    # -- profiling (engine thread) ---------------------------------------------------------
    def start_profile(self, out_dir: str) -> str:
        import torch
        if self._profiler is not None:
            return "already running"
        acts = [torch.profiler.ProfilerActivity.CPU]
        if self.engine.device.type == "cuda":
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._profiler = torch.profiler.profile(activities=acts)
        self._profiler.__enter__()
        self._profile_dir = out_dir
        return "started"

    def stop_profile(self) -> Optional[str]:
        import os
        if self._profiler is None:
            return None
        self._profiler.__exit__(None, None, None)
        os.makedirs(self._profile_dir, exist_ok=True)
        path = os.path.join(self._profile_dir, f"trace_{int(time.time())}.json")
        self._profiler.export_chrome_trace(path)
        self._profiler = None
        self.last_trace = path
        return path

    def reset_prefix_cache(self) -> bool:
        """Only when idle, as the supervisor's daily reset expects."""
        if self.engine.has_work():
            return False
        reset = getattr(self.engine, "reset_prefix_cache", None)
        if reset is not None:
            reset()
        self.engine.metrics.prefix_cache_resets += 1
        return True


# ---------------------------------------------------------------------------------------
# response assembly
# ---------------------------------------------------------------------------------------
@dataclass
class Piece:
    reasoning: str = ""
    content: str = ""
    tool_calls: list = field(default_factory=list)      # ToolCallDelta

    def __bool__(self) -> bool:
        return bool(self.reasoning or self.content or self.tool_calls)


class OutputPipeline:
    """tokens -> text -> (reasoning | content | tool-call deltas), with stop strings."""

    def __init__(self, tok: ChatTokenizer, thinking: bool, tools: Optional[list], stop: Sequence[str] = (),
                 parse_tools: bool = True, primed: str = ""):
        """primed: text that the prompt already ends with as the beginning of the answer (a demanded tool call's
        opening); the parsers see it in front of what the model generates."""
        self.detok = IncrementalDetokenizer(tok)
        self.split = ReasoningSplitter(thinking)
        self.tools = ToolCallParser(tools) if (tools and parse_tools) else None
        self.stop = [s for s in stop if s]
        self.text = ""
        self.stopped = False
        self._pending = ""
        self._primed = primed

    def _route(self, text: str, final: bool) -> Piece:
        r, c = self.split.push(text) if text else ("", "")
        if final:
            r2, c2 = self.split.flush()
            r, c = r + r2, c + c2
        p = Piece(reasoning=r)
        if self.tools is None:
            p.content = c
        else:
            d = self.tools.push(c) if c else None
            if d:
                p.content, p.tool_calls = d.content, d.tool_calls
            if final:
                p.content += self.tools.flush().content
        return p

    def push(self, token_ids: Sequence[int], final: bool, eos_id: Optional[int] = None) -> Piece:
        ids = [t for t in token_ids if t != eos_id]
        text = self._primed + self._pending + self.detok.push(ids)
        self._pending = self._primed = ""
        if self.stop and text:
            hit = min((text.find(s) for s in self.stop if s in text), default=-1)
            if hit >= 0:
                text, self.stopped, final = text[:hit], True, True
            elif not final:
                from .tool_parser import held_back
                k = held_back(text, self.stop)
                if k:
                    text, self._pending = text[:-k], text[-k:]
        self.text += text
        return self._route(text, final)

    @property
    def has_tool_calls(self) -> bool:
        return self.tools is not None and bool(self.tools.complete_calls)


def _usage(n_prompt: int, n_out: int) -> Dict[str, int]:
    return {"prompt_tokens": n_prompt, "completion_tokens": n_out, "total_tokens": n_prompt + n_out}


def flatten_content_parts(messages: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """OpenAI content-part arrays (`"content": [{"type": "text", "text": ...}, ...]`) -> plain strings, text parts joined
    by newlines; any other part type is a 400 (the model reads text only)."""
    out = []
    for m in messages:
        c = m.get("content")
        if isinstance(c, list):
            texts = []
            for part in c:
                kind = part.get("type") if isinstance(part, dict) else None
                if kind not in ("text", "input_text"):
                    raise HTTPException(status_code=400, detail=f"unsupported content part type {kind!r}")
                texts.append(part.get("text", ""))
            m = {**m, "content": "\n".join(texts)}
        out.append(m)
    return out


def forced_tool_prefix(tool_choice: Any, tools: Optional[List[Dict[str, Any]]]) -> Optional[str]:
    """OpenAI `tool_choice` -> the text a demanded call starts with, or None when the model is free to choose
    ("auto", "none", absent).  "required" opens the tool-call block and the first invoke's name attribute; a named
    function also fixes the name.  (The reference leaves both unenforced: SERVING_SURFACE_AUDIT.md:80-95.)"""
    from .encoding import DSML, TOOL_CALLS_BLOCK
    if tool_choice in (None, "auto", "none"):
        return None
    name = None
    if isinstance(tool_choice, dict):
        name = (tool_choice.get("function") or {}).get("name") or tool_choice.get("name")
        if not name:
            raise HTTPException(status_code=400, detail="tool_choice names no function")
    elif tool_choice not in ("required", "any"):
        raise HTTPException(status_code=400, detail=f"unsupported tool_choice {tool_choice!r}")
    known = [t.get("function", {}).get("name") for t in (tools or [])]
    if not known:
        raise HTTPException(status_code=400, detail="tool_choice demands a call but the request has no tools")
    if name is not None and name not in known:
        raise HTTPException(status_code=400, detail=f"tool_choice names {name!r}, which is not among the tools")
    head = f'\n\n<{DSML}{TOOL_CALLS_BLOCK}>\n<{DSML}invoke name="'
    return head + (f'{name}">\n' if name is not None else "")


def logprob_entries(tokenizer, tokens: Sequence[int], lps: Optional[Sequence[Any]]) -> List[Dict[str, Any]]:
    """OpenAI chat `logprobs.content` entries for the tokens of one event."""
    def one(tid: int, lp: float) -> Dict[str, Any]:
        text = tokenizer.decode([int(tid)])
        return {"token": text, "logprob": float(lp), "bytes": list(text.encode("utf-8"))}
    out = []
    for tid, (lp, top) in zip(tokens, lps or []):
        out.append({**one(tid, lp), "top_logprobs": [one(i, v) for i, v in top]})
    return out


def parse_stop(value: Any) -> List[str]:
    if value is None:
        return []
    if isinstance(value, str):
        return [value] if value else []
    if isinstance(value, list) and all(isinstance(x, str) for x in value):
        return [x for x in value if x]
    raise HTTPException(status_code=400, detail="stop must be a string or a list of strings")


def want_usage(body: Dict[str, Any]) -> bool:
    so = body.get("stream_options")
    return isinstance(so, dict) and bool(so.get("include_usage"))


def choice_count(body: Dict[str, Any], limit: int = 16) -> int:
    n = body.get("n", 1)
    if not isinstance(n, int) or isinstance(n, bool) or not 1 <= n <= limit:
        raise HTTPException(status_code=400, detail=f"n must be an integer in [1, {limit}]")
    return n


def attach_response_format(messages: List[Dict[str, Any]], rf: Optional[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """OpenAI `response_format` -> the schema block of the leading system message, which the chat encoding renders
    (overlay/tok_deepseek_v4_encoding.py:258-436 takes it from the message): `json_schema` passes its schema,
    `json_object` asks for any JSON object, `text` (or nothing) leaves the prompt alone.  The output is steered by the
    prompt, as in the reference's serving surface; it is not grammar-constrained."""
    if not rf or rf.get("type") in (None, "text"):
        return list(messages)
    kind = rf.get("type")
    if kind == "json_object":
        schema: Any = {"type": "object"}
    elif kind == "json_schema":
        js = rf.get("json_schema") or {}
        schema = js.get("schema", js)
        if not isinstance(schema, dict) or not schema:
            raise HTTPException(status_code=400, detail="response_format.json_schema.schema must be a non-empty object")
    else:
        raise HTTPException(status_code=400, detail=f"unsupported response_format type {kind!r}")
    msgs = list(messages)
    if msgs and msgs[0].get("role") == "system":
        msgs[0] = {**msgs[0], "response_format": schema}
    else:
        msgs.insert(0, {"role": "system", "content": "", "response_format": schema})
    return msgs


def sampling_from_request(body: Dict[str, Any], eos_id: Optional[int], max_model_len: int, n_prompt: int,
                          default_max: int = 512, default_temperature: float = 1.0) -> SamplingParams:
    try:
        return _sampling_from_request(body, eos_id, max_model_len, n_prompt, default_max, default_temperature)
    except HTTPException:
        raise
    except (TypeError, ValueError, OverflowError) as e:
        raise HTTPException(status_code=400, detail=f"bad sampling parameter: {type(e).__name__}: {e}") from None


def _sampling_from_request(body: Dict[str, Any], eos_id: Optional[int], max_model_len: int, n_prompt: int,
                           default_max: int, default_temperature: float) -> SamplingParams:
    max_tokens = body.get("max_completion_tokens") or body.get("max_tokens") or default_max
    max_tokens = max(1, min(int(max_tokens), max_model_len - n_prompt))
    seed = body.get("seed")
    temp = body.get("temperature")
    top_p = body.get("top_p")
    top_k = body.get("top_k")
    top_p = 1.0 if top_p is None else float(top_p)
    top_k = 0 if top_k is None else int(top_k)
    if not (0.0 < top_p <= 1.0):
        raise HTTPException(status_code=400, detail="top_p must be in (0, 1]")
    if top_k < -1:
        raise HTTPException(status_code=400, detail="top_k must be -1 (off), 0 (off) or positive")
    want_lp = None
    if body.get("logprobs") not in (None, False):
        # chat: `logprobs: true` + `top_logprobs: n`; raw completions: `logprobs: n`
        n_top = body.get("top_logprobs") if isinstance(body.get("logprobs"), bool) else body.get("logprobs")
        want_lp = int(n_top or 0)
        if not 0 <= want_lp <= 20:
            raise HTTPException(status_code=400, detail="top_logprobs must be in [0, 20]")
    return SamplingParams(logprobs=want_lp, temperature=float(default_temperature if temp is None else temp),
                          seed=int(seed) if seed is not None else uuid.uuid4().int & 0x7FFFFFFF,
                          max_tokens=max_tokens, min_tokens=int(body.get("min_tokens", 0) or 0),
                          ignore_eos=bool(body.get("ignore_eos", False)), eos_token_id=eos_id,
                          top_k=max(top_k, 0), top_p=top_p)


def anthropic_to_chat(body: Dict[str, Any]) -> Tuple[List[Dict[str, Any]], Optional[List[Dict[str, Any]]]]:
    """Anthropic /v1/messages request -> chat messages + OpenAI-format tools."""
    msgs: List[Dict[str, Any]] = []
    system = body.get("system")
    if isinstance(system, list):
        system = "\n\n".join(b.get("text", "") for b in system if b.get("type") == "text")
    if system:
        msgs.append({"role": "system", "content": system})
    for m in body.get("messages", []):
        role, content = m.get("role"), m.get("content")
        if isinstance(content, str):
            msgs.append({"role": role, "content": content})
            continue
        text, reasoning, calls = [], [], []
        for b in content or []:
            kind = b.get("type")
            if kind == "text":
                text.append(b.get("text", ""))
            elif kind == "thinking":
                reasoning.append(b.get("thinking", ""))
            elif kind == "tool_use":
                calls.append({"id": b.get("id", ""), "type": "function",
                              "function": {"name": b.get("name", ""), "arguments": json.dumps(b.get("input", {}), ensure_ascii=False)}})
            elif kind == "tool_result":
                if text:
                    msgs.append({"role": role, "content": "\n\n".join(text)})
                    text = []
                c = b.get("content", "")
                msgs.append({"role": "tool", "tool_call_id": b.get("tool_use_id", ""), "content": c})
        if role == "assistant":
            a: Dict[str, Any] = {"role": "assistant", "content": "\n\n".join(text)}
            if reasoning:
                a["reasoning"] = "\n\n".join(reasoning)
            if calls:
                a["tool_calls"] = calls
            msgs.append(a)
        elif text:
            msgs.append({"role": role, "content": "\n\n".join(text)})
    tools = None
    if body.get("tools"):
        tools = [{"type": "function", "function": {"name": t.get("name"), "description": t.get("description", ""),
                                                    "parameters": t.get("input_schema", {})}} for t in body["tools"]]
    return msgs, tools


# ---------------------------------------------------------------------------------------
# the app
# ---------------------------------------------------------------------------------------
def create_app(engine: Engine, tokenizer: ChatTokenizer, model_name: str = "deepseek-v4-flash",
               default_thinking: bool = False, profile_dir: str = "/tmp/stk_profiles",
               default_chat_template_kwargs: Optional[Dict[str, Any]] = None, async_engine: Optional[AsyncEngine] = None,
               default_temperature: float = 1.0):
    app = FastAPI(title="stkernel_b200")
    aeng = async_engine if async_engine is not None else AsyncEngine(engine)
    app.state.async_engine = aeng
    max_len = engine.cfg.sched.max_model_len
    eos_id = tokenizer.eos_token_id
    created = int(time.time())
    base_kwargs = dict(default_chat_template_kwargs or {})

    def err(status: int, msg: str, kind: str = "invalid_request_error"):
        return JSONResponse({"error": {"message": msg, "type": kind, "code": status}}, status_code=status)

    @app.exception_handler(HTTPException)
    async def http_error(request: Request, exc: HTTPException):
        return err(exc.status_code, str(exc.detail))

    def refuse_logprobs(params: SamplingParams):
        if params.logprobs is not None and not getattr(engine, "supports_logprobs", False):
            return err(400, "log-probabilities are not available on this server (speculative decoding, asynchronous "
                            "scheduling or pipeline stages are on)")
        return None

    def sse(obj: Any) -> str:
        return "data: " + (obj if isinstance(obj, str) else json.dumps(obj, ensure_ascii=False)) + "\n\n"

    app.router.on_shutdown.append(aeng.shutdown)

    @app.get("/health")
    async def health():
        return PlainTextResponse("")

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "created": created,
                                            "owned_by": "stkernel_b200", "max_model_len": max_len}]}

    @app.get("/metrics")
    async def metrics():
        return PlainTextResponse(engine.metrics.render(model_name))

    @app.post("/start_profile")
    async def start_profile():
        return {"status": await aeng.call(lambda: aeng.start_profile(profile_dir))}

    @app.post("/stop_profile")
    async def stop_profile():
        return {"trace": await aeng.call(aeng.stop_profile)}

    @app.post("/reset_prefix_cache")
    async def reset_prefix_cache():
        ok = await aeng.call(aeng.reset_prefix_cache)
        return JSONResponse({"reset": ok}, status_code=200 if ok else 409)

    # ---- chat completions ---------------------------------------------------------------
    def prepare_chat(body: Dict[str, Any]):
        kwargs = {**base_kwargs, **(body.get("chat_template_kwargs") or {})}
        if "reasoning_effort" in body and "reasoning_effort" not in kwargs:
            kwargs["reasoning_effort"] = body["reasoning_effort"]
        thinking = thinking_enabled(kwargs, default_thinking)
        if thinking:
            kwargs.setdefault("thinking", True)
        tools = body.get("tools") if body.get("tool_choice") != "none" else None
        msgs = attach_response_format(flatten_content_parts(body["messages"]), body.get("response_format"))
        forced = forced_tool_prefix(body.get("tool_choice"), tools)
        if forced is None:
            return tokenizer.apply_chat_template(msgs, tools=tools, **kwargs), thinking, tools, ""
        # a call is demanded ("required", or a named function): the answer starts inside the tool-call block (and inside
        # the named invoke), without a thinking section, and the model continues from there
        kwargs["thinking"] = False
        prompt = tokenizer.apply_chat_template(msgs, tools=tools, tokenize=False, **kwargs)
        return tokenizer.encode(prompt + forced), False, tools, forced

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        try:
            body = await request.json()
            ids, thinking, tools, forced = prepare_chat(body)
            n_choices = choice_count(body)
        except HTTPException as e:
            return err(e.status_code, str(e.detail))
        except Exception as e:
            return err(400, f"{type(e).__name__}: {e}")
        if len(ids) >= max_len:
            return err(400, f"prompt has {len(ids)} tokens; the model's context is {max_len}")
        params = sampling_from_request(body, eos_id, max_len, len(ids), default_temperature=default_temperature)
        if refuse_logprobs(params) is not None:
            return refuse_logprobs(params)
        stop = parse_stop(body.get("stop"))
        rid = f"chatcmpl-{uuid.uuid4().hex}"
        # one output pipeline (detokenizer, reasoning splitter, tool parser) and one seed per choice
        pipes = [OutputPipeline(tokenizer, thinking, tools, stop, primed=forced) for _ in range(n_choices)]
        seeds = [dataclasses.replace(params, seed=(params.seed + i) & 0x7FFFFFFF) for i in range(n_choices)]
        base = {"id": rid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model_name}
        include_usage = want_usage(body)

        def finish(pipe: OutputPipeline, reason: Optional[str]) -> str:
            if pipe.has_tool_calls:
                return "tool_calls"
            return "stop" if (pipe.stopped or reason == "stop") else (reason or "stop")

        if body.get("stream"):
            async def events():
                n_out = 0
                for i in range(n_choices):
                    yield sse({**base, "choices": [{"index": i, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]})
                merged: asyncio.Queue = asyncio.Queue()

                async def pump(i: int):
                    try:
                        async for ev in aeng.generate(ids, seeds[i]):
                            await merged.put((i, ev))
                            if ev.error or ev.finished:
                                return
                    finally:
                        await merged.put((i, None))

                tasks = [asyncio.ensure_future(pump(i)) for i in range(n_choices)]
                open_choices, done, reasons = n_choices, set(), [None] * n_choices
                try:
                    while open_choices:
                        i, ev = await merged.get()
                        if ev is None:
                            open_choices -= 1
                            if i not in done:
                                done.add(i)
                                yield sse({**base, "choices": [{"index": i, "delta": {}, "finish_reason": finish(pipes[i], reasons[i])}]})
                            continue
                        if i in done:
                            continue
                        if ev.error:
                            yield sse({"error": {"message": ev.error, "type": "internal_error"}})
                            done.add(i)
                            continue
                        n_out += len(ev.tokens)
                        piece = pipes[i].push(ev.tokens, ev.finished, eos_id)
                        delta: Dict[str, Any] = {}
                        if piece.reasoning:
                            delta["reasoning_content"] = piece.reasoning
                        if piece.content:
                            delta["content"] = piece.content
                        if piece.tool_calls:
                            delta["tool_calls"] = [t.to_openai() for t in piece.tool_calls]
                        entries = logprob_entries(tokenizer, ev.tokens, ev.logprobs) if ev.logprobs else None
                        if delta or entries:
                            choice = {"index": i, "delta": delta, "finish_reason": None}
                            if entries:
                                choice["logprobs"] = {"content": entries}
                            yield sse({**base, "choices": [choice]})
                        reasons[i] = ev.finish_reason
                        if pipes[i].stopped or ev.finished:
                            done.add(i)
                            yield sse({**base, "choices": [{"index": i, "delta": {}, "finish_reason": finish(pipes[i], reasons[i])}]})
                            if not ev.finished:
                                tasks[i].cancel()             # a stop string: the generator's exit aborts the request
                finally:
                    for t in tasks:
                        t.cancel()
                if include_usage:
                    yield sse({**base, "choices": [], "usage": _usage(len(ids), n_out)})
                yield sse("[DONE]")
            return StreamingResponse(events(), media_type="text/event-stream")

        async def collect(i: int):
            pipe = pipes[i]
            reasoning, content, n_out, reason = "", "", 0, None
            entries: List[Dict[str, Any]] = []
            async for ev in aeng.generate(ids, seeds[i]):
                if ev.error:
                    return ev.error
                n_out += len(ev.tokens)
                if ev.logprobs:
                    entries += logprob_entries(tokenizer, ev.tokens, ev.logprobs)
                piece = pipe.push(ev.tokens, ev.finished, eos_id)
                reasoning += piece.reasoning
                content += piece.content
                reason = ev.finish_reason
                if pipe.stopped or ev.finished:
                    break
            message: Dict[str, Any] = {"role": "assistant", "content": content or None}
            if reasoning:
                message["reasoning_content"] = reasoning
            if pipe.has_tool_calls:
                message["tool_calls"] = [{"id": c["id"], "type": "function",
                                          "function": {"name": c["name"], "arguments": c["arguments"]}}
                                         for c in pipe.tools.complete_calls]
            choice = {"index": i, "message": message, "finish_reason": finish(pipe, reason)}
            if seeds[i].logprobs is not None:
                choice["logprobs"] = {"content": entries}
            return choice, n_out

        results = await asyncio.gather(*(collect(i) for i in range(n_choices)))
        for r in results:
            if isinstance(r, str):
                return err(500, r, "internal_error")
        return {"id": rid, "object": "chat.completion", "created": base["created"], "model": model_name,
                "choices": [r[0] for r in results], "usage": _usage(len(ids), sum(r[1] for r in results))}

    # ---- raw completions ------------------------------------------------------------------
    async def completions_batch(body: Dict[str, Any], prompts: List[Any], n_choices: int):
        """Every prompt x n samples as one response: choice index = prompt index * n + sample index."""
        all_ids = [list(p) if isinstance(p, list) else tokenizer.encode(p) for p in prompts]
        for ids in all_ids:
            if len(ids) >= max_len:
                return err(400, f"prompt has {len(ids)} tokens; the model's context is {max_len}")
        stop = parse_stop(body.get("stop"))

        async def one(k: int):
            ids = all_ids[k // n_choices]
            params = sampling_from_request(body, eos_id, max_len, len(ids), default_temperature=default_temperature)
            if body.get("seed") is not None:
                params = dataclasses.replace(params, seed=(params.seed + k % n_choices) & 0x7FFFFFFF)
            pipe = OutputPipeline(tokenizer, False, None, stop)
            n_out, reason = 0, None
            async for ev in aeng.generate(ids, params):
                if ev.error:
                    return ev.error
                n_out += len(ev.tokens)
                pipe.push(ev.tokens, ev.finished, eos_id)
                reason = ev.finish_reason
                if pipe.stopped or ev.finished:
                    break
            return {"index": k, "text": pipe.text, "finish_reason": "stop" if pipe.stopped else reason}, n_out

        results = await asyncio.gather(*(one(k) for k in range(len(all_ids) * n_choices)))
        for r in results:
            if isinstance(r, str):
                return err(500, r, "internal_error")
        return {"id": f"cmpl-{uuid.uuid4().hex}", "object": "text_completion", "created": int(time.time()), "model": model_name,
                "choices": [r[0] for r in results],
                "usage": _usage(sum(len(i) for i in all_ids), sum(r[1] for r in results))}

    @app.post("/v1/completions")
    async def completions(request: Request):
        try:
            body = await request.json()
            prompt = body["prompt"]
            n_choices = choice_count(body)
            # a batch of prompts (strings or token lists) and / or several samples per prompt: answered whole
            batch = isinstance(prompt, list) and bool(prompt) and not isinstance(prompt[0], int)
            if batch or n_choices > 1:
                if body.get("stream"):
                    raise HTTPException(status_code=400, detail="streaming takes one prompt and n = 1")
                return await completions_batch(body, list(prompt) if batch else [prompt], n_choices)
            ids = list(prompt) if isinstance(prompt, list) and prompt and isinstance(prompt[0], int) else tokenizer.encode(prompt)
        except HTTPException as e:
            return err(e.status_code, str(e.detail))
        except Exception as e:
            return err(400, f"{type(e).__name__}: {e}")
        if len(ids) >= max_len:
            return err(400, f"prompt has {len(ids)} tokens; the model's context is {max_len}")
        params = sampling_from_request(body, eos_id, max_len, len(ids), default_temperature=default_temperature)
        if refuse_logprobs(params) is not None:
            return refuse_logprobs(params)
        rid = f"cmpl-{uuid.uuid4().hex}"
        pipe = OutputPipeline(tokenizer, False, None, parse_stop(body.get("stop")))
        base = {"id": rid, "object": "text_completion", "created": int(time.time()), "model": model_name}
        if body.get("stream"):
            async def events():
                n_out, reason = 0, None
                async for ev in aeng.generate(ids, params):
                    n_out += len(ev.tokens)
                    piece = pipe.push(ev.tokens, ev.finished, eos_id)
                    if piece.content:
                        yield sse({**base, "choices": [{"index": 0, "text": piece.content, "finish_reason": None}]})
                    reason = ev.finish_reason
                    if pipe.stopped or ev.finished:
                        break
                yield sse({**base, "choices": [{"index": 0, "text": "", "finish_reason": "stop" if pipe.stopped else reason}],
                           "usage": _usage(len(ids), n_out)})
                yield sse("[DONE]")
            return StreamingResponse(events(), media_type="text/event-stream")
        n_out, reason = 0, None
        legacy = {"tokens": [], "token_logprobs": [], "top_logprobs": []}
        async for ev in aeng.generate(ids, params):
            if ev.error:
                return err(500, ev.error, "internal_error")
            n_out += len(ev.tokens)
            for e in logprob_entries(tokenizer, ev.tokens, ev.logprobs) if ev.logprobs else ():
                legacy["tokens"].append(e["token"])
                legacy["token_logprobs"].append(e["logprob"])
                legacy["top_logprobs"].append({t["token"]: t["logprob"] for t in e["top_logprobs"]})
            pipe.push(ev.tokens, ev.finished, eos_id)
            reason = ev.finish_reason
            if pipe.stopped or ev.finished:
                break
        choice = {"index": 0, "text": pipe.text, "finish_reason": "stop" if pipe.stopped else reason}
        if params.logprobs is not None:
            choice["logprobs"] = legacy
        return {**base, "choices": [choice], "usage": _usage(len(ids), n_out)}

    # ---- tokenizer routes -------------------------------------------------------------------
    @app.post("/tokenize")
    async def tokenize(request: Request):
        """{"prompt": str} or {"messages": [...], "tools": [...]} -> the ids the matching completion route would run."""
        try:
            body = await request.json()
            if "messages" in body:
                ids, _, _, _ = prepare_chat(body)
            else:
                ids = tokenizer.encode(body["prompt"])
        except HTTPException as e:
            return err(e.status_code, str(e.detail))
        except Exception as e:
            return err(400, f"{type(e).__name__}: {e}")
        return {"tokens": list(ids), "count": len(ids), "max_model_len": max_len}

    @app.post("/detokenize")
    async def detokenize(request: Request):
        try:
            body = await request.json()
            return {"prompt": tokenizer.decode([int(t) for t in body["tokens"]])}
        except Exception as e:
            return err(400, f"{type(e).__name__}: {e}")

    # ---- Anthropic messages ---------------------------------------------------------------
    def prepare_messages(body: Dict[str, Any]):
        msgs, tools = anthropic_to_chat(body)
        th = body.get("thinking") or {}
        kwargs = dict(base_kwargs)
        if th.get("type") == "enabled":
            kwargs["thinking"] = True
        elif th.get("type") == "disabled":
            kwargs["thinking"] = False
        thinking = thinking_enabled(kwargs, default_thinking)
        if thinking:
            kwargs.setdefault("thinking", True)
        # Anthropic tool_choice: {"type": "auto" | "none" | "any" | "tool", "name": ...}
        tc = body.get("tool_choice") or {}
        kind = tc.get("type") if isinstance(tc, dict) else tc
        if kind == "none":
            tools = None
        forced = forced_tool_prefix({"name": tc.get("name")} if kind == "tool" else ("required" if kind == "any" else None), tools)
        if forced is None:
            return tokenizer.apply_chat_template(msgs, tools=tools, **kwargs), thinking, tools, ""
        kwargs["thinking"] = False
        prompt = tokenizer.apply_chat_template(msgs, tools=tools, tokenize=False, **kwargs)
        return tokenizer.encode(prompt + forced), False, tools, forced

    @app.post("/v1/messages/count_tokens")
    async def count_tokens(request: Request):
        try:
            ids, _, _, _ = prepare_messages(await request.json())
        except Exception as e:
            return err(400, f"{type(e).__name__}: {e}")
        return {"input_tokens": len(ids)}

    @app.post("/v1/messages")
    async def messages(request: Request):
        try:
            body = await request.json()
            ids, thinking, tools, forced = prepare_messages(body)
        except Exception as e:
            return err(400, f"{type(e).__name__}: {e}")
        if len(ids) >= max_len:
            return err(400, f"prompt has {len(ids)} tokens; the model's context is {max_len}")
        params = sampling_from_request(body, eos_id, max_len, len(ids), default_temperature=default_temperature)
        pipe = OutputPipeline(tokenizer, thinking, tools, parse_stop(body.get("stop_sequences")), primed=forced)
        mid = f"msg_{uuid.uuid4().hex[:24]}"

        def stop_reason(reason):
            if pipe.has_tool_calls:
                return "tool_use"
            if pipe.stopped:
                return "stop_sequence"
            return "end_turn" if reason == "stop" else "max_tokens"

        if body.get("stream"):
            async def events():
                def ev_line(kind, payload):
                    return f"event: {kind}\ndata: {json.dumps({'type': kind, **payload}, ensure_ascii=False)}\n\n"
                yield ev_line("message_start", {"message": {"id": mid, "type": "message", "role": "assistant", "model": model_name,
                                                            "content": [], "stop_reason": None,
                                                            "usage": {"input_tokens": len(ids), "output_tokens": 0}}})
                block, kind_open, n_out, reason = -1, None, 0, None
                tool_block: Dict[int, int] = {}

                def open_block(kind, payload):
                    nonlocal block, kind_open
                    out = ""
                    if kind_open is not None:
                        out += ev_line("content_block_stop", {"index": block})
                    block += 1
                    kind_open = kind
                    return out + ev_line("content_block_start", {"index": block, "content_block": payload})

                async for ev in aeng.generate(ids, params):
                    n_out += len(ev.tokens)
                    piece = pipe.push(ev.tokens, ev.finished, eos_id)
                    if piece.reasoning:
                        if kind_open != "thinking":
                            yield open_block("thinking", {"type": "thinking", "thinking": ""})
                        yield ev_line("content_block_delta", {"index": block, "delta": {"type": "thinking_delta", "thinking": piece.reasoning}})
                    if piece.content:
                        if kind_open != "text":
                            yield open_block("text", {"type": "text", "text": ""})
                        yield ev_line("content_block_delta", {"index": block, "delta": {"type": "text_delta", "text": piece.content}})
                    for t in piece.tool_calls:
                        if t.id is not None:
                            yield open_block(f"tool{t.index}", {"type": "tool_use", "id": t.id.replace("call_", "toolu_"), "name": t.name, "input": {}})
                            tool_block[t.index] = block
                        if t.arguments:
                            yield ev_line("content_block_delta", {"index": tool_block[t.index],
                                                                  "delta": {"type": "input_json_delta", "partial_json": t.arguments}})
                    reason = ev.finish_reason
                    if pipe.stopped or ev.finished:
                        break
                if kind_open is not None:
                    yield ev_line("content_block_stop", {"index": block})
                yield ev_line("message_delta", {"delta": {"stop_reason": stop_reason(reason), "stop_sequence": None},
                                                "usage": {"output_tokens": n_out}})
                yield ev_line("message_stop", {})
            return StreamingResponse(events(), media_type="text/event-stream")

        reasoning, content, n_out, reason = "", "", 0, None
        async for ev in aeng.generate(ids, params):
            if ev.error:
                return err(500, ev.error, "api_error")
            n_out += len(ev.tokens)
            piece = pipe.push(ev.tokens, ev.finished, eos_id)
            reasoning += piece.reasoning
            content += piece.content
            reason = ev.finish_reason
            if pipe.stopped or ev.finished:
                break
        blocks: List[Dict[str, Any]] = []
        if reasoning:
            blocks.append({"type": "thinking", "thinking": reasoning})
        if content:
            blocks.append({"type": "text", "text": content})
        if pipe.has_tool_calls:
            for c in pipe.tools.complete_calls:
                blocks.append({"type": "tool_use", "id": c["id"].replace("call_", "toolu_"), "name": c["name"],
                               "input": json.loads(c["arguments"] or "{}")})
        return {"id": mid, "type": "message", "role": "assistant", "model": model_name, "content": blocks,
                "stop_reason": stop_reason(reason), "stop_sequence": None,
                "usage": {"input_tokens": len(ids), "output_tokens": n_out}}

    return app


def main(argv: Optional[Sequence[str]] = None) -> int:
    """`python -m stkernel_b200.serve.api_server --layers N [--tiny] [--tokenizer DIR] [--port P] ...`: one process, one
    device.  The flags are those of the multi-rank worker (`serve/tp_worker.py`), which this runs with a single rank."""
    from .tp_worker import main as worker_main
    return worker_main(argv)


if __name__ == "__main__":
    raise SystemExit(main())
