"""Serving layer on CPU: chat encoding goldens, tool/reasoning parsers (whole and streamed),
tokenizer front end, and the HTTP app over a tiny random-weight engine."""
import json
import os
import random

import pytest

from stkernel_b200.serve import encoding as E
from stkernel_b200.serve.reasoning import ReasoningSplitter, split_reasoning, thinking_enabled
from stkernel_b200.serve.tokenizer import ByteTokenizer, ChatTokenizer, IncrementalDetokenizer, chat_encode_config, render_chat
from stkernel_b200.serve.tool_parser import ToolCallParser, coerce, extract_tool_calls, held_back, schema_types

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "fixtures", "dsv4_encoding_golden.json")))
D = E.DSML
TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {
    "city": {"type": "string"}, "days": {"type": "integer"}, "opts": {"type": "object"}, "t": {"type": ["number", "null"]}}}}}]


# ---- encoding --------------------------------------------------------------------------
@pytest.mark.parametrize("i", range(len(GOLD["encode"])))
def test_encode_golden(i):
    g = GOLD["encode"][i]
    if g["prompt"] is None:
        with pytest.raises(Exception):
            E.encode_messages(g["messages"], **g["kwargs"])
    else:
        assert E.encode_messages(g["messages"], **g["kwargs"]) == g["prompt"]


@pytest.mark.parametrize("i", range(len(GOLD["parse"])))
def test_parse_golden(i):
    g = GOLD["parse"][i]
    if g["message"] is None:
        with pytest.raises(ValueError):
            E.parse_message_from_completion_text(g["text"], g["thinking_mode"])
    else:
        assert E.parse_message_from_completion_text(g["text"], g["thinking_mode"]) == g["message"]


def test_encode_basics():
    p = E.encode_messages([{"role": "user", "content": "hi"}], thinking_mode="chat")
    assert p == f"{E.BOS}{E.USER}hi{E.ASSISTANT}{E.THINK_CLOSE}"
    p = E.encode_messages([{"role": "user", "content": "hi"}], thinking_mode="thinking", reasoning_effort="max")
    assert p.startswith(E.BOS + "Reasoning Effort: Beyond maximum") and p.endswith(E.ASSISTANT + E.THINK_OPEN)
    with pytest.raises(ValueError):
        E.encode_messages([{"role": "user", "content": "hi"}], thinking_mode="other")


def test_encode_roundtrip_with_parser():
    calls = [{"id": "a", "type": "function", "function": {"name": "get_weather", "arguments": json.dumps({"city": "서울", "days": 2})}}]
    body = "plan" + E.THINK_CLOSE + "Checking." + E.dsml_tool_calls(calls) + E.EOS
    m = E.parse_message_from_completion_text(body, "thinking")
    assert m["reasoning"] == "plan" and m["content"] == "Checking."
    assert json.loads(m["tool_calls"][0]["function"]["arguments"]) == {"city": "서울", "days": 2}


def test_tool_results_follow_call_order_and_drop_thinking():
    msgs = [{"role": "user", "content": "q"},
            {"role": "assistant", "content": "", "reasoning": "r1", "tool_calls": [
                {"id": "x", "type": "function", "function": {"name": "f", "arguments": "{}"}},
                {"id": "y", "type": "function", "function": {"name": "g", "arguments": "{}"}}]},
            {"role": "tool", "tool_call_id": "y", "content": "Y"},
            {"role": "tool", "tool_call_id": "x", "content": "X"},
            {"role": "assistant", "content": "done", "reasoning": "r2"},
            {"role": "user", "content": "next"}]
    p = E.encode_messages(msgs, thinking_mode="thinking")
    assert p.index("<tool_result>X") < p.index("<tool_result>Y")
    assert "r1" not in p and "r2" not in p                      # reasoning before the last user turn is dropped
    p2 = E.encode_messages(msgs, thinking_mode="thinking", drop_thinking=False)
    assert "r1" in p2 and "r2" in p2


# ---- tokenizer front end ---------------------------------------------------------------
def test_effort_mapping_and_tools_on_system():
    assert chat_encode_config({"thinking": True, "reasoning_effort": "none"})["thinking_mode"] == "chat"
    assert chat_encode_config({"reasoning_effort": "xhigh"})["reasoning_effort"] == "max"
    assert chat_encode_config({"reasoning_effort": "medium"})["reasoning_effort"] is None
    assert chat_encode_config({"enable_thinking": True})["thinking_mode"] == "thinking"
    p = render_chat([{"role": "system", "content": "SYS"}, {"role": "user", "content": "u"}], TOOLS)
    assert p.startswith(E.BOS + "SYS\n\n## Tools")
    p = render_chat([{"role": "user", "content": "u"}], TOOLS)
    assert p.startswith(E.BOS + "\n\n## Tools") and "get_weather" in p


def test_byte_tokenizer_and_incremental_detok():
    bt = ByteTokenizer(512)
    text = f"{E.BOS}{E.USER}héllo 서울 🙂{E.ASSISTANT}{E.THINK_OPEN}"
    ids = bt.encode(text)
    assert bt.decode(ids) == text and ids[0] == bt.bos_token_id
    d = IncrementalDetokenizer(bt)
    parts = [d.push([t]) for t in ids]
    assert "".join(parts) == text
    assert all("�" not in p for p in parts)
    ct = ChatTokenizer(bt)
    assert ct.apply_chat_template([{"role": "user", "content": "x"}], tokenize=False).endswith(E.THINK_CLOSE)


# ---- reasoning --------------------------------------------------------------------------
def test_reasoning_split():
    assert split_reasoning("a</think>b", True) == ("a", "b")
    assert split_reasoning("<think>a</think>b", True) == ("a", "b")
    assert split_reasoning("only thinking", True) == ("only thinking", None)
    assert split_reasoning("a</think>b", False) == (None, "a</think>b")
    assert thinking_enabled({"thinking": True, "reasoning_effort": "none"}) is False
    assert thinking_enabled({}, default=True) is True and thinking_enabled({"enable_thinking": False}, default=True) is False
    text = f"hmm <｜ not a tag</thin still</think>answer <"
    for step in (1, 2, 5):
        s = ReasoningSplitter(True)
        r = c = ""
        for i in range(0, len(text), step):
            a, b = s.push(text[i:i + step])
            r, c = r + a, c + b
        a, b = s.flush()
        assert (r + a, c + b) == ("hmm <｜ not a tag</thin still", "answer <")


def test_reasoning_recovers_tool_block_without_close():
    text = f'thinking...\n\n<{D}tool_calls>\n<{D}invoke name="get_weather">\n</{D}invoke>\n</{D}tool_calls>'
    r, c = split_reasoning(text, True)
    assert r == "thinking..." and c.startswith(f"\n\n<{D}tool_calls>")


# ---- tool parser --------------------------------------------------------------------------
def _block(name="tool_calls"):
    return (f'Sure.\n\n<{D}{name}>\n<{D}invoke name="get_weather">\n'
            f'<{D}parameter name="city" string="true">서울 "x"\n2</{D}parameter>\n'
            f'<{D}parameter name="days" string="false">3</{D}parameter>\n'
            f'<{D}parameter name="opts" string="false">{{"a": [1, 2]}}</{D}parameter>\n'
            f'<{D}parameter name="t" string="false">null</{D}parameter>\n'
            f'</{D}invoke>\n<{D}invoke name="get_weather">\n'
            f'<{D}parameter name="arguments" string="false">{{"city": "x"}}</{D}parameter>\n'
            f'</{D}invoke>\n<{D}invoke name="noargs">\n</{D}invoke>\n</{D}{name}>')


@pytest.mark.parametrize("name", ["tool_calls", "function_calls"])
def test_extract_tool_calls(name):
    content, calls = extract_tool_calls(_block(name), TOOLS)
    assert content == "Sure."
    assert [c["function"]["name"] for c in calls] == ["get_weather", "get_weather", "noargs"]
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": '서울 "x"\n2', "days": 3, "opts": {"a": [1, 2]}, "t": None}
    assert json.loads(calls[1]["function"]["arguments"]) == {"city": "x"}            # wrapper unwrapped
    assert json.loads(calls[2]["function"]["arguments"]) == {}
    assert all(c["id"].startswith("call_") and len(c["id"]) == 29 for c in calls)


def test_extract_without_calls_returns_text():
    assert extract_tool_calls("plain text") == ("plain text", [])
    broken = f"x <{D}tool_calls>\n<{D}invoke name="
    assert extract_tool_calls(broken) == (broken, [])


@pytest.mark.parametrize("step", [1, 2, 3, 7, 11, 64, 10000])
def test_streaming_matches_whole(step):
    text = _block()
    _, whole = extract_tool_calls(text, TOOLS)
    p = ToolCallParser(TOOLS)
    content, args, names, ids = "", {}, {}, {}
    for i in range(0, len(text), step):
        d = p.push(text[i:i + step])
        content += d.content
        for t in d.tool_calls:
            wire = t.to_openai()
            assert None not in wire.values() and None not in wire["function"].values()    # no null keys on the wire
            args[t.index] = args.get(t.index, "") + (t.arguments or "")
            if t.name is not None:
                assert t.index not in names and t.id is not None
                names[t.index], ids[t.index] = t.name, t.id
    content += p.flush().content
    assert content == "Sure."
    assert [names[i] for i in range(3)] == [c["function"]["name"] for c in whole]
    for i in range(3):
        assert json.loads(args[i]) == json.loads(whole[i]["function"]["arguments"])


def test_streaming_string_param_streams_early_scalars_wait():
    p = ToolCallParser(TOOLS)
    p.push(f'<{D}tool_calls>\n<{D}invoke name="get_weather">\n<{D}parameter name="city" string="true">Seo')
    d = p.push("ul and")
    assert d.tool_calls and d.tool_calls[0].arguments == "ul and"
    p.push(f'</{D}parameter>\n<{D}parameter name="days" string="false">1')
    d = p.push("2")
    assert not d                                               # integer waits for the closing tag
    d = p.push(f"</{D}parameter>")
    assert d.tool_calls[0].arguments == ',"days":12'


def test_schema_helpers():
    assert schema_types({"type": ["integer", "null"]}) == ["integer", "null"]
    assert schema_types({"anyOf": [{"type": "string"}, {"type": "array"}]}) == ["string", "array"]
    assert schema_types({}) == ["string"] and schema_types({"enum": [1, 2]}) == ["integer"]
    assert coerce("5", ["integer"]) == 5 and coerce("5.5", ["number"]) == 5.5 and coerce("true", ["boolean"]) is True
    assert coerce("abc", ["integer"]) == "abc" and coerce('{"a":1}', ["integer"]) == {"a": 1}
    assert coerce("[1]", ["array"]) == [1] and coerce("null", ["integer", "null"]) is None
    assert held_back("abc</thi", ["</think>"]) == 5 and held_back("abc", ["</think>"]) == 0


# ---- HTTP app ------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def client():
    import torch
    from fastapi.testclient import TestClient
    from stkernel_b200.config import EngineConfig, SchedulerConfig, tiny_config
    from stkernel_b200.models.dsv4 import DictSource, build_model_weights
    from stkernel_b200.models.weights import init_random_weights
    from stkernel_b200.runtime.engine import Engine
    from stkernel_b200.serve.api_server import create_app
    torch.manual_seed(0)
    cfg = tiny_config()
    ec = EngineConfig(model=cfg, sched=SchedulerConfig(max_model_len=512, max_num_seqs=4, max_num_batched_tokens=256,
                                                       graph_cap=0)).validate()
    eng = Engine(ec, build_model_weights(cfg, DictSource(init_random_weights(cfg, seed=0)), "cpu"), "cpu", max_context=512)
    app = create_app(eng, ChatTokenizer(ByteTokenizer(cfg.vocab_size)), "tiny-dsv4", profile_dir="/tmp/stk_test_profiles")
    with TestClient(app) as c:
        yield c


def _sse(resp):
    out = []
    for line in resp.iter_lines():
        if line.startswith("data: "):
            out.append(line[6:])
    return out


def test_models_health_metrics(client):
    assert client.get("/health").status_code == 200
    m = client.get("/v1/models").json()
    assert m["data"][0]["id"] == "tiny-dsv4"
    text = client.get("/metrics").text
    assert "vllm:generation_tokens_total" in text and "vllm:num_requests_running" in text
    for name in ("vllm:gpu_cache_usage_perc", "vllm:prefix_cache_queries_total", "vllm:prefix_cache_hits_total",
                 "vllm:time_to_first_token_seconds_sum", "vllm:time_to_first_token_seconds_count"):
        assert name in text


def test_chat_completion_and_usage(client):
    body = {"model": "tiny-dsv4", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0, "ignore_eos": True}
    r = client.post("/v1/chat/completions", json=body).json()
    assert r["object"] == "chat.completion" and r["choices"][0]["finish_reason"] == "length"
    assert r["usage"]["completion_tokens"] == 6 and r["usage"]["prompt_tokens"] > 0
    r2 = client.post("/v1/chat/completions", json=body).json()
    assert r2["choices"][0]["message"] == r["choices"][0]["message"]               # greedy is reproducible
    before = client.get("/metrics").text
    from stkernel_b200.runtime.metrics import parse_prometheus
    assert parse_prometheus(before)['vllm:generation_tokens_total{model_name="tiny-dsv4"}'] >= 12


def test_chat_stream_matches_nonstream(client):
    body = {"messages": [{"role": "user", "content": "stream me"}], "max_tokens": 8, "temperature": 0, "ignore_eos": True}
    whole = client.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"] or ""
    with client.stream("POST", "/v1/chat/completions", json={**body, "stream": True, "stream_options": {"include_usage": True}}) as resp:
        lines = _sse(resp)
    assert lines[-1] == "[DONE]"
    chunks = [json.loads(x) for x in lines[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"])
    assert text == whole
    assert chunks[-1]["usage"]["completion_tokens"] == 8 and chunks[-1]["choices"] == []
    assert chunks[-2]["choices"][0]["finish_reason"] == "length"


def test_several_choices_and_content_parts(client):
    """`n` choices: one seed, detokenizer and parser per choice; streamed chunks carry the choice index and add up to
    the whole answers.  Content-part arrays are read as their text."""
    body = {"messages": [{"role": "user", "content": "pick"}], "max_tokens": 6, "temperature": 1.0, "seed": 5, "ignore_eos": True,
            "n": 3}
    r = client.post("/v1/chat/completions", json=body).json()
    assert [c["index"] for c in r["choices"]] == [0, 1, 2] and r["usage"]["completion_tokens"] == 18
    texts = [c["message"]["content"] or "" for c in r["choices"]]
    assert len(set(texts)) > 1                                                     # different seeds, different samples
    # choice i samples with seed + i: the first choice is the answer of the same request with n = 1
    one = client.post("/v1/chat/completions", json={**body, "n": 1}).json()
    assert one["choices"][0]["message"] == r["choices"][0]["message"]
    shifted = client.post("/v1/chat/completions", json={**body, "n": 1, "seed": 7}).json()
    assert shifted["choices"][0]["message"] == r["choices"][2]["message"]
    with client.stream("POST", "/v1/chat/completions", json={**body, "stream": True, "stream_options": {"include_usage": True}}) as resp:
        lines = _sse(resp)
    assert lines[-1] == "[DONE]"
    chunks = [json.loads(x) for x in lines[:-1]]
    streamed = ["", "", ""]
    finished = {}
    for c in chunks:
        for ch in c["choices"]:
            streamed[ch["index"]] += ch["delta"].get("content", "")
            if ch["finish_reason"]:
                assert ch["index"] not in finished
                finished[ch["index"]] = ch["finish_reason"]
    assert streamed == texts and finished == {0: "length", 1: "length", 2: "length"}
    assert chunks[-1]["usage"]["completion_tokens"] == 18
    assert client.post("/v1/chat/completions", json={**body, "n": 0}).status_code == 400
    assert client.post("/v1/chat/completions", json={**body, "n": 99}).status_code == 400
    # content parts
    parts = {"messages": [{"role": "user", "content": [{"type": "text", "text": "hello"}, {"type": "text", "text": "there"}]}],
             "max_tokens": 4, "temperature": 0, "ignore_eos": True}
    plain = {**parts, "messages": [{"role": "user", "content": "hello\nthere"}]}
    a, b = client.post("/v1/chat/completions", json=parts).json(), client.post("/v1/chat/completions", json=plain).json()
    assert a["choices"][0]["message"] == b["choices"][0]["message"] and a["usage"] == b["usage"]
    bad = {**parts, "messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "x"}}]}]}
    r = client.post("/v1/chat/completions", json=bad)
    assert r.status_code == 400 and "image_url" in r.json()["error"]["message"]


def test_completions_batch_of_prompts_and_samples(client):
    one = lambda p, seed: client.post("/v1/completions", json={"prompt": p, "max_tokens": 5, "temperature": 0.8, "seed": seed,
                                                                "ignore_eos": True}).json()["choices"][0]["text"]
    r = client.post("/v1/completions", json={"prompt": ["first prompt", "second"], "n": 2, "max_tokens": 5, "temperature": 0.8,
                                             "seed": 3, "ignore_eos": True}).json()
    assert [c["index"] for c in r["choices"]] == [0, 1, 2, 3] and r["usage"]["completion_tokens"] == 20
    assert [c["text"] for c in r["choices"]] == [one("first prompt", 3), one("first prompt", 4), one("second", 3), one("second", 4)]
    ids = client.post("/tokenize", json={"prompt": "second"}).json()["tokens"]
    r2 = client.post("/v1/completions", json={"prompt": [ids], "max_tokens": 5, "temperature": 0.8, "seed": 3, "ignore_eos": True}).json()
    assert r2["choices"][0]["text"] == r["choices"][2]["text"]
    assert client.post("/v1/completions", json={"prompt": ["a", "b"], "stream": True}).status_code == 400


def test_log_probabilities(client):
    import math
    body = {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 5, "temperature": 0, "ignore_eos": True,
            "logprobs": True, "top_logprobs": 3}
    r = client.post("/v1/chat/completions", json=body).json()
    entries = r["choices"][0]["logprobs"]["content"]
    assert len(entries) == 5
    for e in entries:
        assert e["logprob"] <= 0 and len(e["top_logprobs"]) == 3
        # greedy: the sampled token is the most likely one, and the alternatives come in decreasing order
        assert e["top_logprobs"][0]["logprob"] == pytest.approx(e["logprob"], abs=1e-5)
        assert [t["logprob"] for t in e["top_logprobs"]] == sorted((t["logprob"] for t in e["top_logprobs"]), reverse=True)
        assert e["bytes"] == list(e["token"].encode("utf-8"))
    # the same answer as without them, and no key when they are not asked for
    plain = client.post("/v1/chat/completions", json={k: v for k, v in body.items() if "logprobs" not in k}).json()
    assert plain["choices"][0]["message"] == r["choices"][0]["message"] and "logprobs" not in plain["choices"][0]
    # streamed: the chunks' entries add up to the same list
    with client.stream("POST", "/v1/chat/completions", json={**body, "stream": True}) as resp:
        chunks = [json.loads(x) for x in _sse(resp)[:-1]]
    streamed = [e for c in chunks for ch in c["choices"] for e in (ch.get("logprobs") or {}).get("content", [])]
    assert [(e["token"], round(e["logprob"], 5)) for e in streamed] == [(e["token"], round(e["logprob"], 5)) for e in entries]
    # raw completions, legacy layout
    raw = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 4, "temperature": 0, "ignore_eos": True,
                                               "logprobs": 2}).json()["choices"][0]["logprobs"]
    assert len(raw["tokens"]) == len(raw["token_logprobs"]) == len(raw["top_logprobs"]) == 4
    assert all(len(d) <= 2 and max(d.values()) <= 0 for d in raw["top_logprobs"])
    assert all(math.isfinite(x) for x in raw["token_logprobs"])
    assert client.post("/v1/chat/completions", json={**body, "top_logprobs": 50}).status_code == 400


def test_tokenizer_routes(client):
    t = client.post("/tokenize", json={"prompt": "abc def"}).json()
    assert t["count"] == len(t["tokens"]) > 0 and t["max_model_len"] == 512
    assert client.post("/detokenize", json={"tokens": t["tokens"]}).json()["prompt"] == "abc def"
    msgs = [{"role": "user", "content": "count me"}]
    chat = client.post("/tokenize", json={"messages": msgs}).json()
    run = client.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 1, "temperature": 0}).json()
    assert chat["count"] == run["usage"]["prompt_tokens"]
    n = client.post("/v1/messages/count_tokens", json={"messages": msgs, "system": "be brief"}).json()["input_tokens"]
    m = client.post("/v1/messages", json={"messages": msgs, "system": "be brief", "max_tokens": 1}).json()
    assert n == m["usage"]["input_tokens"]
    assert client.post("/tokenize", json={}).status_code == 400
    assert client.post("/detokenize", json={"tokens": "x"}).status_code == 400


def test_thinking_mode_routes_to_reasoning(client):
    body = {"messages": [{"role": "user", "content": "think"}], "max_tokens": 5, "temperature": 0, "ignore_eos": True,
            "chat_template_kwargs": {"thinking": True}}
    m = client.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]
    assert m["content"] is None and m.get("reasoning_content")                     # never closed its reasoning


def test_concurrent_requests_and_bad_request(client):
    import concurrent.futures as cf
    def one(i):
        return client.post("/v1/completions", json={"prompt": f"p{i}", "max_tokens": 4, "temperature": 0, "ignore_eos": True}).json()
    with cf.ThreadPoolExecutor(4) as ex:
        outs = list(ex.map(one, range(6)))
    assert all(o["usage"]["completion_tokens"] == 4 for o in outs)
    assert client.post("/v1/chat/completions", json={"messages": [{"role": "alien", "content": "x"}]}).status_code == 400
    long = {"messages": [{"role": "user", "content": "x" * 600}]}
    assert client.post("/v1/chat/completions", json=long).status_code == 400


def test_anthropic_messages(client):
    body = {"model": "tiny-dsv4", "max_tokens": 5, "temperature": 0, "system": "S", "ignore_eos": True,
            "messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}]}
    r = client.post("/v1/messages", json=body).json()
    assert r["type"] == "message" and r["stop_reason"] == "max_tokens" and r["usage"]["output_tokens"] == 5
    with client.stream("POST", "/v1/messages", json={**body, "stream": True}) as resp:
        kinds = [json.loads(x)["type"] for x in _sse(resp)]
    assert kinds[0] == "message_start" and kinds[-1] == "message_stop" and "message_delta" in kinds


def test_profile_and_cache_reset(client):
    assert client.post("/start_profile").json()["status"] == "started"
    client.post("/v1/completions", json={"prompt": "x", "max_tokens": 2, "temperature": 0})
    trace = client.post("/stop_profile").json()["trace"]
    assert trace and os.path.exists(trace)
    assert client.post("/reset_prefix_cache").json()["reset"] is True
    assert "stk:prefix_cache_resets_total" in client.get("/metrics").text


# ---- scripted engine: the HTTP layer's handling of reasoning + DSML tool calls end to end -------------------
class ScriptedEngine:
    """Stands in for the engine: every request emits the token ids of a fixed completion text, one per step."""

    def __init__(self, tok, text):
        import types
        from stkernel_b200.runtime.metrics import Metrics
        self.tok, self.script = tok, tok.encode(text) + [tok.eos_token_id]
        self.cfg = types.SimpleNamespace(sched=types.SimpleNamespace(max_model_len=4096))
        self.metrics = Metrics()
        import torch
        self.device = torch.device("cpu")
        self.requests, self._next, self._live = {}, 0, []
        self.prompts = []

    def add_request(self, prompt, params):
        import types
        rid = self._next
        self._next += 1
        self.prompts.append(list(prompt))
        self.requests[rid] = types.SimpleNamespace(req_id=rid, prompt=prompt, params=params, output=[], finished=False, finish_reason=None)
        self._live.append(rid)
        return rid

    def has_work(self):
        return bool(self._live)

    def step(self):
        out = []
        for rid in list(self._live):
            r = self.requests[rid]
            tokn = self.script[len(r.output)]
            r.output.append(tokn)
            out.append((rid, tokn))
            if tokn == self.tok.eos_token_id or len(r.output) >= r.params.max_tokens:
                r.finished, r.finish_reason = True, "stop" if tokn == self.tok.eos_token_id else "length"
                self._live.remove(rid)
        return out

    def abort(self, rid):
        r = self.requests.get(rid)
        if r is None or r.finished:
            return False
        r.finished, r.finish_reason = True, "abort"
        self._live.remove(rid)
        return True

    def release(self, rid):
        self.requests.pop(rid, None)


TOOL_COMPLETION = ('I should look it up.' + E.THINK_CLOSE + 'Let me check.' +
                   E.dsml_tool_calls([{"function": {"name": "get_weather", "arguments": json.dumps({"city": "서울", "days": 2})}}]))


@pytest.fixture()
def tool_client():
    from fastapi.testclient import TestClient
    from stkernel_b200.serve.api_server import create_app
    tok = ChatTokenizer(ByteTokenizer(1024))
    with TestClient(create_app(ScriptedEngine(tok, TOOL_COMPLETION), tok, "scripted")) as c:
        yield c


def test_chat_with_tools_nonstream(tool_client):
    body = {"messages": [{"role": "user", "content": "weather?"}], "tools": TOOLS, "max_tokens": 2000,
            "chat_template_kwargs": {"thinking": True}}
    r = tool_client.post("/v1/chat/completions", json=body).json()
    ch = r["choices"][0]
    assert ch["finish_reason"] == "tool_calls"
    m = ch["message"]
    assert m["reasoning_content"] == "I should look it up." and m["content"] == "Let me check."
    call = m["tool_calls"][0]
    assert call["function"]["name"] == "get_weather" and json.loads(call["function"]["arguments"]) == {"city": "서울", "days": 2}
    # without thinking the same bytes are content up to the block (the </think> tag stays literal text)
    r2 = tool_client.post("/v1/chat/completions", json={**body, "chat_template_kwargs": {}}).json()
    assert "reasoning_content" not in r2["choices"][0]["message"] and r2["choices"][0]["finish_reason"] == "tool_calls"


def test_chat_with_tools_stream_deltas(tool_client):
    body = {"messages": [{"role": "user", "content": "weather?"}], "tools": TOOLS, "max_tokens": 2000, "stream": True,
            "chat_template_kwargs": {"thinking": True}, "stream_options": {"include_usage": True}}
    with tool_client.stream("POST", "/v1/chat/completions", json=body) as resp:
        lines = _sse(resp)
    chunks = [json.loads(x) for x in lines[:-1]]
    reasoning = "".join(c["choices"][0]["delta"].get("reasoning_content", "") for c in chunks if c["choices"])
    content = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"])
    assert reasoning == "I should look it up." and content == "Let me check."
    name, args, ids = None, "", set()
    for c in chunks:
        for ch in c["choices"]:
            for t in ch["delta"].get("tool_calls", []):
                assert t["index"] == 0 and None not in t.values() and None not in t["function"].values()
                if "id" in t:
                    ids.add(t["id"])
                    name = t["function"]["name"]
                args += t["function"].get("arguments", "")
    assert name == "get_weather" and len(ids) == 1 and json.loads(args) == {"city": "서울", "days": 2}
    finals = [c["choices"][0]["finish_reason"] for c in chunks if c["choices"] and c["choices"][0]["finish_reason"]]
    assert finals == ["tool_calls"] and chunks[-1]["usage"]["completion_tokens"] > 0


def test_anthropic_tool_use_blocks(tool_client):
    body = {"model": "scripted", "max_tokens": 2000, "thinking": {"type": "enabled"},
            "tools": [{"name": "get_weather", "description": "w", "input_schema": TOOLS[0]["function"]["parameters"]}],
            "messages": [{"role": "user", "content": "weather?"},
                         {"role": "assistant", "content": [{"type": "tool_use", "id": "toolu_1", "name": "get_weather", "input": {"city": "x"}}]},
                         {"role": "user", "content": [{"type": "tool_result", "tool_use_id": "toolu_1", "content": "sunny"},
                                                      {"type": "text", "text": "and Seoul?"}]}]}
    r = tool_client.post("/v1/messages", json=body).json()
    kinds = [b["type"] for b in r["content"]]
    assert kinds == ["thinking", "text", "tool_use"] and r["stop_reason"] == "tool_use"
    assert r["content"][2]["input"] == {"city": "서울", "days": 2} and r["content"][2]["id"].startswith("toolu_")
    with tool_client.stream("POST", "/v1/messages", json={**body, "stream": True}) as resp:
        events = [json.loads(x) for x in _sse(resp)]
    starts = [e["content_block"]["type"] for e in events if e["type"] == "content_block_start"]
    assert starts == ["thinking", "text", "tool_use"]
    partial = "".join(e["delta"]["partial_json"] for e in events if e["type"] == "content_block_delta" and e["delta"]["type"] == "input_json_delta")
    assert json.loads(partial) == {"city": "서울", "days": 2}
    assert [e["delta"]["stop_reason"] for e in events if e["type"] == "message_delta"] == ["tool_use"]


def test_demanded_tool_call_starts_inside_the_call():
    """tool_choice "required" / a named function: the prompt ends with the opening of the call, the model continues it,
    and the parsers see the opening in front of what was generated."""
    from fastapi.testclient import TestClient
    from stkernel_b200.serve.api_server import create_app, forced_tool_prefix
    tok = ChatTokenizer(ByteTokenizer(1024))
    whole = E.dsml_tool_calls([{"function": {"name": "get_weather", "arguments": json.dumps({"city": "Busan", "days": 1})}}])
    named = forced_tool_prefix({"type": "function", "function": {"name": "get_weather"}}, TOOLS)
    anyone = forced_tool_prefix("required", TOOLS)
    assert whole.startswith(named) and named.startswith(anyone) and anyone.endswith('invoke name="')
    assert forced_tool_prefix("auto", TOOLS) is None and forced_tool_prefix(None, TOOLS) is None
    for choice, prefix in (({"type": "function", "function": {"name": "get_weather"}}, named), ("required", anyone)):
        eng = ScriptedEngine(tok, whole[len(prefix):])            # the model writes the rest of the call
        with TestClient(create_app(eng, tok, "scripted")) as c:
            body = {"messages": [{"role": "user", "content": "2+2? no tools please"}], "tools": TOOLS, "max_tokens": 500,
                    "tool_choice": choice, "chat_template_kwargs": {"thinking": True}}
            r = c.post("/v1/chat/completions", json=body).json()
            ch = r["choices"][0]
            assert ch["finish_reason"] == "tool_calls" and not ch["message"].get("reasoning_content")
            call = ch["message"]["tool_calls"][0]["function"]
            assert call["name"] == "get_weather" and json.loads(call["arguments"]) == {"city": "Busan", "days": 1}
            prompt = tok.decode(eng.prompts[0])
            assert prompt.endswith(prefix) and E.THINK_OPEN not in prompt.split(prefix)[0][-20:]
            with c.stream("POST", "/v1/chat/completions", json={**body, "stream": True}) as resp:
                chunks = [json.loads(x) for x in _sse(resp)[:-1]]
            names = [t["function"].get("name") for ck in chunks for ch2 in ck["choices"] for t in ch2["delta"].get("tool_calls", [])]
            args = "".join(t["function"].get("arguments", "") for ck in chunks for ch2 in ck["choices"]
                           for t in ch2["delta"].get("tool_calls", []))
            assert "get_weather" in names and json.loads(args) == {"city": "Busan", "days": 1}
            # Anthropic wire: {"type": "tool", "name": ...} / {"type": "any"}
            a_choice = {"type": "tool", "name": "get_weather"} if isinstance(choice, dict) else {"type": "any"}
            a_tools = [{"name": "get_weather", "description": "w", "input_schema": TOOLS[0]["function"]["parameters"]}]
            m = c.post("/v1/messages", json={"messages": [{"role": "user", "content": "hi"}], "tools": a_tools, "max_tokens": 500,
                                             "tool_choice": a_choice}).json()
            use = [b for b in m["content"] if b["type"] == "tool_use"]
            assert m["stop_reason"] == "tool_use" and use[0]["name"] == "get_weather" and use[0]["input"] == {"city": "Busan", "days": 1}
    with TestClient(create_app(ScriptedEngine(tok, "x"), tok, "scripted")) as c:
        base = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 5}
        assert c.post("/v1/chat/completions", json={**base, "tool_choice": "required"}).status_code == 400          # no tools
        bad = {"type": "function", "function": {"name": "nope"}}
        assert c.post("/v1/chat/completions", json={**base, "tools": TOOLS, "tool_choice": bad}).status_code == 400


def test_stop_string_ends_stream_early(tool_client):
    body = {"messages": [{"role": "user", "content": "x"}], "max_tokens": 2000, "stop": ["check"], "chat_template_kwargs": {"thinking": True}}
    r = tool_client.post("/v1/chat/completions", json=body).json()
    assert r["choices"][0]["message"]["content"] == "Let me " and r["choices"][0]["finish_reason"] == "stop"
    # streamed, two choices: each ends at its own stop string and the stream still closes with [DONE]
    with tool_client.stream("POST", "/v1/chat/completions", json={**body, "n": 2, "stream": True,
                                                                   "stream_options": {"include_usage": True}}) as resp:
        lines = _sse(resp)
    assert lines[-1] == "[DONE]"
    chunks = [json.loads(x) for x in lines[:-1]]
    text, fin = ["", ""], {}
    for c in chunks:
        for ch in c["choices"]:
            text[ch["index"]] += ch["delta"].get("content", "")
            if ch["finish_reason"]:
                fin[ch["index"]] = ch["finish_reason"]
    assert text == ["Let me ", "Let me "] and fin == {0: "stop", 1: "stop"}


def test_top_p_top_k_and_response_format_reach_the_engine_and_the_prompt():
    """`top_p` / `top_k` become sampling parameters (bad values are refused), `response_format` lands in the system
    block of the rendered prompt."""
    from stkernel_b200.serve.api_server import attach_response_format, sampling_from_request
    p = sampling_from_request({"top_p": 0.9, "top_k": 40, "temperature": 0.7, "seed": 1}, 1, 4096, 10)
    assert p.top_p == 0.9 and p.top_k == 40 and p.truncates
    p = sampling_from_request({"top_k": -1, "seed": 1}, 1, 4096, 10)
    assert p.top_k == 0 and p.top_p == 1.0 and not p.truncates
    with pytest.raises(Exception):
        sampling_from_request({"top_p": 0.0}, 1, 4096, 10)
    msgs = [{"role": "user", "content": "give me json"}]
    assert attach_response_format(msgs, None) == msgs and attach_response_format(msgs, {"type": "text"}) == msgs
    out = attach_response_format(msgs, {"type": "json_object"})
    assert out[0]["role"] == "system" and out[0]["response_format"] == {"type": "object"} and out[1:] == msgs
    schema = {"type": "object", "properties": {"a": {"type": "integer"}}, "required": ["a"]}
    sys_first = [{"role": "system", "content": "be brief"}] + msgs
    out = attach_response_format(sys_first, {"type": "json_schema", "json_schema": {"name": "x", "schema": schema}})
    assert out[0]["content"] == "be brief" and out[0]["response_format"] == schema
    from stkernel_b200.serve.tokenizer import render_chat
    text = render_chat(out)
    assert '"required"' in text and "be brief" in text
    with pytest.raises(Exception):
        attach_response_format(msgs, {"type": "grammar"})


def test_truncated_sampling_matches_the_definition_on_cpu():
    """top-k / top-p on the reference path: the sampled token always lies in the truncated set, greedy is unchanged,
    and k = 1 equals the arg-max whatever the noise."""
    import torch
    from stkernel_b200.ops import reference as R
    from stkernel_b200.ops import sampling as S
    torch.manual_seed(0)
    B, V = 6, 500
    logits = torch.randn(B, V) * 3
    temp = torch.full((B,), 0.8)
    seed = torch.arange(B, dtype=torch.int64)
    pos = torch.arange(B, dtype=torch.int64) + 5
    k = torch.tensor([1, 5, 0, 50, 0, 3], dtype=torch.int32)
    p = torch.tensor([1.0, 1.0, 0.5, 0.9, 0.05, 0.7])
    tok, proc = S.gumbel_argmax(logits, temp, seed, pos, want_processed=True, top_k=k, top_p=p)
    keep = R.truncation_mask(logits, temp, k, p)
    assert all(bool(keep[i, tok[i]]) for i in range(B))
    assert tok[0] == logits[0].argmax()
    assert int(keep[1].sum()) == 5 and int(keep[5].sum()) <= 3
    pr = torch.softmax(logits[2] / 0.8, -1)
    assert pr[keep[2]].sum() >= 0.5 and pr[keep[2]].sum() - pr[keep[2]].min() < 0.5      # minimal nucleus
    assert torch.isinf(proc[~keep]).all() and torch.isfinite(proc[keep]).all()
    # untruncated call is unchanged by the new arguments
    t0, _ = S.gumbel_argmax(logits, temp, seed, pos)
    t1, _ = S.gumbel_argmax(logits, temp, seed, pos, top_k=torch.zeros(B, dtype=torch.int32), top_p=torch.ones(B))
    assert torch.equal(t0, t1)


from stkernel_b200.serve.api_server import OutputPipeline  # noqa: E402

_PIPE_TOK = ChatTokenizer(ByteTokenizer(1024))
PIPE_TOOLS = [{"type": "function", "function": {"name": "get_weather", "description": "w", "parameters": {
                  "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}, "opts": {"type": "object"}}}}},
              {"type": "function", "function": {"name": "f2", "description": "x", "parameters": {
                  "type": "object", "properties": {"q": {"type": "string"}}}}}]


# ---- randomised chunking of the whole output pipeline --------------------------------------------------------------
def _pipe_run(text, thinking, stop, sizes):
    ids = _PIPE_TOK.encode(text)
    pipe = OutputPipeline(_PIPE_TOK, thinking, PIPE_TOOLS, stop)
    r = c = ""; calls = {}
    i = 0; k = 0
    while i < len(ids) and not pipe.stopped:
        n = sizes[k % len(sizes)]; k += 1
        chunk = ids[i:i + n]; i += n
        p = pipe.push(chunk, i >= len(ids), None)
        r += p.reasoning; c += p.content
        for t in p.tool_calls:
            d = t.to_openai()
            e = calls.setdefault(d["index"], {"name": "", "arguments": ""})
            f = d.get("function", {})
            if f.get("name"): e["name"] = f["name"]
            e["arguments"] += f.get("arguments", "")
    if i >= len(ids) and not pipe.stopped and k == 0:
        pass
    return r, c, calls, pipe.stopped


def test_output_pipeline_is_independent_of_how_tokens_are_grouped():
    """Detokenizer, stop strings, reasoning splitter and tool-call parser together: any grouping of the tokens into steps
    gives the reasoning, content, tool calls and stop flag of pushing them all at once."""
    import random
    rng = random.Random(0)
    for trial in range(150):
        think = rng.random() < 0.5
        parts = []
        if think:
            parts.append(rng.choice(["I think so.", "Let me <see> 한글 생각", "", "multi\nline\n\nthought"]) + E.THINK_CLOSE)
        parts.append(rng.choice(["Answer: 42.", "한국어 답변 ✓ emoji 🙂", "", "text with < and <｜ partial", "stop here please"]))
        if rng.random() < 0.6:
            calls = [{"function": {"name": rng.choice(["get_weather", "f2"]),
                                   "arguments": json.dumps(rng.choice([{"city": "서울", "days": 2}, {"q": "a<b>c"},
                                                                       {"city": "x", "opts": {"a": [1, 2]}}, {}]))}}
                     for _ in range(rng.randint(1, 3))]
            parts.append(E.dsml_tool_calls(calls))
        text = "".join(parts)
        stop = rng.choice([[], [], ["please"], ["42"]])
        whole = _pipe_run(text, think, stop, [10 ** 6])
        for _ in range(3):
            sizes = [rng.randint(1, 9) for _ in range(7)]
            assert _pipe_run(text, think, stop, sizes) == whole, (text, stop, sizes)


def test_random_request_bodies_never_cause_a_server_error_or_stop_the_engine_thread():
    """Wrongly typed and contradictory fields on every POST route: the answer is a 2xx or a 4xx, never a 5xx, and the
    server still answers a well-formed request afterwards."""
    import random
    from fastapi.testclient import TestClient
    from stkernel_b200.serve.api_server import create_app
    tok = ChatTokenizer(ByteTokenizer(1024))
    rng = random.Random(0)
    vals = [None, True, False, 0, -1, 1, 3, 0.5, -0.5, "", "x", "auto", "none", "required", [], [1, 2], ["a"], {},
            {"type": "json_object"}, {"type": "function", "function": {"name": "get_weather"}},
            [{"role": "user", "content": "hi"}], [{"role": "user"}], [{"content": "x"}], [{"role": "tool", "content": "r"}],
            [{"role": "assistant", "tool_calls": [{"function": {"name": "f", "arguments": "{"}}]}],
            [{"role": "user", "content": [{"type": "text", "text": "a"}]}], TOOLS, [{"type": "function"}], "think",
            {"thinking": True}, {"include_usage": True}]
    keys = ["messages", "prompt", "max_tokens", "temperature", "top_p", "top_k", "n", "stream", "stop", "seed", "tools",
            "tool_choice", "response_format", "logprobs", "top_logprobs", "chat_template_kwargs", "stream_options",
            "min_tokens", "ignore_eos", "system", "thinking", "stop_sequences", "reasoning_effort", "max_completion_tokens",
            "tokens"]
    routes = ["/v1/chat/completions", "/v1/completions", "/v1/messages", "/tokenize", "/detokenize", "/v1/messages/count_tokens"]
    with TestClient(create_app(ScriptedEngine(tok, "hello world"), tok, "scripted"), raise_server_exceptions=False) as c:
        for _ in range(400):
            body = {k: rng.choice(vals) for k in rng.sample(keys, rng.randint(0, 7))}
            if rng.random() < 0.6:
                body["messages"] = [{"role": "user", "content": "hi"}]
            if rng.random() < 0.3:
                body["prompt"] = "hello"
            body.setdefault("max_tokens", 3)
            path = rng.choice(routes)
            r = c.post(path, json=body)
            assert r.status_code < 500, (path, body, r.text[:200])
        ok = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3})
        assert ok.status_code == 200 and ok.json()["usage"]["completion_tokens"] == 3
