"""OpenAI-compatible server on CPU with a random tiny model and the byte tokenizer: endpoints, streaming,
400s before generation, structured output through the grammar engine, prefix-cache reuse across turns."""
import json
import socket
import threading
import time

import pytest
import requests

pytest.importorskip("fastapi")
pytest.importorskip("uvicorn")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture(scope="module")
def server():
    import uvicorn
    from phaseshift_b200.apps import server as srv
    a = srv.build_parser().parse_args(["--random-model", "tiny", "--device", "cpu", "--max-seq-len", "1024",
                                       "--max-concurrent-requests", "2", "--prefix-cache-capacity-tokens", "2048",
                                       "--default-max-output-tokens", "24"])
    rt, tok, stop = srv.build_runtime(a)
    app = srv.create_app(rt.serving, tok, "tiny-test", 24, stop, 1024)
    port = _free_port()
    cfg = uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error")
    us = uvicorn.Server(cfg)
    th = threading.Thread(target=us.run, daemon=True)
    th.start()
    url = f"http://127.0.0.1:{port}"
    for _ in range(200):
        try:
            if requests.get(url + "/health", timeout=1).ok:
                break
        except Exception:
            time.sleep(0.05)
    yield url, rt
    us.should_exit = True
    app.state.engine_thread.cmd.put(("stop",))
    th.join(timeout=10)


@pytest.mark.timeout(300)
def test_models_and_chat_completion(server):
    url, rt = server
    assert requests.get(url + "/v1/models").json()["data"][0]["id"] == "tiny-test"
    assert requests.get(url + "/v1/models/tiny-test").json()["object"] == "model"
    assert requests.get(url + "/v1/models/other").status_code == 404
    r = requests.post(url + "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 8})
    assert r.status_code == 200
    j = r.json()
    assert j["choices"][0]["finish_reason"] in ("length", "stop") and j["usage"]["completion_tokens"] <= 8
    assert j["choices"][0]["message"]["role"] == "assistant"
    r2 = requests.post(url + "/v1/responses", json={"input": "hello", "max_output_tokens": 5})
    assert r2.status_code == 200 and r2.json()["output"][0]["content"][0]["type"] == "output_text"


@pytest.mark.timeout(300)
def test_streaming_and_prefix_cache_across_turns(server):
    url, rt = server
    msgs = [{"role": "system", "content": "s" * 80}, {"role": "user", "content": "first question " * 3},
            {"role": "assistant", "content": "an answer"}, {"role": "user", "content": "second"}]
    with requests.post(url + "/v1/chat/completions", json={"messages": msgs, "max_tokens": 6, "stream": True}, stream=True) as r:
        lines = [l.decode() for l in r.iter_lines() if l]
    assert lines[-1] == "data: [DONE]" and json.loads(lines[0][6:])["choices"][0]["delta"]["role"] == "assistant"
    assert json.loads(lines[-2][6:])["choices"][0]["finish_reason"] in ("length", "stop")
    # same history, new last turn -> the boundary checkpoint saved by the first request is restored
    msgs2 = msgs[:3] + [{"role": "user", "content": "another"}]
    j = requests.post(url + "/v1/chat/completions", json={"messages": msgs2, "max_tokens": 4}).json()
    assert j["usage"]["prompt_tokens_details"]["cached_tokens"] > 64


@pytest.mark.timeout(300)
def test_bad_requests_are_rejected_before_generation(server):
    url, rt = server
    post = lambda b: requests.post(url + "/v1/chat/completions", json=b)
    m = [{"role": "user", "content": "x"}]
    assert post({"messages": m, "reasoning_effort": "extreme"}).status_code == 400
    assert post({"messages": []}).status_code == 400
    assert post({"messages": m, "tools": [{"type": "function", "function": {"name": "f", "strict": True, "parameters": {
        "type": "object", "properties": {"a": {"type": "string"}}, "required": []}}}]}).status_code == 400
    assert post({"messages": m, "tool_choice": {"type": "function", "function": {"name": "nope"}},
                 "tools": [{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}}]}).status_code == 400
    assert post({"messages": m, "response_format": {"type": "yaml"}}).status_code == 400
    assert post({"messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "x"}}]}]}).status_code == 400


@pytest.mark.timeout(300)
def test_json_schema_response_format_is_enforced(server):
    url, rt = server
    if rt.serving.constraints is None:
        pytest.skip("grammar engine not available")
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}}, "required": ["ok"], "additionalProperties": False}
    j = requests.post(url + "/v1/chat/completions", json={
        "messages": [{"role": "user", "content": "json please"}], "max_tokens": 40,
        "response_format": {"type": "json_schema", "json_schema": {"name": "r", "schema": schema}}}).json()
    txt = j["choices"][0]["message"]["content"]
    assert isinstance(json.loads(txt)["ok"], bool)       # a random model produced schema-valid JSON


@pytest.mark.timeout(300)
def test_sampling_parameters_seed_determinism_and_limits(server):
    """Same seed -> same stochastic completion, another seed may differ; max_tokens and max_completion_tokens cap the output;
    the usage block adds up."""
    url, rt = server
    body = {"messages": [{"role": "user", "content": "sample"}], "max_tokens": 12, "temperature": 0.9, "top_p": 0.95, "top_k": 50,
            "seed": 7}
    a = requests.post(url + "/v1/chat/completions", json=body).json()
    b = requests.post(url + "/v1/chat/completions", json=body).json()
    assert a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]
    u = a["usage"]
    assert u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"] and 1 <= u["completion_tokens"] <= 12
    c = requests.post(url + "/v1/chat/completions", json=dict(body, max_completion_tokens=3)).json()
    assert c["usage"]["completion_tokens"] <= 3
    g1 = requests.post(url + "/v1/chat/completions", json=dict(body, temperature=0)).json()
    g2 = requests.post(url + "/v1/chat/completions", json=dict(body, temperature=0, seed=99)).json()
    assert g1["choices"][0]["message"]["content"] == g2["choices"][0]["message"]["content"]     # greedy ignores the seed


@pytest.mark.timeout(300)
def test_concurrent_requests_are_batched_and_all_answered(server):
    """More simultaneous requests than sequence slots: the scheduler queues the rest; every request gets its own answer and
    equal prompts get equal greedy answers."""
    url, rt = server
    out = [None] * 5

    def go(i):
        out[i] = requests.post(url + "/v1/chat/completions", json={
            "messages": [{"role": "user", "content": "same prompt" if i % 2 == 0 else f"prompt number {i}"}], "max_tokens": 6}).json()
    ths = [threading.Thread(target=go, args=(i,)) for i in range(5)]
    for t in ths:
        t.start()
    for t in ths:
        t.join(timeout=120)
    assert all(o is not None and o["choices"][0]["finish_reason"] in ("length", "stop") for o in out)
    assert out[0]["choices"][0]["message"]["content"] == out[2]["choices"][0]["message"]["content"] == out[4]["choices"][0]["message"]["content"]
    assert len({o["id"] for o in out}) == 5


@pytest.mark.timeout(300)
def test_context_window_and_malformed_bodies(server):
    url, rt = server
    r = requests.post(url + "/v1/chat/completions", json={"messages": [{"role": "user", "content": "x" * 4000}]})
    assert r.status_code == 400 and "context window" in r.json()["error"]["message"]
    r = requests.post(url + "/v1/chat/completions", data="{not json", headers={"content-type": "application/json"})
    assert r.status_code == 400 and r.json()["error"]["type"] == "invalid_request_error"
    r = requests.post(url + "/v1/chat/completions", json={"messages": "hello"})
    assert r.status_code == 400
    r = requests.post(url + "/v1/chat/completions", json={"messages": [{"role": "wizard", "content": "x"}]})
    assert r.status_code == 400
    # a prompt that nearly fills the window: the completion budget is clamped to what is left, not rejected
    r = requests.post(url + "/v1/chat/completions", json={"messages": [{"role": "user", "content": "y" * 900}], "max_tokens": 500})
    assert r.status_code == 200 and r.json()["usage"]["total_tokens"] <= 1024
    assert requests.get(url + "/health").json() == {"status": "ok"}        # the engine thread survived all of it


@pytest.mark.timeout(300)
def test_tool_calls_forced_by_tool_choice(server):
    """tool_choice = required / a named function constrains the output to a tool call whose arguments satisfy the schema;
    tool_choice = none never returns one."""
    url, rt = server
    if rt.serving.constraints is None:
        pytest.skip("grammar engine not available")
    tools = [{"type": "function", "function": {"name": "set_flag", "description": "sets a flag", "parameters": {
        "type": "object", "properties": {"on": {"type": "boolean"}}, "required": ["on"], "additionalProperties": False}}},
        {"type": "function", "function": {"name": "other", "parameters": {"type": "object", "properties": {}, "additionalProperties": False}}}]
    body = {"messages": [{"role": "user", "content": "call it"}], "tools": tools, "max_tokens": 300}
    j = requests.post(url + "/v1/chat/completions", json=dict(body, tool_choice={"type": "function", "function": {"name": "set_flag"}})).json()
    ch = j["choices"][0]
    assert ch["finish_reason"] == "tool_calls" and ch["message"]["tool_calls"][0]["function"]["name"] == "set_flag"
    assert isinstance(json.loads(ch["message"]["tool_calls"][0]["function"]["arguments"])["on"], bool)
    assert ch["message"]["tool_calls"][0]["type"] == "function" and ch["message"]["tool_calls"][0]["id"]
    j = requests.post(url + "/v1/chat/completions", json=dict(body, tool_choice="required")).json()
    assert j["choices"][0]["finish_reason"] == "tool_calls"
    assert j["choices"][0]["message"]["tool_calls"][0]["function"]["name"] in ("set_flag", "other")
    j = requests.post(url + "/v1/chat/completions", json=dict(body, tool_choice="none", max_tokens=8)).json()
    assert "tool_calls" not in j["choices"][0]["message"] and j["choices"][0]["finish_reason"] in ("length", "stop")


@pytest.mark.timeout(300)
def test_streaming_chunks_reassemble_to_the_non_streamed_answer(server):
    url, rt = server
    body = {"messages": [{"role": "user", "content": "stream me"}], "max_tokens": 10}
    whole = requests.post(url + "/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"]
    with requests.post(url + "/v1/chat/completions", json=dict(body, stream=True), stream=True) as r:
        assert r.headers["content-type"].startswith("text/event-stream")
        chunks = [json.loads(l.decode()[6:]) for l in r.iter_lines() if l and l != b"data: [DONE]"]
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks)
    assert text == whole
    assert len({c["id"] for c in chunks}) == 1 and all(c["object"] == "chat.completion.chunk" for c in chunks)
    assert chunks[-1]["choices"][0]["finish_reason"] in ("length", "stop") and all(c["choices"][0]["finish_reason"] is None for c in chunks[:-1])


@pytest.mark.timeout(300)
def test_client_disconnect_cancels_the_request_and_frees_its_slot(server):
    """A streaming client that goes away: the engine cancels the request; afterwards every slot serves again."""
    url, rt = server
    with requests.post(url + "/v1/chat/completions", json={"messages": [{"role": "user", "content": "long"}], "max_tokens": 400,
                                                           "stream": True}, stream=True) as r:
        it = r.iter_lines()
        next(it)                      # the role chunk arrived: generation is under way
    time.sleep(0.5)
    ok = [requests.post(url + "/v1/chat/completions", json={"messages": [{"role": "user", "content": f"after {i}"}], "max_tokens": 4})
          for i in range(3)]
    assert all(o.status_code == 200 for o in ok)
    deadline = time.time() + 20
    while time.time() < deadline and not rt.serving.idle():
        time.sleep(0.1)
    assert rt.serving.idle()


@pytest.mark.timeout(300)
def test_responses_endpoint_with_instructions_and_message_list(server):
    url, rt = server
    r = requests.post(url + "/v1/responses", json={"instructions": "be brief", "input": [{"role": "user", "content": "hello"}],
                                                   "max_output_tokens": 5})
    j = r.json()
    # five tokens cannot finish a random model's answer: the response is cut at the limit and says so
    assert r.status_code == 200 and j["object"] == "response" and j["status"] in ("completed", "incomplete")
    if j["status"] == "incomplete":
        assert j["incomplete_details"] == {"reason": "max_output_tokens"}
    assert j["usage"]["output_tokens"] <= 5 and j["usage"]["input_tokens"] > 0 and j["id"].startswith("resp_")
    assert requests.post(url + "/v1/responses", json={"input": [{"role": "user", "content": [{"type": "image_url"}]}]}).status_code == 400


@pytest.mark.timeout(300)
def test_responses_endpoint_items_tools_structured_output_and_streaming(server):
    """The Responses API surface: conversation items (function calls and their outputs), flat tool definitions with a forced
    call, `text.format` JSON schemas, and the event stream, all agreeing with the non-streamed result."""
    url, rt = server
    # streaming: deltas concatenate to the final text, which equals the non-streamed answer (greedy)
    body = {"input": "tell me", "max_output_tokens": 10}
    plain = requests.post(url + "/v1/responses", json=body).json()
    events = []
    with requests.post(url + "/v1/responses", json=dict(body, stream=True), stream=True) as r:
        assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
        for line in r.iter_lines(decode_unicode=True):
            if line and line.startswith("data: "):
                events.append(json.loads(line[6:]))
    kinds = [e["type"] for e in events]
    assert kinds[0] == "response.created" and kinds[-1] in ("response.completed", "response.incomplete")
    assert kinds[-2] == "response.output_text.done"
    deltas = "".join(e["delta"] for e in events if e["type"] == "response.output_text.delta")
    assert deltas == events[-2]["text"] == plain["output_text"]
    assert events[-1]["response"]["usage"] == plain["usage"]
    assert [e["sequence_number"] for e in events] == sorted(e["sequence_number"] for e in events)
    # conversation items: an earlier function call and its output are part of the prompt
    items = [{"role": "user", "content": [{"type": "input_text", "text": "weather?"}]},
             {"type": "function_call", "call_id": "call_0", "name": "get_weather", "arguments": "{\"city\": \"Oslo\"}"},
             {"type": "function_call_output", "call_id": "call_0", "output": "4 degrees"}]
    a = requests.post(url + "/v1/responses", json={"input": items, "max_output_tokens": 4}).json()
    b = requests.post(url + "/v1/responses", json={"input": items[:1], "max_output_tokens": 4}).json()
    assert a["usage"]["input_tokens"] > b["usage"]["input_tokens"]
    assert requests.post(url + "/v1/responses", json={"input": [{"type": "computer_call"}]}).status_code == 400
    if rt.serving.constraints is None:
        return
    # a forced call with the flat tool form comes back as a function_call item with schema-valid arguments
    tool = {"type": "function", "name": "get_weather", "strict": True,
            "parameters": {"type": "object", "properties": {"city": {"type": "string", "enum": ["Oslo", "Rome"]}},
                           "required": ["city"], "additionalProperties": False}}
    j = requests.post(url + "/v1/responses", json={"input": "weather?", "tools": [tool], "max_output_tokens": 300,
                                                   "tool_choice": {"type": "function", "name": "get_weather"}}).json()
    calls = [o for o in j["output"] if o["type"] == "function_call"]
    assert len(calls) == 1 and calls[0]["name"] == "get_weather" and json.loads(calls[0]["arguments"])["city"] in ("Oslo", "Rome")
    # structured output through text.format
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}}, "required": ["ok"], "additionalProperties": False}
    j = requests.post(url + "/v1/responses", json={"input": "json", "max_output_tokens": 40,
                                                   "text": {"format": {"type": "json_schema", "name": "r", "schema": schema}}}).json()
    assert isinstance(json.loads(j["output_text"])["ok"], bool)


@pytest.mark.timeout(300)
def test_stop_sequences_cut_the_answer_and_streams_report_usage(server):
    """`stop` strings end the answer at their first occurrence (not shown), in the plain and in the streamed form, with
    characters that might begin a stop sequence held back; `stream_options.include_usage` adds a usage chunk."""
    url, rt = server
    if rt.serving.constraints is None:
        pytest.skip("grammar engine not available")
    # a grammar keeps the random model on letters, so that the answer is a text of 24 characters
    body = {"messages": [{"role": "user", "content": "stop test"}], "max_tokens": 24,
            "response_format": {"type": "grammar", "grammar": "root ::= [a-j]+"}}
    full = requests.post(url + "/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"]
    pick = None
    for i in range(2, max(2, len(full) - 2)):
        sub = full[i:i + 2]
        if "\\ufffd" not in sub and "\\ufffd" not in full[:i] and full.find(sub) == i:
            pick = (i, sub)
            break
    if pick is None:
        pytest.skip("the random model's answer has no usable substring")
    i, sub = pick
    j = requests.post(url + "/v1/chat/completions", json=dict(body, stop=[sub, "never-appears"])).json()
    assert j["choices"][0]["message"]["content"] == full[:i] and j["choices"][0]["finish_reason"] == "stop"
    chunks = []
    with requests.post(url + "/v1/chat/completions", json=dict(body, stop=sub, stream=True, stream_options={"include_usage": True}),
                       stream=True) as r:
        for line in r.iter_lines(decode_unicode=True):
            if line and line.startswith("data: ") and line != "data: [DONE]":
                chunks.append(json.loads(line[6:]))
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c.get("choices"))
    assert text == full[:i]
    assert [c["choices"][0]["finish_reason"] for c in chunks if c.get("choices")][-1] == "stop"
    usage = [c["usage"] for c in chunks if "usage" in c]
    assert len(usage) == 1 and usage[0]["total_tokens"] == usage[0]["prompt_tokens"] + usage[0]["completion_tokens"]
    # a stop that never completes changes nothing, and held-back characters are delivered at the end
    chunks = []
    with requests.post(url + "/v1/chat/completions", json=dict(body, stop=full[-1] + "\\x00never", stream=True), stream=True) as r:
        for line in r.iter_lines(decode_unicode=True):
            if line and line.startswith("data: ") and line != "data: [DONE]":
                chunks.append(json.loads(line[6:]))
    assert "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c.get("choices")) == full
    assert requests.post(url + "/v1/chat/completions", json=dict(body, stop=["a", "b", "c", "d", "e"])).status_code == 400
    deadline = time.time() + 30
    while time.time() < deadline and not rt.serving.idle():
        time.sleep(0.1)
    assert rt.serving.idle()


@pytest.mark.timeout(120)
def test_capabilities_the_server_lacks_are_refused_not_ignored(server):
    url, rt = server
    base = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 2}
    for extra in ({"n": 2}, {"logprobs": True}, {"top_logprobs": 3}, {"modalities": ["text", "audio"]}, {"audio": {"voice": "x"}},
                  {"temperature": -1}, {"top_p": 1.5}, {"temperature": "hot"}):
        r = requests.post(url + "/v1/chat/completions", json=dict(base, **extra))
        assert r.status_code == 400 and r.json()["error"]["type"] == "invalid_request_error", extra
    assert requests.post(url + "/v1/chat/completions", json=dict(base, n=1, modalities=["text"], temperature=0, top_p=1)).status_code == 200
    assert requests.get(url + "/v1/embeddings").status_code in (404, 405)
    assert requests.post(url + "/v1/embeddings", json={"input": "x"}).status_code in (404, 405)


def _stream(url, body):
    chunks = []
    with requests.post(url + "/v1/chat/completions", json=dict(body, stream=True), stream=True) as r:
        assert r.status_code == 200
        for line in r.iter_lines(decode_unicode=True):
            if line and line.startswith("data: ") and line != "data: [DONE]":
                chunks.append(json.loads(line[6:]))
    return [c["choices"][0] for c in chunks if c.get("choices")]


@pytest.mark.timeout(300)
def test_streams_separate_reasoning_answer_and_tool_calls(server):
    """With reasoning on, the text in front of the closing think tag streams as `reasoning_content`, the rest as `content`,
    and the tag itself is never shown; tool-call markup never streams as content.  Both agree with the plain response."""
    url, rt = server
    if rt.serving.constraints is None:
        pytest.skip("grammar engine not available")
    g = 'root ::= [a-e] [a-e] [a-e] [a-e] "</think>" [f-j] [f-j] [f-j] [f-j] [f-j]'
    body = {"messages": [{"role": "user", "content": "think"}], "max_tokens": 40, "reasoning_effort": "low",
            "response_format": {"type": "grammar", "grammar": g}}
    plain = requests.post(url + "/v1/chat/completions", json=body).json()["choices"][0]["message"]
    assert len(plain["reasoning_content"]) == 4 and len(plain["content"]) == 5 and "think" not in plain["content"]
    ch = _stream(url, body)
    assert "".join(c["delta"].get("reasoning_content", "") for c in ch) == plain["reasoning_content"]
    assert "".join(c["delta"].get("content", "") for c in ch) == plain["content"]
    order = [("r" if "reasoning_content" in c["delta"] else "c") for c in ch if c["delta"].get("reasoning_content") or c["delta"].get("content")]
    assert order == sorted(order, reverse=True)                                  # all reasoning comes first
    # a forced tool call: the stream carries no markup, only the call at the end
    tool = {"type": "function", "function": {"name": "get_weather", "strict": True, "parameters": {
        "type": "object", "properties": {"city": {"type": "string", "enum": ["Oslo", "Rome"]}}, "required": ["city"],
        "additionalProperties": False}}}
    tb = {"messages": [{"role": "user", "content": "weather?"}], "tools": [tool], "max_tokens": 300,
          "tool_choice": {"type": "function", "function": {"name": "get_weather"}}}
    ch = _stream(url, tb)
    shown = "".join(c["delta"].get("content", "") for c in ch)
    assert "<tool_call>" not in shown and "get_weather" not in shown
    assert ch[-1]["finish_reason"] == "tool_calls" and ch[-1]["delta"]["tool_calls"][0]["function"]["name"] == "get_weather"


@pytest.mark.timeout(300)
def test_agent_loop_tool_result_round_trip_reuses_the_prefix(server):
    """An agent turn pair: forced tool call, then the call and its result go back in the history; the second request
    restores the shared prefix (tools, system prompt, first user turn) from the cache instead of prefilling it again."""
    url, rt = server
    if rt.serving.constraints is None:
        pytest.skip("grammar engine not available")
    tool = {"type": "function", "function": {"name": "lookup", "strict": True, "parameters": {
        "type": "object", "properties": {"key": {"type": "string", "enum": ["alpha", "beta"]}}, "required": ["key"],
        "additionalProperties": False}}}
    history = [{"role": "system", "content": "You are a careful assistant that always looks things up before answering. " * 6},
               {"role": "user", "content": "what is alpha?"}]
    first = requests.post(url + "/v1/chat/completions", json={
        "messages": history, "tools": [tool], "max_tokens": 300,
        "tool_choice": {"type": "function", "function": {"name": "lookup"}}}).json()
    call = first["choices"][0]["message"]["tool_calls"][0]
    assert first["choices"][0]["finish_reason"] == "tool_calls" and json.loads(call["function"]["arguments"])["key"] in ("alpha", "beta")
    history += [{"role": "assistant", "content": None, "tool_calls": [call]},
                {"role": "tool", "tool_call_id": call["id"], "content": "alpha is the first letter"}]
    second = requests.post(url + "/v1/chat/completions", json={"messages": history, "tools": [tool], "max_tokens": 6}).json()
    assert second["choices"][0]["finish_reason"] in ("stop", "length", "tool_calls")
    assert second["usage"]["prompt_tokens"] > first["usage"]["prompt_tokens"]
    assert second["usage"]["prompt_tokens_details"]["cached_tokens"] > 0


def test_metrics_endpoint_exposes_the_serving_counters(server):
    url, rt = server
    requests.post(url + "/v1/chat/completions", json={"messages": [{"role": "user", "content": "count me"}], "max_tokens": 3})
    r = requests.get(url + "/metrics")
    assert r.status_code == 200 and r.headers["content-type"].startswith("text/plain")
    vals = {l.split()[0]: float(l.split()[1]) for l in r.text.splitlines() if l and not l.startswith("#")}
    assert vals["phaseshift_steps_total"] >= 1 and vals["phaseshift_generated_tokens_total"] >= 1
    assert vals["phaseshift_prefill_tokens_total"] >= 1 and vals["phaseshift_requests_active"] == 0
    assert vals["phaseshift_kv_pages_free"] > 0 and "phaseshift_prefix_cache_hits_total" in vals
    assert all(l.startswith(("# HELP phaseshift_", "# TYPE phaseshift_", "phaseshift_")) for l in r.text.splitlines() if l)


@pytest.mark.timeout(300)
def test_bounded_admission_answers_429_when_the_queue_is_full():
    """One slot, one queued request allowed: while two requests are in flight a third is refused with 429 and a retry hint;
    once they finish the server accepts again."""
    import uvicorn
    from phaseshift_b200.apps import server as srv
    a = srv.build_parser().parse_args(["--random-model", "tiny", "--device", "cpu", "--max-seq-len", "256",
                                       "--max-concurrent-requests", "1", "--prefix-cache-capacity-tokens", "0",
                                       "--max-queued-requests", "1"])
    rt, tok, stop = srv.build_runtime(a)
    app = srv.create_app(rt.serving, tok, "tiny-429", 24, stop, 256, max_in_flight=2)
    port = _free_port()
    us = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=us.run, daemon=True)
    th.start()
    url = f"http://127.0.0.1:{port}"
    for _ in range(200):
        try:
            if requests.get(url + "/health", timeout=1).ok:
                break
        except Exception:
            time.sleep(0.05)
    try:
        body = {"messages": [{"role": "user", "content": "long answer please"}], "max_tokens": 120}
        results = []
        ts = [threading.Thread(target=lambda: results.append(requests.post(url + "/v1/chat/completions", json=body).status_code))
              for _ in range(2)]
        for t in ts:
            t.start()
        deadline = time.time() + 30
        while time.time() < deadline and len(app.state.engine_thread.out) < 2:
            time.sleep(0.01)
        r = requests.post(url + "/v1/chat/completions", json=dict(body, max_tokens=2))
        assert r.status_code == 429 and r.headers["Retry-After"] == "1" and r.json()["error"]["type"] == "rate_limit_error"
        assert requests.post(url + "/v1/responses", json={"input": "x", "max_output_tokens": 2}).status_code == 429
        for t in ts:
            t.join(120)
        assert results == [200, 200]
        assert requests.post(url + "/v1/chat/completions", json=dict(body, max_tokens=2)).status_code == 200
    finally:
        us.should_exit = True
        app.state.engine_thread.cmd.put(("stop",))
        th.join(timeout=10)
