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
    a = srv.build_parser().parse_args(["--random-model", "tiny", "--device", "cpu", "--max-seq-len", "512",
                                       "--max-concurrent-requests", "2", "--prefix-cache-capacity-tokens", "2048",
                                       "--default-max-output-tokens", "24"])
    rt, tok, stop = srv.build_runtime(a)
    app = srv.create_app(rt.serving, tok, "tiny-test", 24, stop, 512)
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
