"""phaseshift-server: OpenAI-compatible HTTP server in one process.

The reference chains LocalAI (Go) -> gRPC backend (Python) -> ``phaseshift-compute --serve-stdio``
(src/apps/server/phaseshift_server.py, backend/phaseshift_backend.py, backend/compute_client.py); the
three hops exist only because of its Go front end.  Here FastAPI talks to the serving loop directly: a
single engine thread owns the GPU and steps the continuous batcher, HTTP handlers exchange messages with
it through queues.  Preserved surface (docs/user/server.md:79-330): ``/v1/chat/completions`` (stream and
non-stream, tools, strict tools, ``response_format``), ``/v1/responses``, ``/v1/models``, opt-in reasoning,
HTTP 400 for bad schemas / tool contracts / unknown ``reasoning_effort`` before generation starts,
``finish_reason="cancelled"`` when the client disconnects, fail-closed structured output.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import queue
import sys
import threading
import time
import uuid
from typing import Dict, List, Optional

from ..serving import chat

try:        # module-level names so FastAPI can resolve the handlers' (string) annotations
    from fastapi import FastAPI, Request
    from fastapi.responses import JSONResponse, StreamingResponse
except Exception:  # pragma: no cover - the server app needs fastapi; everything else imports without it
    FastAPI = Request = JSONResponse = StreamingResponse = None


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="phaseshift-server")
    ap.add_argument("--model-dir"); ap.add_argument("--random-model", choices=["tiny", "4b", "27b"])
    ap.add_argument("--preset", default=None); ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000); ap.add_argument("--max-seq-len", type=int, default=32768)
    ap.add_argument("--arena-gib", type=float, default=0); ap.add_argument("--device", default=None)
    ap.add_argument("--kv-cache-dtype", default="bf16", choices=["bf16", "fp8_e4m3", "nvfp4", "psq4", "psq8"])
    ap.add_argument("--page-tokens", type=int, default=16); ap.add_argument("--max-concurrent-requests", type=int, default=4)
    ap.add_argument("--kv-cache-capacity-tokens", type=int, default=0)
    ap.add_argument("--prefix-cache-capacity-tokens", type=int, default=16384)
    ap.add_argument("--prefix-cache-max-entries", type=int, default=8)
    ap.add_argument("--default-max-output-tokens", type=int, default=4096)
    ap.add_argument("--dflash2-model-dir"); ap.add_argument("--dflash2-drafts", type=int, default=7)
    ap.add_argument("--model-name", default="phaseshift"); ap.add_argument("--verify-weights", type=int, default=0)
    ap.add_argument("--startup-timeout", type=int, default=120)
    ap.add_argument("--max-queued-requests", type=int, default=0,
                    help="requests that may wait for a slot; more are answered with HTTP 429 (0: unbounded queue)")
    # the upstream server is a front end that spawns the compute binary (docs/user/server.md:79-102); here the engine lives
    # in the server process, so the two paths are accepted and unused
    ap.add_argument("--compute", default=None, help="accepted for compatibility (the engine runs in this process)")
    ap.add_argument("--localai-binary", default=None, help="accepted for compatibility")
    ap.add_argument("--tp", type=int, default=1, choices=[1, 2, 4, 8], help="tensor-parallel ranks, one process per GPU")
    return ap


class EngineThread(threading.Thread):
    """Owns the serving loop.  Commands in: ("submit", ticket, kwargs) / ("cancel", ticket).  Each ticket has
    an out-queue receiving ("token", id) / ("done", info) / ("error", message)."""

    def __init__(self, serving):
        super().__init__(daemon=True)
        self.srv = serving
        self.cmd: "queue.Queue" = queue.Queue()
        self.out: Dict[int, "queue.Queue"] = {}
        self.rid_of: Dict[int, int] = {}
        self.ticket_of: Dict[int, int] = {}
        self._next = 1
        self._lock = threading.Lock()
        self.running = True
        self.ready = threading.Event()

    def new_ticket(self) -> int:
        with self._lock:
            t = self._next
            self._next += 1
            self.out[t] = queue.Queue()
            return t

    def run(self):
        self.ready.set()
        while self.running:
            try:
                while True:
                    c = self.cmd.get(block=self.srv.idle(), timeout=0.05 if self.srv.idle() else None)
                    self._handle(c)
            except queue.Empty:
                pass
            if self.srv.idle():
                continue
            for e in self.srv.step():
                t = self.ticket_of.get(e.request_id)
                if t is None:
                    continue
                if e.kind == "token":
                    self.out[t].put(("token", e.token_id))
                else:
                    self.out[t].put((e.kind, e.info))
                    self.srv.batcher.retire(e.request_id)
                    self.ticket_of.pop(e.request_id, None)
                    self.rid_of.pop(t, None)

    def _handle(self, c):
        if c[0] == "submit":
            _, t, kw = c
            try:
                rid = self.srv.submit(**kw)
                self.rid_of[t] = rid
                self.ticket_of[rid] = t
            except Exception as e:
                self.out[t].put(("error", {"message": str(e), "bad_request": True}))
        elif c[0] == "cancel":
            rid = self.rid_of.pop(c[1], None)
            if rid is not None and self.srv.cancel(rid):
                r = self.srv.request(rid)
                self.out[c[1]].put(("done", {"generated_ids": r["generated"], "finish_reason": "cancelled",
                                             "prompt_tokens": r["prompt_tokens"], "restored_tokens": r["restored_tokens"],
                                             "prefill_tokens": r["prefill_tokens"], "cache_checkpoint_tokens": 0}))
                self.ticket_of.pop(rid, None)
        elif c[0] == "stop":
            self.running = False


def create_app(serving, tokenizer, model_name: str, default_max_output_tokens: int, stop_ids: List[int], max_seq_len: int,
               max_in_flight: int = 0):
    """``max_in_flight`` > 0: requests beyond that many being generated or queued are answered with HTTP 429."""
    if FastAPI is None:
        raise RuntimeError("fastapi is required for phaseshift-server")
    app = FastAPI(title="phaseshift-b200")
    eng = EngineThread(serving)
    eng.start()
    app.state.engine_thread = eng

    def bad(msg: str, code: int = 400):
        return JSONResponse({"error": {"message": msg, "type": "invalid_request_error"}}, status_code=code)

    def overloaded():
        """Admission at the door: a bounded queue instead of an unbounded backlog (the client retries)."""
        if max_in_flight > 0 and len(eng.out) >= max_in_flight:
            return JSONResponse({"error": {"message": f"server is at its limit of {max_in_flight} requests in flight",
                                           "type": "rate_limit_error"}}, status_code=429, headers={"Retry-After": "1"})
        return None

    def prepare(body: dict):
        msgs = body.get("messages")
        if not isinstance(msgs, list):
            raise chat.RequestError("messages must be a list")
        # capabilities this server does not have are refused, not ignored (a client must not believe it got them)
        if body.get("n") not in (None, 1):
            raise chat.RequestError("n > 1 is not supported: one completion per request")
        if body.get("logprobs") or body.get("top_logprobs"):
            raise chat.RequestError("logprobs are not supported")
        if body.get("audio") is not None or any(m_ != "text" for m_ in (body.get("modalities") or ["text"])):
            raise chat.RequestError("only the text modality is supported")
        for key in ("temperature", "top_p"):
            v = body.get(key)
            if v is not None and (not isinstance(v, (int, float)) or isinstance(v, bool) or v < 0 or (key == "top_p" and v > 1)):
                raise chat.RequestError(f"{key} out of range")
        effort = body.get("reasoning_effort")
        if effort not in (None, "none", "low", "medium", "high"):
            raise chat.RequestError(f"unknown reasoning_effort {effort!r}")
        reasoning = effort in ("low", "medium", "high")
        tools, mode, forced = chat.validate_tools(body.get("tools"), body.get("tool_choice"))
        cons = chat.response_format_constraint(body.get("response_format"))
        if mode in ("required", "named"):
            if cons:
                raise chat.RequestError("response_format cannot be combined with a required tool call")
            cons = {"structural_tag": chat.structural_tag_for_tools(tools, forced, True)}
        elif mode == "auto" and tools and any(t["function"].get("strict") for t in tools):
            cons = cons or {"structural_tag": chat.structural_tag_for_tools(tools, None, False)}
        if cons and serving.constraints is None:
            raise chat.RequestError("structured output was requested but this server has no grammar engine configured")
        if "json_schema" in cons:      # the serving loop takes grammar / structural_tag; wrap the schema as a tag-less format
            cons = {"structural_tag": json.dumps({"type": "structural_tag",
                                                  "format": {"type": "json_schema", "json_schema": json.loads(cons["json_schema"])}})}
        stops = chat.parse_stop(body.get("stop"))
        rp = chat.render_prompt(tokenizer, msgs, tools if mode != "none" else None, reasoning)
        max_new = int(body.get("max_completion_tokens") or body.get("max_tokens") or default_max_output_tokens)
        if len(rp.ids) + 1 > max_seq_len:
            raise chat.RequestError(f"prompt of {len(rp.ids)} tokens exceeds the context window of {max_seq_len}")
        max_new = max(1, min(max_new, max_seq_len - len(rp.ids)))
        kw = dict(prompt=rp.ids, max_new_tokens=max_new, temperature=float(body.get("temperature") or 0.0),
                  top_p=float(body.get("top_p") or 1.0), top_k=int(body.get("top_k") or 0), seed=int(body.get("seed") or 0),
                  stop_tokens=stop_ids, checkpoint_position=rp.checkpoint_position, grammar=cons.get("grammar"),
                  structural_tag=cons.get("structural_tag"))
        body["_stops"] = stops
        return kw, reasoning, mode

    def finish_reason(info, has_calls: bool) -> str:
        if has_calls:
            return "tool_calls"
        return {"stop": "stop", "length": "length", "cancelled": "cancelled", "error": "error"}.get(info.get("finish_reason"), "stop")

    @app.get("/health")
    def health():
        return {"status": "ok"}

    @app.get("/metrics")
    def metrics():
        """Counters of the serving loop in the Prometheus text format (monitoring of a deployment; no upstream counterpart)."""
        from fastapi.responses import PlainTextResponse
        srv = getattr(serving, "srv", serving)                       # the tensor-parallel leader wraps the loop
        st = dict(getattr(srv, "stats", {}) or {})
        lines = []

        def put(name: str, kind: str, value, help_: str) -> None:
            lines.extend([f"# HELP phaseshift_{name} {help_}", f"# TYPE phaseshift_{name} {kind}", f"phaseshift_{name} {value}"])
        put("steps_total", "counter", st.get("steps", 0), "engine steps executed")
        put("generated_tokens_total", "counter", st.get("tokens", 0), "tokens sampled")
        put("prefill_tokens_total", "counter", st.get("prefill_tokens", 0), "prompt tokens prefilled (restored prefixes excluded)")
        put("failed_steps_total", "counter", st.get("failed_steps", 0), "steps that ended with a non-zero device status")
        b = getattr(srv, "batcher", None)
        if b is not None and hasattr(b, "active_count"):
            put("requests_active", "gauge", b.active_count(), "requests holding a sequence slot")
            put("requests_queued", "gauge", b.queued_count(), "requests waiting for admission")
            put("kv_pages_free", "gauge", b.free_pages(), "free pages of the key/value cache")
        pc = getattr(srv, "prefix", None)
        if pc is not None:
            sm = pc.summary()
            put("prefix_cache_hits_total", "counter", sm.get("hits", 0), "prompts that restored a cached prefix")
            put("prefix_cache_misses_total", "counter", sm.get("misses", 0), "prompts without a cached prefix")
            put("prefix_cache_tokens", "gauge", sm.get("used_tokens", 0), "tokens held by the prefix cache")
        put("requests_in_flight", "gauge", len(eng.ticket_of), "HTTP requests being generated")
        return PlainTextResponse("\n".join(lines) + "\n", media_type="text/plain; version=0.0.4")

    @app.get("/v1/models")
    def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "phaseshift-b200"}]}

    @app.get("/v1/models/{model_id}")
    def model_info(model_id: str):
        if model_id != model_name:
            return JSONResponse({"error": {"message": f"model {model_id!r} not found", "type": "invalid_request_error"}},
                                status_code=404)
        return {"id": model_name, "object": "model", "owned_by": "phaseshift-b200"}

    async def wait_item(q: "queue.Queue", request: Request, ticket: int):
        while True:
            try:
                return q.get_nowait()
            except queue.Empty:
                if await request.is_disconnected():
                    eng.cmd.put(("cancel", ticket))
                await asyncio.sleep(0.002)

    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request):
        try:
            body = await request.json()
            kw, reasoning, mode = prepare(body)
        except chat.RequestError as e:
            return bad(str(e))
        except Exception as e:
            return bad(f"malformed request: {e}")
        busy = overloaded()
        if busy is not None:
            return busy
        watcher = chat.StopWatcher(body.get("_stops") or [])
        t = eng.new_ticket()
        eng.cmd.put(("submit", t, kw))
        q = eng.out[t]
        cid, created = "chatcmpl-" + uuid.uuid4().hex[:24], int(time.time())
        think, tools_open = chat.StopWatcher([chat.THINK_CLOSE]), chat.StopWatcher([chat.TOOL_OPEN])

        def view(text: str, final: bool):
            """Decoded text so far -> (reasoning to show, answer to show, stop sequence complete?).  With reasoning on, the
            prompt ended with the opening tag: everything up to the closing tag is reasoning.  Stop sequences apply to
            the answer.  Text that may still become the closing tag or a stop sequence is held back until `final`."""
            r, ans = "", text
            if reasoning:
                k = text.find(chat.THINK_CLOSE)
                if k < 0:
                    return (text if final else text[:think.feed(text)[0]]).lstrip(), "", False
                r, ans = text[:k].lstrip(), text[k + len(chat.THINK_CLOSE):].lstrip()
            safe, hit = watcher.feed(ans)
            if hit is None and final:
                safe = len(ans)
            return r, ans[:safe], hit is not None

        def chunk(delta: dict, fin=None) -> str:
            return "data: " + json.dumps({"id": cid, "object": "chat.completion.chunk", "created": created, "model": model_name,
                                          "choices": [{"index": 0, "delta": delta, "finish_reason": fin}]}) + "\n\n"

        if body.get("stream"):
            async def gen():
                ids: List[int] = []
                sent_r = sent_a = 0
                cut = False                              # a stop sequence is complete
                yield chunk({"role": "assistant"})
                while True:
                    kind, val = await wait_item(q, request, t)
                    if kind == "token":
                        if cut:
                            continue                     # the request is being cancelled: nothing after the stop is shown
                        ids.append(val)
                        text = tokenizer.decode([i for i in ids if i not in stop_ids], skip_special_tokens=True)
                        if text.endswith("\ufffd"):
                            continue                     # incomplete UTF-8 sequence: wait for more bytes
                        r, a, cut = view(text, False)
                        if cut:
                            eng.cmd.put(("cancel", t))
                        if len(r) > sent_r:
                            yield chunk({"reasoning_content": r[sent_r:]})
                            sent_r = len(r)
                        if mode != "none":               # tool-call markup is not content: show the text in front of it only
                            a = a[:tools_open.feed(a)[0]]
                        if len(a) > sent_a:
                            yield chunk({"content": a[sent_a:]})
                            sent_a = len(a)
                        continue
                    if kind == "error":
                        yield "data: " + json.dumps({"error": {"message": val.get("message", "error")}}) + "\n\n"
                    else:
                        n_out = len(ids) if cut else len(val["generated_ids"])
                        if cut:
                            val = dict(val, finish_reason="stop")
                            text = tokenizer.decode([i for i in ids if i not in stop_ids], skip_special_tokens=True)
                        else:
                            text = tokenizer.decode([i for i in val["generated_ids"] if i not in stop_ids], skip_special_tokens=True)
                        r, a, _ = view(text, True)
                        calls = chat.parse_tool_calls(a)[1] if mode != "none" else []
                        if calls:
                            a = a[:a.find(chat.TOOL_OPEN)]
                        if len(r) > sent_r:
                            yield chunk({"reasoning_content": r[sent_r:]})
                        if len(a) > sent_a:              # what was held back as a possible tag or stop sequence
                            yield chunk({"content": a[sent_a:]})
                        yield chunk({"tool_calls": calls} if calls else {}, finish_reason(val, bool(calls)))
                        if (body.get("stream_options") or {}).get("include_usage"):
                            yield "data: " + json.dumps({"id": cid, "object": "chat.completion.chunk", "created": created,
                                                         "model": model_name, "choices": [],
                                                         "usage": {"prompt_tokens": val["prompt_tokens"], "completion_tokens": n_out,
                                                                   "total_tokens": val["prompt_tokens"] + n_out}}) + "\n\n"
                    yield "data: [DONE]\n\n"
                    eng.out.pop(t, None)
                    return
            return StreamingResponse(gen(), media_type="text/event-stream")
        seen: List[int] = []
        cut = False
        while True:
            kind, val = await wait_item(q, request, t)
            if kind == "token":
                if watcher.stops and not cut:
                    seen.append(val)
                    cut = view(tokenizer.decode([i for i in seen if i not in stop_ids], skip_special_tokens=True), False)[2]
                    if cut:
                        eng.cmd.put(("cancel", t))       # a stop sequence is complete: the rest is not needed
                continue
            eng.out.pop(t, None)
            if kind == "error":
                return bad(val.get("message", "error"), 400 if val.get("bad_request") else 500)
            if cut:
                val = dict(val, finish_reason="stop", generated_ids=seen)
            text = tokenizer.decode([i for i in val["generated_ids"] if i not in stop_ids], skip_special_tokens=True)
            reasoning_text, answer, hit = view(text, True)
            if hit:
                val = dict(val, finish_reason="stop")
            reasoning_text = reasoning_text.strip()
            answer, calls = chat.parse_tool_calls(answer) if mode != "none" else (answer, [])
            msg = {"role": "assistant", "content": answer or None if calls else answer}
            if calls:
                msg["tool_calls"] = calls
            if reasoning_text:
                msg["reasoning_content"] = reasoning_text
            return {"id": cid, "object": "chat.completion", "created": created, "model": model_name,
                    "choices": [{"index": 0, "message": msg, "finish_reason": finish_reason(val, bool(calls))}],
                    "usage": {"prompt_tokens": val["prompt_tokens"], "completion_tokens": len(val["generated_ids"]),
                              "total_tokens": val["prompt_tokens"] + len(val["generated_ids"]),
                              "prompt_tokens_details": {"cached_tokens": val.get("restored_tokens", 0)}}}

    def responses_to_chat(body: dict) -> dict:
        """Responses-API request -> the chat request `prepare` understands: input items (messages, function calls and their
        outputs), flat tool definitions, `text.format`, `reasoning.effort`."""
        inp = body.get("input")
        msgs: List[dict] = []
        if isinstance(inp, str):
            msgs.append({"role": "user", "content": inp})
        else:
            for it in list(inp or []):
                if not isinstance(it, dict):
                    raise chat.RequestError("input items must be objects")
                kind = it.get("type", "message")
                if kind == "message":
                    msgs.append({"role": it.get("role", "user"), "content": it.get("content")})
                elif kind == "function_call":
                    msgs.append({"role": "assistant", "content": None, "tool_calls": [
                        {"id": it.get("call_id"), "type": "function",
                         "function": {"name": it.get("name"), "arguments": it.get("arguments", "{}")}}]})
                elif kind == "function_call_output":
                    out = it.get("output")
                    msgs.append({"role": "tool", "tool_call_id": it.get("call_id"),
                                 "content": out if isinstance(out, str) else json.dumps(out)})
                else:
                    raise chat.RequestError(f"unsupported input item type {kind!r}")
        if body.get("instructions"):
            msgs = [{"role": "system", "content": body["instructions"]}] + msgs
        tools = None
        if body.get("tools") is not None:
            tools = []
            for t in body["tools"]:
                if isinstance(t, dict) and t.get("type") == "function" and "function" not in t:
                    t = {"type": "function", "function": {k: v for k, v in t.items() if k != "type"}}
                tools.append(t)
        choice = body.get("tool_choice")
        if isinstance(choice, dict) and choice.get("type") == "function" and "function" not in choice:
            choice = {"type": "function", "function": {"name": choice.get("name")}}
        fmt = (body.get("text") or {}).get("format")
        rf = None
        if isinstance(fmt, dict) and fmt.get("type") not in (None, "text"):
            rf = {"type": "json_schema", "json_schema": {"name": fmt.get("name", "response"), "schema": fmt.get("schema")}} \
                if fmt["type"] == "json_schema" else fmt
        return {"messages": msgs, "max_tokens": body.get("max_output_tokens"), "temperature": body.get("temperature"),
                "top_p": body.get("top_p"), "seed": body.get("seed"), "tools": tools, "tool_choice": choice,
                "response_format": rf, "reasoning_effort": (body.get("reasoning") or {}).get("effort")}

    def response_object(rid: str, created: int, val: dict, reasoning: bool, mode: str, status: Optional[str] = None) -> dict:
        text = tokenizer.decode([i for i in val["generated_ids"] if i not in stop_ids], skip_special_tokens=True)
        reasoning_text, answer = chat.split_reasoning(text, reasoning) if reasoning else ("", text)
        answer, calls = chat.parse_tool_calls(answer) if mode != "none" else (answer, [])
        output: List[dict] = []
        if reasoning_text:
            output.append({"type": "reasoning", "id": "rs_" + uuid.uuid4().hex[:24],
                           "summary": [{"type": "summary_text", "text": reasoning_text}]})
        if answer or not calls:
            output.append({"type": "message", "id": "msg_" + uuid.uuid4().hex[:24], "role": "assistant", "status": "completed",
                           "content": [{"type": "output_text", "text": answer, "annotations": []}]})
        for c in calls:
            output.append({"type": "function_call", "id": "fc_" + uuid.uuid4().hex[:24], "call_id": c["id"], "status": "completed",
                           "name": c["function"]["name"], "arguments": c["function"]["arguments"]})
        fr = val["finish_reason"]
        obj = {"id": rid, "object": "response", "created_at": created, "model": model_name,
               "status": status or {"stop": "completed", "length": "incomplete"}.get(fr, fr),
               "output": output, "output_text": answer,
               "usage": {"input_tokens": val["prompt_tokens"], "output_tokens": len(val["generated_ids"]),
                         "total_tokens": val["prompt_tokens"] + len(val["generated_ids"]),
                         "input_tokens_details": {"cached_tokens": val.get("restored_tokens", 0)}}}
        if fr == "length":
            obj["incomplete_details"] = {"reason": "max_output_tokens"}
        return obj

    @app.post("/v1/responses")
    async def responses(request: Request):
        try:
            body = await request.json()
            kw, reasoning, mode = prepare(responses_to_chat(body))
        except chat.RequestError as e:
            return bad(str(e))
        except Exception as e:
            return bad(f"malformed request: {e}")
        busy = overloaded()
        if busy is not None:
            return busy
        t = eng.new_ticket()
        eng.cmd.put(("submit", t, kw))
        q = eng.out[t]
        rid, created = "resp_" + uuid.uuid4().hex[:24], int(time.time())
        if body.get("stream"):
            def sse(event: str, payload: dict) -> str:
                return f"event: {event}\ndata: " + json.dumps(dict(payload, type=event)) + "\n\n"

            async def gen():
                ids: List[int] = []
                sent, seq = 0, 0
                shell = {"id": rid, "object": "response", "created_at": created, "model": model_name, "status": "in_progress",
                         "output": []}
                yield sse("response.created", {"sequence_number": seq, "response": shell})
                while True:
                    kind, val = await wait_item(q, request, t)
                    if kind == "token":
                        ids.append(val)
                        text = tokenizer.decode([i for i in ids if i not in stop_ids], skip_special_tokens=True)
                        if text.endswith("\ufffd"):
                            continue                     # incomplete UTF-8 sequence: wait for more bytes
                        delta, sent = text[sent:], len(text)
                        if delta:
                            seq += 1
                            yield sse("response.output_text.delta", {"sequence_number": seq, "output_index": 0,
                                                                     "content_index": 0, "delta": delta})
                        continue
                    eng.out.pop(t, None)
                    seq += 1
                    if kind == "error":
                        yield sse("error", {"sequence_number": seq, "message": val.get("message", "error")})
                        return
                    obj = response_object(rid, created, val, reasoning, mode)
                    yield sse("response.output_text.done", {"sequence_number": seq, "output_index": 0, "content_index": 0,
                                                            "text": obj["output_text"]})
                    final = "response.completed" if obj["status"] == "completed" else "response.incomplete"
                    yield sse(final, {"sequence_number": seq + 1, "response": obj})
                    return
            return StreamingResponse(gen(), media_type="text/event-stream")
        while True:
            kind, val = await wait_item(q, request, t)
            if kind == "token":
                continue
            eng.out.pop(t, None)
            if kind == "error":
                return bad(val.get("message", "error"), 400 if val.get("bad_request") else 500)
            return response_object(rid, created, val, reasoning, mode)

    return app


def load_tokenizer(model_dir: Optional[str], vocab_size: int):
    if model_dir:
        import os
        if any(os.path.exists(os.path.join(model_dir, f)) for f in ("tokenizer.json", "tokenizer_config.json")):
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(model_dir)
    return chat.ByteTokenizer(vocab_size)


def build_runtime(a):
    from .compute import ComputeRuntime
    ns = argparse.Namespace(model_dir=a.model_dir, random_model=a.random_model, preset=a.preset, device=a.device,
                            max_seq_len=a.max_seq_len, page_tokens=a.page_tokens, arena_gib=a.arena_gib,
                            max_concurrent_requests=a.max_concurrent_requests,
                            kv_cache_capacity_tokens=a.kv_cache_capacity_tokens or (a.max_concurrent_requests + 1) * (a.max_seq_len + 1),
                            kv_cache_dtype=a.kv_cache_dtype, prefix_cache_capacity_tokens=a.prefix_cache_capacity_tokens,
                            prefix_cache_max_entries=a.prefix_cache_max_entries, constraint_tokenizer_info=None,
                            verify_weights=a.verify_weights, dflash2_model_dir=a.dflash2_model_dir, dflash2_drafts=a.dflash2_drafts,
                            dflash2_ngram_tail=0, dflash2_ngram_n=0, max_scheduled_tokens=2048, tp=getattr(a, "tp", 1))
    rt = ComputeRuntime(ns)
    tok = load_tokenizer(a.model_dir, rt.cfg.vocab_size)
    try:
        from ..runtime.constraints import TokenConstraintCompiler
        if isinstance(tok, chat.ByteTokenizer):
            comp = TokenConstraintCompiler(tok.vocab_strings()[:rt.cfg.vocab_size], rt.cfg.vocab_size, [tok.eos_token_id], vocab_type="raw")
        else:
            comp = TokenConstraintCompiler.from_tokenizer(tok, rt.cfg.vocab_size, rt.cfg.eos_token_ids)
        rt.serving.constraints = comp
    except Exception as e:      # fail closed: structured requests will be rejected with 400
        print(f"[server] grammar engine unavailable: {e}", file=sys.stderr)
    stop = list(rt.cfg.eos_token_ids) or [getattr(tok, "eos_token_id", 2)]
    return rt, tok, stop


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    if not a.model_dir and not a.random_model:
        print("phaseshift-server: --model-dir is required", file=sys.stderr)
        return 2
    import uvicorn
    if a.tp > 1:
        if a.dflash2_model_dir:
            print("phaseshift-server: --tp with --dflash2-model-dir is not supported", file=sys.stderr)
            return 2
        from ..parallel.launch import spawn_ranks
        spawn_ranks(a.tp, "phaseshift_b200.apps.server", list(sys.argv[1:] if argv is None else argv))
    rt, tok, stop = build_runtime(a)
    if a.tp > 1:
        # rank 0 serves HTTP; the other ranks replay its commands (runtime/tp_serving.py)
        from ..runtime.tp_serving import TpServingLeader, follow
        if rt.rank != 0:
            follow(rt.serving, rt.host_group)
            return 0
        import atexit
        rt.serving = TpServingLeader(rt.serving, rt.host_group)
        atexit.register(rt.serving.shutdown)
    app = create_app(rt.serving, tok, a.model_name, a.default_max_output_tokens, stop, a.max_seq_len,
                     max_in_flight=a.max_concurrent_requests + a.max_queued_requests if a.max_queued_requests > 0 else 0)
    print(f"phaseshift-server: model={a.model_name} ctx={a.max_seq_len} concurrency={a.max_concurrent_requests} "
          f"prefix_cache={a.prefix_cache_capacity_tokens}x{a.prefix_cache_max_entries} http://{a.host}:{a.port}", file=sys.stderr)
    uvicorn.run(app, host=a.host, port=a.port, log_level="warning")
    return 0


if __name__ == "__main__":
    sys.exit(main())
