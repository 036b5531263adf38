"""Chat codec and tool-call constraints for the OpenAI-compatible server.

Behaviour follows the reference's Python edge (src/apps/common/phaseshift_chat/codec.py:120-333,
tool_constraint.py:39-422): render messages to prompt ids with a *stable prefix-cache boundary* (the
history rendered without the generation prompt, used only when it is an exact token prefix of the full
prompt), optional reasoning (``<think>...</think>``) split, tool-call parsing, ``tool_choice`` policy with
strict-schema validation, and grammar / structural-tag builders that constrain generation to a valid call.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
TOOL_OPEN, TOOL_CLOSE = "<tool_call>", "</tool_call>"


class RequestError(ValueError):
    """Maps to HTTP 400: rejected before generation starts."""


class ByteTokenizer:
    """Fallback tokenizer for model directories without tokenizer assets (tests, random-init models):
    token = byte + 3; ids 0/1/2 = pad/bos/eos."""
    eos_token_id = 2

    def __init__(self, vocab_size: int = 259):
        self.vocab_size = max(vocab_size, 259)

    def encode(self, text: str) -> List[int]:
        return [b + 3 for b in text.encode("utf-8")]

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return bytes(i - 3 for i in ids if 3 <= i < 259).decode("utf-8", "replace")

    def apply_chat_template(self, messages, add_generation_prompt=True, tokenize=True, tools=None, **kw):
        text = ""
        if tools:
            text += "<|tools|>" + json.dumps(tools, sort_keys=True) + "\n"
        for m in messages:
            text += f"<|{m['role']}|>{_content_text(m)}\n"
        if add_generation_prompt:
            text += "<|assistant|>"
        return self.encode(text) if tokenize else text

    def vocab_strings(self) -> List[str]:
        return ["<pad>", "<bos>", "<eos>"] + [chr(b) if b < 128 else f"<0x{b:02X}>" for b in range(256)] + \
               [f"<extra_{i}>" for i in range(self.vocab_size - 259)]


def _content_text(m: dict) -> str:
    c = m.get("content")
    if c is None:
        c = ""
    if isinstance(c, list):
        parts = []
        for p in c:
            if p.get("type") not in ("text", "input_text", "output_text"):
                raise RequestError(f"unsupported content part type {p.get('type')!r} (text only)")
            parts.append(p.get("text", ""))
        c = "".join(parts)
    if m.get("tool_calls"):
        for tc in m["tool_calls"]:
            fn = tc.get("function", {})
            c += TOOL_OPEN + json.dumps({"name": fn.get("name"), "arguments": _maybe_json(fn.get("arguments"))}) + TOOL_CLOSE
    return c


def _maybe_json(s):
    if isinstance(s, str):
        try:
            return json.loads(s)
        except Exception:
            return s
    return s


@dataclass
class RenderedPrompt:
    ids: List[int]
    checkpoint_position: int = 0      # 0 = no stable boundary


def render_prompt(tok, messages: List[dict], tools: Optional[List[dict]] = None, reasoning: bool = False) -> RenderedPrompt:
    if not messages:
        raise RequestError("messages must not be empty")
    for m in messages:
        if m.get("role") not in ("system", "user", "assistant", "tool", "developer"):
            raise RequestError(f"unknown role {m.get('role')!r}")
    kw = {"tools": tools} if tools else {}
    full = list(tok.apply_chat_template(messages, add_generation_prompt=True, tokenize=True, **kw))
    if reasoning:
        full += tok.encode(THINK_OPEN) if hasattr(tok, "encode") else []
    boundary = 0
    # history = everything before the last user turn; stable across the next request of the same conversation
    last_user = max((i for i, m in enumerate(messages) if m["role"] == "user"), default=-1)
    if last_user > 0:
        hist = list(tok.apply_chat_template(messages[:last_user], add_generation_prompt=False, tokenize=True, **kw))
        if len(hist) < len(full) and full[:len(hist)] == hist:
            boundary = len(hist)
    return RenderedPrompt(full, boundary)


def split_reasoning(text: str, opened: bool) -> Tuple[str, str]:
    """(reasoning, answer).  ``opened``: the prompt already ended with <think>."""
    if opened:
        if THINK_CLOSE in text:
            r, a = text.split(THINK_CLOSE, 1)
            return r.strip(), a.lstrip()
        return text.strip(), ""
    m = re.search(re.escape(THINK_OPEN) + r"(.*?)" + re.escape(THINK_CLOSE), text, re.S)
    if m:
        return m.group(1).strip(), (text[:m.start()] + text[m.end():]).strip()
    return "", text


def parse_tool_calls(text: str) -> Tuple[str, List[dict]]:
    calls = []
    for i, m in enumerate(re.finditer(re.escape(TOOL_OPEN) + r"(.*?)" + re.escape(TOOL_CLOSE), text, re.S)):
        try:
            obj = json.loads(m.group(1))
            calls.append({"id": f"call_{i}", "type": "function",
                          "function": {"name": obj["name"], "arguments": json.dumps(obj.get("arguments", {}))}})
        except Exception:
            continue
    rest = re.sub(re.escape(TOOL_OPEN) + r".*?" + re.escape(TOOL_CLOSE), "", text, flags=re.S).strip()
    return rest, calls


# ------------------------------------------------------------------------------------------------ tools
def validate_tools(tools: Optional[List[dict]], tool_choice) -> Tuple[List[dict], str, Optional[str]]:
    """Returns (tools, mode, forced_name) with mode in none|auto|required|named.  Raises RequestError on a
    malformed tool list, an unknown tool name or a schema strict mode cannot honour."""
    tools = tools or []
    names = set()
    for t in tools:
        if t.get("type") != "function" or "function" not in t or not t["function"].get("name"):
            raise RequestError("every tool must be {type: function, function: {name, parameters}}")
        fn = t["function"]
        if fn["name"] in names:
            raise RequestError(f"duplicate tool name {fn['name']!r}")
        names.add(fn["name"])
        params = fn.get("parameters", {"type": "object"})
        if not isinstance(params, dict) or params.get("type", "object") != "object":
            raise RequestError(f"tool {fn['name']!r}: parameters must be a JSON schema of type object")
        if fn.get("strict"):
            if params.get("additionalProperties", False) is not False:
                raise RequestError(f"tool {fn['name']!r}: strict mode requires additionalProperties: false")
            req = set(params.get("required", []))
            if set(params.get("properties", {})) != req:
                raise RequestError(f"tool {fn['name']!r}: strict mode requires every property to be listed in required")
    if tool_choice in (None, "auto"):
        return tools, ("auto" if tools else "none"), None
    if tool_choice == "none":
        return tools, "none", None
    if tool_choice == "required":
        if not tools:
            raise RequestError("tool_choice=required needs at least one tool")
        return tools, "required", None
    if isinstance(tool_choice, dict) and tool_choice.get("type") == "function":
        n = tool_choice.get("function", {}).get("name")
        if n not in names:
            raise RequestError(f"tool_choice names unknown tool {n!r}")
        return tools, "named", n
    raise RequestError(f"unsupported tool_choice {tool_choice!r}")


def tool_call_schema(tools: List[dict], forced: Optional[str]) -> dict:
    """JSON schema of one call object {name, arguments} over the allowed tools."""
    alts = []
    for t in tools:
        fn = t["function"]
        if forced and fn["name"] != forced:
            continue
        alts.append({"type": "object", "properties": {"name": {"const": fn["name"]},
                                                       "arguments": fn.get("parameters", {"type": "object"})},
                     "required": ["name", "arguments"], "additionalProperties": False})
    return alts[0] if len(alts) == 1 else {"anyOf": alts}


def structural_tag_for_tools(tools: List[dict], forced: Optional[str], required: bool) -> str:
    """Structural-tag JSON for XGrammar: free text with ``<tool_call>{schema-constrained json}</tool_call>``
    segments (at least one when a call is required)."""
    tags = []
    for t in tools:
        fn = t["function"]
        if forced and fn["name"] != forced:
            continue
        schema = {"type": "object", "properties": {"name": {"const": fn["name"]},
                                                    "arguments": fn.get("parameters", {"type": "object"})},
                  "required": ["name", "arguments"], "additionalProperties": False}
        tags.append({"type": "tag", "begin": TOOL_OPEN, "content": {"type": "json_schema", "json_schema": schema},
                     "end": TOOL_CLOSE})
    fmt = {"type": "triggered_tags", "triggers": [TOOL_OPEN], "tags": tags, "at_least_one": bool(required or forced),
           "stop_after_first": bool(forced)}
    return json.dumps({"type": "structural_tag", "format": fmt})


def response_format_constraint(rf: Optional[dict]) -> Dict[str, Optional[str]]:
    """OpenAI response_format -> {json_schema | grammar}.  Unknown types are rejected."""
    if not rf or rf.get("type") in (None, "text"):
        return {}
    if rf["type"] == "json_object":
        return {"json_schema": json.dumps({"type": "object"})}
    if rf["type"] == "json_schema":
        js = rf.get("json_schema", {})
        if "schema" not in js:
            raise RequestError("response_format.json_schema.schema is required")
        return {"json_schema": json.dumps(js["schema"])}
    if rf["type"] in ("gbnf", "grammar"):
        if not rf.get("grammar"):
            raise RequestError("response_format.grammar is required")
        return {"grammar": rf["grammar"]}
    raise RequestError(f"unsupported response_format type {rf['type']!r}")


# ------------------------------------------------------------------------------------------------ stop sequences
def parse_stop(stop) -> List[str]:
    """OpenAI `stop`: a string or up to four strings."""
    if stop is None:
        return []
    if isinstance(stop, str):
        stop = [stop]
    if not isinstance(stop, list) or len(stop) > 4 or not all(isinstance(x, str) and x for x in stop):
        raise RequestError("stop must be a non-empty string or a list of up to 4 non-empty strings")
    return list(stop)


class StopWatcher:
    """Text-level stop sequences over a growing decoded text.  `feed(text)` returns (safe, hit): `safe` = how many
    characters may be shown (text that could still turn out to be the beginning of a stop sequence is held back), `hit` =
    index of the earliest stop sequence once one is complete (the answer is text[:hit]), else None."""

    def __init__(self, stops: Sequence[str]):
        self.stops = list(stops)
        self.hold = max((len(x) for x in self.stops), default=1) - 1

    def feed(self, text: str) -> Tuple[int, Optional[int]]:
        hits = [i for i in (text.find(x) for x in self.stops) if i >= 0]
        if hits:
            return min(hits), min(hits)
        if not self.stops:
            return len(text), None
        safe = len(text)
        for x in self.stops:                       # hold back the longest tail of `text` that is a proper prefix of a stop
            for k in range(min(len(x) - 1, len(text)), 0, -1):
                if text.endswith(x[:k]):
                    safe = min(safe, len(text) - k)
                    break
        return safe, None
