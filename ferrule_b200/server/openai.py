"""OpenAI-compatible request / response types with greedy-only validation.

Requests reject unknown fields.  Only exact greedy decoding is served: n = 1, temperature 0,
top_p 1, top_k 1 (or -1/0 = unset), min_p 0, repetition_penalty 1, no presence/frequency
penalties, no logprobs, tools, response_format, echo or best_of; at most 4 non-empty stop strings;
`max_tokens` defaults to 16.  Finish reasons map: max tokens / context -> "length";
EOS / stop string / no candidate -> "stop"; cancelled -> "cancelled".  Errors use the OpenAI
envelope `{"error": {"message", "type", "param", "code"}}`.

Counterpart of crates/ferrule-server/src/openai.rs:140-205, :237-356 (validation), :373-479
(chunks, responses, usage), :526-534 (finish reason mapping).
"""
from __future__ import annotations

import uuid
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..runtime.session import FinishReason
from ..utils.tokenizer import ChatMessage

DEFAULT_MAX_TOKENS = 16
MAX_STOP = 4


class RequestError(ValueError):
    def __init__(self, message: str, param: Optional[str] = None, code: Optional[str] = None, status: int = 400,
                 etype: str = "invalid_request_error"):
        super().__init__(message)
        self.message, self.param, self.code, self.status, self.etype = message, param, code, status, etype

    def envelope(self) -> Dict[str, Any]:
        return {"error": {"message": self.message, "type": self.etype, "param": self.param, "code": self.code}}


_COMMON = {"model", "max_tokens", "max_completion_tokens", "stream", "stream_options", "stop", "n", "temperature",
           "top_p", "top_k", "min_p", "repetition_penalty", "presence_penalty", "frequency_penalty", "logprobs",
           "top_logprobs", "seed", "user", "ignore_eos", "session_id", "return_token_ids"}
_CHAT_ONLY = {"messages", "tools", "tool_choice", "response_format", "functions", "function_call"}
_COMPLETION_ONLY = {"prompt", "echo", "best_of", "suffix", "logit_bias"}


def _num(body: Dict[str, Any], key: str, expected: float, also=()) -> None:
    v = body.get(key)
    if v is None:
        return
    if not isinstance(v, (int, float)) or isinstance(v, bool) or (float(v) != expected and v not in also):
        raise RequestError(f"only greedy decoding is supported: `{key}` must be {expected:g}", key, "unsupported_value")


def _validate_sampling(body: Dict[str, Any]) -> None:
    _num(body, "n", 1)
    _num(body, "temperature", 0)
    _num(body, "top_p", 1)
    _num(body, "top_k", 1, also=(0, -1))
    _num(body, "min_p", 0)
    _num(body, "repetition_penalty", 1)
    _num(body, "presence_penalty", 0)
    _num(body, "frequency_penalty", 0)
    _num(body, "best_of", 1)
    if body.get("logprobs") not in (None, False, 0):
        raise RequestError("`logprobs` is not supported", "logprobs", "unsupported_parameter")
    if body.get("top_logprobs") not in (None, 0):
        raise RequestError("`top_logprobs` is not supported", "top_logprobs", "unsupported_parameter")
    for key in ("tools", "tool_choice", "functions", "function_call", "response_format", "logit_bias", "suffix"):
        if body.get(key) not in (None, [], {}):
            raise RequestError(f"`{key}` is not supported", key, "unsupported_parameter")
    if body.get("echo") not in (None, False):
        raise RequestError("`echo` is not supported", "echo", "unsupported_parameter")


def _stops(body: Dict[str, Any]) -> List[str]:
    s = body.get("stop")
    if s is None:
        return []
    if isinstance(s, str):
        s = [s]
    if not isinstance(s, list) or any(not isinstance(x, str) for x in s):
        raise RequestError("`stop` must be a string or a list of strings", "stop")
    if len(s) > MAX_STOP:
        raise RequestError(f"at most {MAX_STOP} stop strings are supported", "stop")
    if any(x == "" for x in s):
        raise RequestError("stop strings must be non-empty", "stop")
    return s


def _max_tokens(body: Dict[str, Any]) -> int:
    v = body.get("max_completion_tokens", body.get("max_tokens"))
    if v is None:
        return DEFAULT_MAX_TOKENS
    if not isinstance(v, int) or isinstance(v, bool) or v < 1:
        raise RequestError("`max_tokens` must be a positive integer", "max_tokens")
    return v


@dataclass
class ParsedRequest:
    kind: str                      # "chat" | "completion"
    model: str
    prompt_text: Optional[str]
    prompt_tokens: Optional[List[int]]
    messages: List[ChatMessage]
    max_tokens: int
    stop: List[str]
    stream: bool
    include_usage: bool
    ignore_eos: bool
    session_id: Optional[str]
    return_token_ids: bool = False        # extension: stream every committed token id (chunks may carry empty text)


def _check_fields(body: Any, allowed: set) -> Dict[str, Any]:
    if not isinstance(body, dict):
        raise RequestError("request body must be a JSON object")
    unknown = sorted(set(body) - allowed)
    if unknown:
        raise RequestError(f"unknown field `{unknown[0]}`", unknown[0], "unknown_field")
    return body


def _stream_opts(body: Dict[str, Any]) -> Tuple[bool, bool]:
    stream = bool(body.get("stream", False))
    so = body.get("stream_options")
    include = False
    if so is not None:
        if not isinstance(so, dict) or set(so) - {"include_usage"}:
            raise RequestError("`stream_options` only supports `include_usage`", "stream_options")
        if not stream:
            raise RequestError("`stream_options` requires `stream: true`", "stream_options")
        include = bool(so.get("include_usage", False))
    return stream, include


def parse_chat_request(body: Any) -> ParsedRequest:
    body = _check_fields(body, _COMMON | _CHAT_ONLY)
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise RequestError("`messages` must be a non-empty list", "messages")
    out = []
    for i, m in enumerate(msgs):
        if not isinstance(m, dict) or set(m) - {"role", "content", "name"}:
            raise RequestError(f"messages[{i}] has unsupported fields", "messages")
        if m.get("role") not in ("system", "user", "assistant"):
            raise RequestError(f"messages[{i}].role must be system, user or assistant", "messages")
        if not isinstance(m.get("content"), str):
            raise RequestError(f"messages[{i}].content must be a string", "messages")
        out.append(ChatMessage(m["role"], m["content"]))
    _validate_sampling(body)
    stream, include = _stream_opts(body)
    return ParsedRequest("chat", str(body.get("model", "")), None, None, out, _max_tokens(body), _stops(body), stream,
                         include, bool(body.get("ignore_eos", False)), body.get("session_id"),
                         bool(body.get("return_token_ids", False)))


def parse_completion_request(body: Any) -> ParsedRequest:
    body = _check_fields(body, _COMMON | _COMPLETION_ONLY)
    p = body.get("prompt")
    text, toks = None, None
    if isinstance(p, str):
        text = p
    elif isinstance(p, list) and p and all(isinstance(x, int) and not isinstance(x, bool) for x in p):
        toks = list(p)
    elif isinstance(p, list) and len(p) == 1 and isinstance(p[0], str):
        text = p[0]
    else:
        raise RequestError("`prompt` must be a string or a list of token ids", "prompt")
    _validate_sampling(body)
    stream, include = _stream_opts(body)
    return ParsedRequest("completion", str(body.get("model", "")), text, toks, [], _max_tokens(body), _stops(body),
                         stream, include, bool(body.get("ignore_eos", False)), body.get("session_id"),
                         bool(body.get("return_token_ids", False)))


def finish_reason(reason: FinishReason) -> str:
    return reason.openai()


def new_id(kind: str) -> str:
    return ("chatcmpl-" if kind == "chat" else "cmpl-") + uuid.uuid4().hex[:24]


def usage(prompt_tokens: int, completion_tokens: int) -> Dict[str, int]:
    return {"prompt_tokens": prompt_tokens, "completion_tokens": completion_tokens,
            "total_tokens": prompt_tokens + completion_tokens}


def chat_chunk(rid: str, model: str, created: int, delta: Dict[str, Any], finish: Optional[str] = None,
               usage_obj: Optional[Dict[str, int]] = None, empty_choices: bool = False) -> Dict[str, Any]:
    d = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": model,
         "choices": [] if empty_choices else [{"index": 0, "delta": delta, "finish_reason": finish}]}
    if usage_obj is not None:
        d["usage"] = usage_obj
    return d


def completion_chunk(rid: str, model: str, created: int, text: str, finish: Optional[str] = None,
                     usage_obj: Optional[Dict[str, int]] = None, empty_choices: bool = False) -> Dict[str, Any]:
    d = {"id": rid, "object": "text_completion", "created": created, "model": model,
         "choices": [] if empty_choices else [{"index": 0, "text": text, "finish_reason": finish, "logprobs": None}]}
    if usage_obj is not None:
        d["usage"] = usage_obj
    return d


def chat_response(rid: str, model: str, created: int, text: str, finish: str, u: Dict[str, int]) -> Dict[str, Any]:
    return {"id": rid, "object": "chat.completion", "created": created, "model": model,
            "choices": [{"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": finish}],
            "usage": u}


def completion_response(rid: str, model: str, created: int, text: str, finish: str, u: Dict[str, int]) -> Dict[str, Any]:
    return {"id": rid, "object": "text_completion", "created": created, "model": model,
            "choices": [{"index": 0, "text": text, "finish_reason": finish, "logprobs": None}], "usage": u}
