"""OpenAI-compatible HTTP / SSE front end (ASGI, Starlette).

Routes: GET /health, GET /v1/models, POST /v1/chat/completions, POST /v1/completions,
POST /v1/tokenize and /tokenize.  Streaming responses are server-sent events
(`data: {json}\\n\\n`, terminated by `data: [DONE]`), with a comment line as keep-alive while the
model is busy; an optional final usage chunk is sent when `stream_options.include_usage` is set.
When the client disconnects the request is cancelled in the engine.  Errors use the OpenAI
envelope.

Counterpart of crates/ferrule-server/src/http.rs:47-72 (router), :90-141 (chat), :349-351, :580, :747
(SSE framing, keep-alive, [DONE]), :517-540 (disconnect guard), :876-910 (error envelope).
"""
from __future__ import annotations

import asyncio
import json
import time
from typing import Any, AsyncIterator, Dict, Optional

from starlette.applications import Starlette
from starlette.requests import Request
from starlette.responses import JSONResponse, Response, StreamingResponse
from starlette.routing import Route

from ..utils.tokenizer import ChatTemplate, render_chat, template_for_model
from . import openai as oa
from .worker import ModelWorker, WorkerError

KEEPALIVE_S = 10.0


def _error(exc: Exception) -> JSONResponse:
    if isinstance(exc, oa.RequestError):
        return JSONResponse(exc.envelope(), status_code=exc.status)
    if isinstance(exc, WorkerError):
        etype = "invalid_request_error" if exc.status == 400 else "server_error"
        return JSONResponse({"error": {"message": str(exc), "type": etype, "param": None, "code": exc.code}},
                            status_code=exc.status)
    return JSONResponse({"error": {"message": str(exc), "type": "server_error", "param": None, "code": "internal_error"}},
                        status_code=500)


async def _json_body(request: Request) -> Any:
    try:
        return json.loads(await request.body())
    except ValueError:
        raise oa.RequestError("request body is not valid JSON", code="invalid_json")


def _sse(obj: Dict[str, Any]) -> bytes:
    return b"data: " + json.dumps(obj, separators=(",", ":"), ensure_ascii=False).encode() + b"\n\n"


def build_app(worker: ModelWorker, model_name: Optional[str] = None, template: Optional[ChatTemplate] = None,
              keepalive_s: float = KEEPALIVE_S) -> Starlette:
    name = model_name or worker.model_name
    tmpl = template or template_for_model(name)

    async def health(request: Request) -> Response:
        ok = worker.healthy
        return JSONResponse({"status": "ok" if ok else "unhealthy"}, status_code=200 if ok else 503)

    async def models(request: Request) -> Response:
        return JSONResponse({"object": "list", "data": [{"id": name, "object": "model", "created": 0,
                                                         "owned_by": "ferrule_b200"}]})

    async def tokenize(request: Request) -> Response:
        try:
            body = await _json_body(request)
            if not isinstance(body, dict) or set(body) - {"model", "prompt", "text", "add_special_tokens"}:
                raise oa.RequestError("tokenize accepts `model` and `prompt`")
            text = body.get("prompt", body.get("text"))
            if not isinstance(text, str):
                raise oa.RequestError("`prompt` must be a string", "prompt")
            ids = worker.tokenize(text)
            return JSONResponse({"tokens": ids, "count": len(ids), "max_model_len": worker.engine.cfg.scheduler.ctx_size})
        except Exception as exc:  # noqa: BLE001
            return _error(exc)

    async def _run(request: Request, parsed: oa.ParsedRequest) -> Response:
        if parsed.model and parsed.model != name:
            raise oa.RequestError(f"model `{parsed.model}` is not served here", "model", "model_not_found", 404)
        if parsed.kind == "chat":
            text, toks = render_chat(parsed.messages, tmpl), None
        else:
            text, toks = parsed.prompt_text, parsed.prompt_tokens
        rid = oa.new_id(parsed.kind)
        created = int(time.time())
        stream = await worker.submit(text=text, token_ids=toks, max_tokens=parsed.max_tokens, stop=parsed.stop,
                                     ignore_eos=parsed.ignore_eos, session_id=parsed.session_id, request_id=rid)
        chat = parsed.kind == "chat"
        if not parsed.stream:
            parts, n = [], 0
            try:
                while True:
                    if await request.is_disconnected():
                        stream.close()
                        return Response(status_code=499)
                    try:
                        ev = await asyncio.wait_for(stream.next(), 1.0)
                    except asyncio.TimeoutError:
                        continue
                    if ev.kind == "token":
                        parts.append(ev.text)
                    elif ev.kind == "error":
                        raise WorkerError(ev.message, 500, "engine_failure")
                    else:
                        u = oa.usage(ev.prompt_tokens or stream.prompt_tokens, ev.completion_tokens)
                        fr = oa.finish_reason(ev.reason)
                        text_out = "".join(parts)
                        body = (oa.chat_response if chat else oa.completion_response)(rid, name, created, text_out, fr, u)
                        return JSONResponse(body)
            except asyncio.CancelledError:
                stream.close()
                raise

        async def gen() -> AsyncIterator[bytes]:
            try:
                if chat:
                    yield _sse(oa.chat_chunk(rid, name, created, {"role": "assistant", "content": ""}))
                while True:
                    try:
                        ev = await asyncio.wait_for(stream.next(), keepalive_s)
                    except asyncio.TimeoutError:
                        yield b": keep-alive\n\n"
                        continue
                    if ev.kind == "token":
                        if ev.text or (parsed.return_token_ids and ev.token >= 0):
                            obj = (oa.chat_chunk(rid, name, created, {"content": ev.text}) if chat
                                   else oa.completion_chunk(rid, name, created, ev.text))
                            if parsed.return_token_ids and ev.token >= 0:
                                obj["token_ids"] = [ev.token]
                            yield _sse(obj)
                    elif ev.kind == "error":
                        yield _sse({"error": {"message": ev.message, "type": "server_error", "param": None,
                                              "code": "engine_failure"}})
                        break
                    else:
                        fr = oa.finish_reason(ev.reason)
                        yield _sse(oa.chat_chunk(rid, name, created, {}, fr) if chat
                                   else oa.completion_chunk(rid, name, created, "", fr))
                        if parsed.include_usage:
                            u = oa.usage(ev.prompt_tokens or stream.prompt_tokens, ev.completion_tokens)
                            yield _sse(oa.chat_chunk(rid, name, created, {}, None, u, empty_choices=True) if chat
                                       else oa.completion_chunk(rid, name, created, "", None, u, empty_choices=True))
                        break
                yield b"data: [DONE]\n\n"
            finally:
                stream.close()          # no-op after a normal finish; cancels on disconnect

        return StreamingResponse(gen(), media_type="text/event-stream",
                                 headers={"Cache-Control": "no-cache", "X-Accel-Buffering": "no"})

    async def chat_completions(request: Request) -> Response:
        try:
            return await _run(request, oa.parse_chat_request(await _json_body(request)))
        except Exception as exc:  # noqa: BLE001
            return _error(exc)

    async def completions(request: Request) -> Response:
        try:
            return await _run(request, oa.parse_completion_request(await _json_body(request)))
        except Exception as exc:  # noqa: BLE001
            return _error(exc)

    async def metrics(request: Request) -> Response:
        from ..utils.observability import METRICS
        return JSONResponse({"metrics": METRICS.snapshot(), "worker": worker.stats()})

    return Starlette(routes=[
        Route("/health", health, methods=["GET"]),
        Route("/v1/models", models, methods=["GET"]),
        Route("/v1/chat/completions", chat_completions, methods=["POST"]),
        Route("/v1/completions", completions, methods=["POST"]),
        Route("/v1/tokenize", tokenize, methods=["POST"]),
        Route("/tokenize", tokenize, methods=["POST"]),
        Route("/metrics", metrics, methods=["GET"]),
    ])


def serve(worker: ModelWorker, host: str = "127.0.0.1", port: int = 8000, model_name: Optional[str] = None,
          log_level: str = "warning", template: Optional[ChatTemplate] = None) -> None:
    """Blocking: run the ASGI app under uvicorn until interrupted, then stop the worker."""
    import uvicorn
    app = build_app(worker, model_name, template)
    try:
        uvicorn.run(app, host=host, port=port, log_level=log_level)
    finally:
        worker.stop()
