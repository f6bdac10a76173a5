"""OpenAI-compatible HTTP service (FastAPI) on top of ``YvInferenceEngine``.

Endpoints follow the reference service (tools/infer/server.py:312-405): ``/v1/models``, ``/v1/chat/completions``
(with SSE streaming: ``chat.completion.chunk`` events then ``[DONE]``, :500-538), ``/v1/completions``,
``/v1/embeddings``, ``/healthz``, ``/readyz``, ``/stats``.  The chat prompt is the ``[role]: content`` lines joined
by newlines (:1077-1084).  One background thread drives the engine's scheduler so that concurrent requests are
batched; handlers wait on their request object.
"""
from __future__ import annotations

import asyncio
import json
import threading
import time
import uuid
from typing import Any, Dict, List, Optional

from pydantic import BaseModel, Field

from ..models.generation import YvSamplingConfig
from .engine import YvEngineConfig, YvInferenceEngine


class PiscesLxChatMessage(BaseModel):
    role: str = "user"
    content: str = ""


class PiscesLxChatCompletionRequest(BaseModel):
    model: str = "yv"
    messages: List[PiscesLxChatMessage] = Field(default_factory=list)
    max_tokens: int = 128
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    stream: bool = False
    stop: Optional[List[str]] = None


class PiscesLxCompletionRequest(BaseModel):
    model: str = "yv"
    prompt: str = ""
    max_tokens: int = 128
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    stream: bool = False


class PiscesLxEmbeddingRequest(BaseModel):
    model: str = "yv"
    input: Any = ""


class PiscesLxInferService:
    def __init__(self, engine: YvInferenceEngine, model_name: str = "yv"):
        self.engine, self.model_name = engine, model_name
        self._stop = False
        self._wake = threading.Event()
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self.started = time.time()
        self.ready = False

    def _loop(self) -> None:
        self.ready = True
        while not self._stop:
            if self.engine.has_work():
                try:
                    self.engine.step()
                except Exception as e:  # keep serving; the failing requests are closed with an error
                    self.engine.stats["errors"] += 1
                    for r in list(self.engine.running) + list(self.engine.waiting):
                        r.finished, r.finish_reason = True, f"error: {e}"
                    self.engine.running.clear()
                    self.engine.waiting.clear()
            else:
                self._wake.wait(0.005)
                self._wake.clear()

    def start(self) -> None:
        if not self._thread.is_alive():
            self._thread.start()

    def stop(self) -> None:
        self._stop = True
        self._wake.set()

    def _sampling(self, temperature: float, top_k: int, top_p: float) -> YvSamplingConfig:
        if temperature <= 0:
            return YvSamplingConfig(strategy="greedy")
        return YvSamplingConfig(strategy="top_k_top_p", temperature=temperature, top_k=top_k, top_p=top_p)

    def submit(self, prompt: str, max_tokens: int, temperature: float, top_k: int, top_p: float, on_token=None):
        ids = self.engine.tokenizer.encode(prompt)
        req = self.engine.add_request(ids, max_tokens, self._sampling(temperature, top_k, top_p), on_token=on_token)
        self._wake.set()
        return req

    @staticmethod
    def chat_prompt(messages: List[PiscesLxChatMessage]) -> str:
        return "\n".join(f"[{m.role}]: {m.content}" for m in messages)

    # ---- app ----------------------------------------------------------------------------------------------
    def build_app(self):
        from fastapi import FastAPI
        from fastapi.responses import JSONResponse, StreamingResponse

        app = FastAPI(title="pisceslx_b200 inference service")
        svc = self

        @app.on_event("startup")
        async def _startup() -> None:
            svc.start()

        @app.get("/healthz")
        async def healthz():
            return {"status": "ok", "uptime": time.time() - svc.started}

        @app.get("/readyz")
        async def readyz():
            return JSONResponse({"ready": svc.ready}, status_code=200 if svc.ready else 503)

        @app.get("/stats")
        async def stats():
            return svc.engine.get_stats()

        @app.get("/v1/models")
        async def models():
            return {"object": "list", "data": [{"id": svc.model_name, "object": "model", "owned_by": "pisceslx_b200"}]}

        async def _wait(req) -> None:
            while not req.finished:
                await asyncio.sleep(0.002)

        def _usage(req) -> Dict[str, int]:
            return {"prompt_tokens": len(req.prompt_ids), "completion_tokens": len(req.output_ids),
                    "total_tokens": len(req.prompt_ids) + len(req.output_ids)}

        @app.post("/v1/chat/completions")
        async def chat(body: PiscesLxChatCompletionRequest):
            prompt = svc.chat_prompt(body.messages)
            cid = "chatcmpl-" + uuid.uuid4().hex[:24]
            if body.stream:
                async def gen():
                    req = svc.submit(prompt, body.max_tokens, body.temperature, body.top_k, body.top_p)
                    sent = 0
                    while not req.finished or sent < len(req.output_ids):
                        while sent < len(req.output_ids):
                            piece = svc.engine.tokenizer.decode([req.output_ids[sent]])
                            sent += 1
                            chunk = {"id": cid, "object": "chat.completion.chunk", "created": int(time.time()),
                                     "model": body.model,
                                     "choices": [{"index": 0, "delta": {"content": piece}, "finish_reason": None}]}
                            yield f"data: {json.dumps(chunk)}\n\n"
                        await asyncio.sleep(0.002)
                    end = {"id": cid, "object": "chat.completion.chunk", "created": int(time.time()), "model": body.model,
                           "choices": [{"index": 0, "delta": {}, "finish_reason": req.finish_reason}]}
                    yield f"data: {json.dumps(end)}\n\n"
                    yield "data: [DONE]\n\n"
                return StreamingResponse(gen(), media_type="text/event-stream")
            req = svc.submit(prompt, body.max_tokens, body.temperature, body.top_k, body.top_p)
            await _wait(req)
            return {"id": cid, "object": "chat.completion", "created": int(time.time()), "model": body.model,
                    "choices": [{"index": 0, "message": {"role": "assistant",
                                                         "content": svc.engine.tokenizer.decode(req.output_ids)},
                                 "finish_reason": req.finish_reason}],
                    "usage": _usage(req)}

        @app.post("/v1/completions")
        async def completions(body: PiscesLxCompletionRequest):
            req = svc.submit(body.prompt, body.max_tokens, body.temperature, body.top_k, body.top_p)
            await _wait(req)
            return {"id": "cmpl-" + uuid.uuid4().hex[:24], "object": "text_completion", "created": int(time.time()),
                    "model": body.model,
                    "choices": [{"index": 0, "text": svc.engine.tokenizer.decode(req.output_ids),
                                 "finish_reason": req.finish_reason}],
                    "usage": _usage(req)}

        @app.post("/v1/embeddings")
        async def embeddings(body: PiscesLxEmbeddingRequest):
            texts = body.input if isinstance(body.input, list) else [body.input]
            data = [{"object": "embedding", "index": i, "embedding": svc.engine.embeddings(str(t))}
                    for i, t in enumerate(texts)]
            return {"object": "list", "data": data, "model": body.model}

        return app


class PiscesLxBackendServer:
    """``manage.py serve`` entry: builds the model, the engine and runs uvicorn."""

    def __init__(self, args: Any):
        self.args = args

    def run(self) -> None:
        import uvicorn

        from ..engine.loader import load_model_for_inference
        model = load_model_for_inference(getattr(self.args, "model_size", "0.01B"), getattr(self.args, "ckpt", None),
                                         getattr(self.args, "device", None))
        engine = YvInferenceEngine(model, cfg=YvEngineConfig(num_blocks=getattr(self.args, "kv_blocks", 1024)))
        app = PiscesLxInferService(engine, getattr(self.args, "model_size", "yv")).build_app()
        uvicorn.run(app, host=getattr(self.args, "host", "127.0.0.1"), port=int(getattr(self.args, "port", 8000)))
