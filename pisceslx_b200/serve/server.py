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
from . import schemas as S
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


class PiscesLxRateLimited(RuntimeError):
    pass


class PiscesLxRateLimiter:
    """Token buckets by key: ``rate`` tokens per second refill a bucket of ``burst`` tokens; ``allow`` takes one or
    says no.  The clock can be injected for tests."""

    def __init__(self, rate: float, burst: int, clock=time.monotonic):
        self.rate, self.burst, self.clock = float(rate), int(burst), clock
        self._state: Dict[str, List[float]] = {}
        self._lock = threading.Lock()

    def allow(self, key: str = "default", cost: float = 1.0) -> bool:
        now = self.clock()
        with self._lock:
            tokens, last = self._state.get(key, [float(self.burst), now])
            tokens = min(float(self.burst), tokens + (now - last) * self.rate)
            ok = tokens >= cost
            self._state[key] = [tokens - cost if ok else tokens, now]
            return ok


class PiscesLxInferService:
    def __init__(self, engine: YvInferenceEngine, model_name: str = "yv", rate_limiter: Optional[PiscesLxRateLimiter] = None):
        self.engine, self.model_name = engine, model_name
        self.rate_limiter = rate_limiter
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

    def attach_generator(self, generator: Any) -> None:
        """Serve ``/v1/images/generations``, ``/v1/videos/generations`` and ``/v1/audio/speech`` from a
        ``models.multimodal.YvGenerator`` (tensors become base64 of raw uint8 RGB / int16 PCM)."""
        import base64

        def image(body: Dict[str, Any]):
            rq = S.PiscesLxImageGenerationRequest(**{k: v for k, v in body.items() if k in S.PiscesLxImageGenerationRequest.model_fields})
            out = []
            for i in range(max(1, rq.n)):
                r = generator.generate_from_text(rq.prompt, "image", seed=None if rq.seed is None else rq.seed + i,
                                                 steps=rq.steps, guidance_scale=rq.guidance_scale)
                if not r.success:
                    raise RuntimeError(r.error)
                img = ((r.data[0].float().clamp(-1, 1) + 1) * 127.5).round().byte().permute(1, 2, 0).contiguous().cpu()
                out.append(S.PiscesLxImageData(b64_json=base64.b64encode(img.numpy().tobytes()).decode(),
                                               width=img.shape[1], height=img.shape[0]).model_dump())
            return out

        def video(body: Dict[str, Any]):
            rq = S.PiscesLxVideoGenerationRequest(**{k: v for k, v in body.items() if k in S.PiscesLxVideoGenerationRequest.model_fields})
            r = generator.generate_from_text(rq.prompt, "video", seed=rq.seed, num_frames=rq.num_frames)
            if not r.success:
                raise RuntimeError(r.error)
            v = ((r.data[0].float().clamp(-1, 1) + 1) * 127.5).round().byte().permute(0, 2, 3, 1).contiguous().cpu()
            return [S.PiscesLxVideoData(b64_json=base64.b64encode(v.numpy().tobytes()).decode(), frames=v.shape[0],
                                        height=v.shape[1], width=v.shape[2], fps=int(r.metadata.get("fps", 24))).model_dump()]

        def audio(body: Dict[str, Any]):
            rq = S.PiscesLxAudioSpeechRequest(**{k: v for k, v in body.items() if k in S.PiscesLxAudioSpeechRequest.model_fields})
            r = generator.generate_from_text(rq.input, "audio", duration=rq.duration)
            if not r.success:
                raise RuntimeError(r.error)
            pcm = (r.data[0].float().clamp(-1, 1) * 32767).round().short().cpu()
            return S.PiscesLxAudioSpeechResponse(sample_rate=int(r.metadata.get("sample_rate", 16000)), samples=pcm.numel(),
                                                 b64_pcm16=base64.b64encode(pcm.numpy().tobytes()).decode()).model_dump()

        if not hasattr(self, "media"):
            self.media = {}
        self.media.update({"image": image, "video": video, "audio": audio})

    def submit(self, prompt: str, max_tokens: int, temperature: float, top_k: int, top_p: float, on_token=None):
        if getattr(self, "rate_limiter", None) is not None and not self.rate_limiter.allow("requests"):
            raise PiscesLxRateLimited("request rate limit reached")
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

        @app.exception_handler(PiscesLxRateLimited)
        async def _limited(_request, exc):
            return JSONResponse(S.PiscesLxErrorResponse(error=str(exc), code=429).model_dump(), status_code=429)

        @app.exception_handler(ValueError)
        async def _bad_request(_request, exc):
            return JSONResponse(S.PiscesLxErrorResponse(error=str(exc), code=400).model_dump(), status_code=400)

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
            return S.PiscesLxModelListResponse(data=[S.PiscesLxModelInfo(id=svc.model_name)]).model_dump()

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
                req = svc.submit(prompt, body.max_tokens, body.temperature, body.top_k, body.top_p)

                async def gen():
                    sent = 0
                    while not req.finished or sent < len(req.output_ids):
                        while sent < len(req.output_ids):
                            piece = svc.engine.tokenizer.decode([req.output_ids[sent]])
                            sent += 1
                            yield S.PiscesLxChatCompletionChunk(id=cid, model=body.model, choices=[
                                S.PiscesLxChatCompletionChunkChoice(
                                    delta=S.PiscesLxChatCompletionChunkDelta(content=piece))]).sse()
                        await asyncio.sleep(0.002)
                    end = {"id": cid, "object": "chat.completion.chunk", "created": int(time.time()), "model": body.model,
                           "choices": [{"index": 0, "delta": {}, "finish_reason": req.finish_reason}]}
                    yield f"data: {json.dumps(end)}\n\n"
                    yield "data: [DONE]\n\n"
                return StreamingResponse(gen(), media_type="text/event-stream")
            req = svc.submit(prompt, body.max_tokens, body.temperature, body.top_k, body.top_p)
            await _wait(req)
            return S.PiscesLxChatCompletionResponse(
                id=cid, model=body.model, usage=S.PiscesLxChatCompletionUsage(**_usage(req)),
                choices=[S.PiscesLxChatCompletionChoice(
                    message=S.PiscesLxResponseMessage(content=svc.engine.tokenizer.decode(req.output_ids)),
                    finish_reason=req.finish_reason)]).model_dump()

        @app.post("/v1/completions")
        async def completions(body: PiscesLxCompletionRequest):
            req = svc.submit(body.prompt, body.max_tokens, body.temperature, body.top_k, body.top_p)
            await _wait(req)
            return S.PiscesLxCompletionResponse(
                model=body.model, usage=S.PiscesLxChatCompletionUsage(**_usage(req)),
                choices=[S.PiscesLxCompletionChoice(text=svc.engine.tokenizer.decode(req.output_ids),
                                                    finish_reason=req.finish_reason)]).model_dump()

        @app.post("/v1/embeddings")
        async def embeddings(body: PiscesLxEmbeddingRequest):
            texts = body.input if isinstance(body.input, list) else [body.input]
            data = [S.PiscesLxEmbeddingData(index=i, embedding=svc.engine.embeddings(str(t))) for i, t in enumerate(texts)]
            return S.PiscesLxEmbeddingResponse(data=data, model=body.model).model_dump()

        svc._add_extended_routes(app)
        return app

    # ---- tools, agents, runs, media (reference tools/infer/server.py:312-405) -----------------------------
    def _generate_text(self, prompt: str, max_new_tokens: int = 256) -> str:
        req = self.submit(prompt, max_new_tokens, 0.0, 0, 1.0)
        while not req.finished:
            time.sleep(0.002)
        return self.engine.tokenizer.decode(req.output_ids)

    def _add_extended_routes(self, app) -> None:
        from fastapi.responses import JSONResponse

        from ..engine.runstore import PiscesLxRunStore
        from ..models.reasoning import YvAgentic, YvToolRegistry
        svc = self
        if not hasattr(self, "tools"):
            self.tools = YvToolRegistry()
        if not hasattr(self, "runs"):
            self.runs = PiscesLxRunStore()
        if not hasattr(self, "media"):
            self.media: Dict[str, Any] = {}       # "image" / "video" / "audio": callables attached by the deployment

        @app.get("/v1/tools/list")
        async def tools_list():
            return {"object": "list", "data": [{"name": t.name, "description": t.description, "parameters": t.parameters}
                                               for t in svc.tools.tools.values()]}

        @app.post("/v1/tools/search")
        async def tools_search(body: Dict[str, Any]):
            q = str(body.get("query", "")).lower()
            hits = [t for t in svc.tools.tools.values() if q in t.name.lower() or q in t.description.lower()]
            return {"object": "list", "data": [{"name": t.name, "description": t.description} for t in hits]}

        @app.post("/v1/tools/execute")
        async def tools_execute(body: Dict[str, Any]):
            name, args = body.get("name", ""), body.get("arguments", {}) or {}
            try:
                return {"name": name, "result": svc.tools.call(name, args), "error": None}
            except KeyError as e:
                return JSONResponse({"name": name, "result": None, "error": str(e)}, status_code=404)
            except Exception as e:
                return JSONResponse({"name": name, "result": None, "error": f"{type(e).__name__}: {e}"}, status_code=400)

        @app.get("/v1/agents/list")
        async def agents_list():
            return {"object": "list", "data": [{"id": "react", "description": "ReAct loop over the registered tools"}]}

        @app.post("/v1/agents/execute")
        async def agents_execute(body: Dict[str, Any]):
            agent = YvAgentic(lambda p, n: svc._generate_text(p, n), svc.tools, max_turns=int(body.get("max_turns", 4)),
                              max_new_tokens=int(body.get("max_tokens", 128)))
            out = await asyncio.get_event_loop().run_in_executor(None, agent.run, str(body.get("task", "")))
            return {"agent": "react", "result": out}

        @app.post("/v1/agents/swarm")
        async def agents_swarm(body: Dict[str, Any]):
            tasks = [str(t) for t in body.get("tasks", [])]
            loop = asyncio.get_event_loop()

            def one(task: str):
                return YvAgentic(lambda p, n: svc._generate_text(p, n), svc.tools, max_turns=int(body.get("max_turns", 3)),
                                 max_new_tokens=int(body.get("max_tokens", 96))).run(task)
            results = await asyncio.gather(*[loop.run_in_executor(None, one, t) for t in tasks])
            return {"results": [{"task": t, "result": r} for t, r in zip(tasks, results)]}

        @app.get("/v1/runs")
        async def runs_list():
            return {"object": "list", "data": svc.runs.list_runs()}

        @app.get("/v1/runs/{run_id}")
        async def runs_get(run_id: str):
            try:
                return {"run_id": run_id, "state": svc.runs.read_state(run_id),
                        "events": svc.runs.read_jsonl(run_id, "events.jsonl")[-20:]}
            except Exception as e:
                return JSONResponse({"error": f"{type(e).__name__}: {e}"}, status_code=404)

        @app.post("/v1/runs/{run_id}/control")
        async def runs_control(run_id: str, body: Dict[str, Any]):
            cmd = str(body.get("command", ""))
            if cmd not in ("pause", "resume", "stop", "checkpoint"):
                return JSONResponse({"error": f"unknown command {cmd!r}"}, status_code=400)
            if run_id not in svc.runs.list_runs():
                return JSONResponse({"error": f"unknown run {run_id!r}"}, status_code=404)
            svc.runs.send_control(run_id, cmd)
            return {"run_id": run_id, "command": cmd, "accepted": True}

        def _media(kind: str):
            async def handler(body: Dict[str, Any]):
                fn = svc.media.get(kind)
                if fn is None:
                    return JSONResponse({"error": f"no {kind} generator is attached to this deployment "
                                                  f"(attach one with service.media[{kind!r}] = callable)"}, status_code=501)
                out = await asyncio.get_event_loop().run_in_executor(None, fn, body)
                return {"created": int(time.time()), "data": out}
            return handler

        app.post("/v1/images/generations")(_media("image"))
        app.post("/v1/images/edits")(_media("image"))
        app.post("/v1/videos/generations")(_media("video"))
        app.post("/v1/audio/speech")(_media("audio"))


class PiscesLxAgentInterceptor:
    """Sits between a chat request and the engine (reference tools/infer/agent_interceptor.py:112).  Modes: ``off``
    passes the completion through; ``auto`` looks for ``<tool_call>`` blocks in the completion, runs the named tools,
    appends their results as a tool message and asks the model to continue, up to ``max_rounds``; ``forced`` does the
    same but first prepends the tool catalogue to the prompt."""

    def __init__(self, generate, tools, mode: str = "auto", max_rounds: int = 3):
        if mode not in ("off", "auto", "forced"):
            raise ValueError(mode)
        self.generate, self.tools, self.mode, self.max_rounds = generate, tools, mode, max_rounds

    def run(self, prompt: str, max_new_tokens: int = 256) -> Dict[str, Any]:
        from ..models.reasoning import parse_tool_calls
        if self.mode == "forced":
            prompt = f"You may call these tools with <tool_call> blocks:\n{self.tools.describe()}\n\n{prompt}"
        text = self.generate(prompt, max_new_tokens)
        trace: List[Dict[str, Any]] = []
        if self.mode == "off":
            return {"content": text, "tool_calls": trace, "rounds": 0}
        rounds = 0
        while rounds < self.max_rounds:
            calls = parse_tool_calls(text)
            if not calls:
                break
            rounds += 1
            results = []
            for name, args in calls:
                try:
                    res = self.tools.call(name, args)
                    err = None
                except Exception as e:
                    res, err = None, f"{type(e).__name__}: {e}"
                trace.append({"name": name, "arguments": args, "result": res, "error": err})
                results.append(f"<tool_result name=\"{name}\">{res if err is None else err}</tool_result>")
            prompt = f"{prompt}\n{text}\n" + "\n".join(results) + "\n"
            text = self.generate(prompt, max_new_tokens)
        return {"content": text, "tool_calls": trace, "rounds": rounds}


class PiscesLxModelRouter:
    """Resolves a request's model id to a model size and a fallback chain (reference tools/infer/model_router.py:91):
    ``piscesl1-7b``, ``7B``, ``yv-0.5b`` -> size; unknown or unavailable sizes fall back to the next smaller one."""

    ORDER = ["0.01B", "0.1B", "0.5B", "1.5B", "7B", "32B", "64B", "70B", "128B", "314B", "671B", "1T"]

    def __init__(self, available: Optional[List[str]] = None, default_size: str = "7B"):
        self.available = list(available) if available else [default_size]
        self.default = default_size
        self.load: Dict[str, int] = {s: 0 for s in self.available}

    @classmethod
    def parse_size(cls, model_id: str) -> Optional[str]:
        import re
        m = re.match(r"^(?:[a-z0-9]+[-_])?([0-9.]+)\s*([bmt])$", model_id.strip().lower())
        if not m:
            return None
        num, unit = m.group(1), m.group(2).upper()
        cand = f"{num}{unit}"
        for s in cls.ORDER:
            if s.lower() == cand.lower():
                return s
        return None

    def resolve(self, model_id: str) -> Dict[str, Any]:
        size = self.parse_size(model_id)
        strategy = "explicit"
        if size is None:
            size, strategy = self.default, "auto"
        chain = [s for s in reversed(self.ORDER[: self.ORDER.index(size)]) if s in self.available] \
            if size in self.ORDER else []
        if size not in self.available:
            strategy = "fallback"
            size = chain[0] if chain else (self.default if self.default in self.available else self.available[0])
            chain = chain[1:]
        self.load[size] = self.load.get(size, 0) + 1
        return {"model_id": model_id, "model_size": size, "strategy": strategy, "fallback_chain": chain}


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
