"""Typed bodies of the inference service's routes (reference tools/infer/server.py:120-310 declares the same set as
pydantic models).  The routes build their answers through these classes, so a malformed answer fails in the server
instead of at the client; clients may use them to parse what they receive."""
from __future__ import annotations

import time
import uuid
from typing import Any, Dict, List, Optional

from pydantic import BaseModel, Field


def _now() -> int:
    return int(time.time())


# ---- chat / completion ----------------------------------------------------------------------------------------------
class PiscesLxChatCompletionUsage(BaseModel):
    prompt_tokens: int = 0
    completion_tokens: int = 0
    total_tokens: int = 0


class PiscesLxFunctionCall(BaseModel):
    name: str
    arguments: str = "{}"


class PiscesLxResponseMessage(BaseModel):
    role: str = "assistant"
    content: Optional[str] = ""
    function_call: Optional[PiscesLxFunctionCall] = None


class PiscesLxChatCompletionChoice(BaseModel):
    index: int = 0
    message: PiscesLxResponseMessage
    finish_reason: Optional[str] = None


class PiscesLxChatCompletionResponse(BaseModel):
    id: str = Field(default_factory=lambda: "chatcmpl-" + uuid.uuid4().hex[:24])
    object: str = "chat.completion"
    created: int = Field(default_factory=_now)
    model: str = "yv"
    choices: List[PiscesLxChatCompletionChoice]
    usage: PiscesLxChatCompletionUsage = Field(default_factory=PiscesLxChatCompletionUsage)


class PiscesLxChatCompletionChunkDelta(BaseModel):
    role: Optional[str] = None
    content: Optional[str] = None


class PiscesLxChatCompletionChunkChoice(BaseModel):
    index: int = 0
    delta: PiscesLxChatCompletionChunkDelta = Field(default_factory=PiscesLxChatCompletionChunkDelta)
    finish_reason: Optional[str] = None


class PiscesLxChatCompletionChunk(BaseModel):
    id: str
    object: str = "chat.completion.chunk"
    created: int = Field(default_factory=_now)
    model: str = "yv"
    choices: List[PiscesLxChatCompletionChunkChoice]

    def sse(self) -> str:
        return f"data: {self.model_dump_json(exclude_none=True)}\n\n"


class PiscesLxCompletionChoice(BaseModel):
    index: int = 0
    text: str = ""
    finish_reason: Optional[str] = None


class PiscesLxCompletionResponse(BaseModel):
    id: str = Field(default_factory=lambda: "cmpl-" + uuid.uuid4().hex[:24])
    object: str = "text_completion"
    created: int = Field(default_factory=_now)
    model: str = "yv"
    choices: List[PiscesLxCompletionChoice]
    usage: PiscesLxChatCompletionUsage = Field(default_factory=PiscesLxChatCompletionUsage)


# ---- embeddings / models / health ---------------------------------------------------------------------------------------
class PiscesLxEmbeddingData(BaseModel):
    object: str = "embedding"
    index: int = 0
    embedding: List[float]


class PiscesLxEmbeddingResponse(BaseModel):
    object: str = "list"
    data: List[PiscesLxEmbeddingData]
    model: str = "yv"


class PiscesLxModelInfo(BaseModel):
    id: str
    object: str = "model"
    owned_by: str = "pisceslx_b200"


class PiscesLxModelListResponse(BaseModel):
    object: str = "list"
    data: List[PiscesLxModelInfo]


class PiscesLxHealthResponse(BaseModel):
    status: str = "ok"
    uptime_s: float = 0.0


class PiscesLxReadyResponse(BaseModel):
    ready: bool = True
    running: int = 0
    waiting: int = 0


class PiscesLxErrorResponse(BaseModel):
    error: str
    code: int = 400


# ---- tools / agents / runs -------------------------------------------------------------------------------------------
class PiscesLxToolExecuteRequest(BaseModel):
    name: str
    arguments: Dict[str, Any] = Field(default_factory=dict)


class PiscesLxToolExecuteResponse(BaseModel):
    name: str
    result: Any = None


class PiscesLxToolSearchRequest(BaseModel):
    query: str = ""
    limit: int = 10


class PiscesLxToolListResponse(BaseModel):
    data: List[Dict[str, Any]]


class PiscesLxAgentInfo(BaseModel):
    name: str
    description: str = ""


class PiscesLxAgentExecuteRequest(BaseModel):
    task: str
    agent: str = "default"
    max_steps: int = 4


class PiscesLxAgentExecuteResponse(BaseModel):
    agent: str
    answer: str
    steps: List[Dict[str, Any]] = Field(default_factory=list)


class PiscesLxSwarmExecuteRequest(BaseModel):
    task: str
    agents: List[str] = Field(default_factory=lambda: ["default"])


class PiscesLxSwarmExecuteResponse(BaseModel):
    answers: Dict[str, str]
    consensus: str = ""


class PiscesLxRunInfo(BaseModel):
    run_id: str
    spec: Dict[str, Any] = Field(default_factory=dict)
    state: Dict[str, Any] = Field(default_factory=dict)


class PiscesLxRunListResponse(BaseModel):
    data: List[str]


class PiscesLxRunControlRequest(BaseModel):
    command: str


class PiscesLxRunControlResponse(BaseModel):
    run_id: str
    command: str
    accepted: bool = True


# ---- media ---------------------------------------------------------------------------------------------------------------
class PiscesLxImageGenerationRequest(BaseModel):
    prompt: str = ""
    n: int = 1
    size: Optional[str] = None
    steps: Optional[int] = None
    seed: Optional[int] = None
    guidance_scale: Optional[float] = None


class PiscesLxImageEditRequest(PiscesLxImageGenerationRequest):
    image: Optional[str] = None                 # base64 of raw uint8 RGB, row-major


class PiscesLxImageData(BaseModel):
    b64_json: str                               # base64 of raw uint8 RGB, row-major
    width: int
    height: int


class PiscesLxImageGenerationResponse(BaseModel):
    created: int = Field(default_factory=_now)
    data: List[PiscesLxImageData]


class PiscesLxVideoGenerationRequest(BaseModel):
    prompt: str = ""
    num_frames: Optional[int] = None
    seed: Optional[int] = None


class PiscesLxVideoData(BaseModel):
    b64_json: str                               # base64 of raw uint8 RGB frames, [T, H, W, 3]
    frames: int
    width: int
    height: int
    fps: int


class PiscesLxVideoGenerationResponse(BaseModel):
    created: int = Field(default_factory=_now)
    data: List[PiscesLxVideoData]


class PiscesLxAudioSpeechRequest(BaseModel):
    input: str = ""
    duration: Optional[float] = None


class PiscesLxAudioSpeechResponse(BaseModel):
    created: int = Field(default_factory=_now)
    sample_rate: int
    samples: int
    b64_pcm16: str                              # base64 of little-endian int16 PCM


class PiscesLxResponseFormat(BaseModel):
    type: str = "text"                              # "text" | "json_object"


class PiscesLxTool(BaseModel):
    type: str = "function"
    function: Dict[str, Any]


class PiscesLxServiceStats(BaseModel):
    uptime_seconds: float = 0
    request_count: int = 0
    success_count: int = 0
    error_count: int = 0
    qps: float = 0
    latency_p50_ms: Optional[float] = None
    latency_p95_ms: Optional[float] = None
    model_size: Optional[str] = None
    engine_status: Optional[Dict[str, Any]] = None
    resource: Optional[Dict[str, Any]] = None
