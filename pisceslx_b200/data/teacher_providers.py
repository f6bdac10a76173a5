"""Teacher providers for distillation (reference tools/data/distill/offline_teacher_provider.py:81-830): one interface -
logits, hidden states, attentions for a batch of token ids - over a local model, an inference server, or a remote API that
only returns the log-probabilities of its top tokens.

Every network call goes through an injectable ``transport`` (``transport(url, payload, headers, timeout) -> dict``); the
default uses ``requests``.  Tests and offline runs pass their own, so nothing here needs a network to be exercised.

Remote APIs return top-k log-probabilities per position, not logits.  ``get_logits`` turns them into a dense tensor whose
unlisted entries share the left-over probability mass evenly (so that a softmax of the result reproduces the listed
probabilities); ``get_sparse_targets`` returns the (ids, log-probabilities) pair as it is, which is what the sparse KL of
``data.augment.PiscesLxOfflineTeacherProvider.sparse_kl`` consumes without materialising [B, T, V]."""
from __future__ import annotations

import contextlib
import math
import time
from abc import ABC, abstractmethod
from dataclasses import dataclass
from enum import Enum
from typing import Any, Callable, Dict, Iterator, List, Optional, Tuple

import torch
from torch import Tensor

Transport = Callable[[str, Dict[str, Any], Dict[str, str], float], Dict[str, Any]]


class PiscesLxTeacherProviderType(str, Enum):
    LOCAL = "local"
    SERVER = "server"
    REMOTE = "remote"


@dataclass
class PiscesLxTeacherConfig:
    provider_type: str = "local"
    model_path: Optional[str] = None
    device: str = "auto"
    torch_dtype: str = "float16"
    offload_strategy: str = "auto"
    server_url: Optional[str] = None
    api_key: Optional[str] = None
    api_type: Optional[str] = None
    model_name: Optional[str] = None
    remote_distill_mode: str = "logprobs"
    base_url: Optional[str] = None
    max_retries: int = 3
    timeout: int = 60
    batch_size: int = 8
    layer_indices: Optional[List[int]] = None
    output_hidden_states: bool = True
    output_attentions: bool = True
    alpha: float = 0.5
    temperature: float = 2.0
    top_logprobs: int = 20
    vocab_size: Optional[int] = None

    def __post_init__(self) -> None:
        self.provider_type = str(getattr(self.provider_type, "value", self.provider_type)).lower()      # the factory knows which names exist
        if not 0.0 <= self.alpha <= 1.0:
            raise ValueError("alpha must lie in [0, 1]")
        if self.temperature <= 0:
            raise ValueError("temperature must be positive")


def _default_transport(url: str, payload: Dict[str, Any], headers: Dict[str, str], timeout: float) -> Dict[str, Any]:
    import requests
    r = requests.post(url, json=payload, headers=headers, timeout=timeout)
    r.raise_for_status()
    return r.json()


class PiscesLxTeacherProvider(ABC):
    def __init__(self, config: PiscesLxTeacherConfig):
        self.config = config
        self.calls = 0

    @abstractmethod
    def get_logits(self, input_ids: Tensor) -> Tensor:
        ...

    def get_hidden_states(self, input_ids: Tensor) -> Optional[List[Tensor]]:
        return None

    def get_attentions(self, input_ids: Tensor) -> Optional[List[Tensor]]:
        return None

    def _select(self, layers: Optional[List[Tensor]]) -> Optional[List[Tensor]]:
        idx = self.config.layer_indices
        if layers is None or idx is None:
            return layers
        return [layers[i] for i in idx if -len(layers) <= i < len(layers)]

    def get_all_outputs(self, input_ids: Tensor) -> Dict[str, Any]:
        out: Dict[str, Any] = {"logits": self.get_logits(input_ids)}
        if self.config.output_hidden_states:
            out["hidden_states"] = self.get_hidden_states(input_ids)
        if self.config.output_attentions:
            out["attentions"] = self.get_attentions(input_ids)
        return out

    def soft_targets(self, input_ids: Tensor) -> Tensor:
        """softmax(logits / temperature): what the student's KL term is taken against."""
        return torch.softmax(self.get_logits(input_ids).float() / self.config.temperature, -1)

    def is_available(self) -> bool:
        return True

    def close(self) -> None:
        pass

    def __enter__(self) -> "PiscesLxTeacherProvider":
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()


class PiscesLxLocalTeacherProvider(PiscesLxTeacherProvider):
    """A model in this process: pass it as ``model=``, or give ``config.model_path`` (a model size or a checkpoint) and it is
    loaded on first use through ``engine.loader``.  One forward serves logits and hidden states when both are asked for
    the same ids in a row."""

    def __init__(self, config: PiscesLxTeacherConfig, model_class: Any = None, tokenizer: Any = None, model: Any = None):
        super().__init__(config)
        self.model_class, self.tokenizer, self._model = model_class, tokenizer, model
        self._memo: Optional[Tuple[int, Dict[str, Any]]] = None

    def _device(self) -> torch.device:
        d = self.config.device
        if d in ("auto", None):
            return torch.device("cuda" if torch.cuda.is_available() else "cpu")
        return torch.device(d)

    def _lazy_init(self) -> Any:
        if self._model is None:
            if not self.config.model_path:
                raise ValueError("a local teacher needs model= or config.model_path")
            if self.model_class is not None:
                m = self.model_class.from_pretrained(self.config.model_path) if hasattr(self.model_class, "from_pretrained") else self.model_class(self.config.model_path)
            else:
                from ..engine.loader import load_model_for_inference
                import os
                size, ckpt = (self.config.model_name or "0.01B", self.config.model_path) if os.path.exists(self.config.model_path) else (self.config.model_path, None)
                m = load_model_for_inference(size, ckpt, str(self._device()))
            self._model = m
        self._model.eval()
        for p in self._model.parameters():
            p.requires_grad_(False)
        return self._model

    @torch.no_grad()
    def _forward(self, input_ids: Tensor) -> Dict[str, Any]:
        key = (id(input_ids), input_ids.data_ptr(), input_ids._version, tuple(input_ids.shape))      # the same tensor object, unmodified: no device read
        if self._memo is not None and self._memo[0] == key:
            return self._memo[1]
        m = self._lazy_init()
        dev = next(m.parameters()).device
        ids = input_ids.to(dev)
        self.calls += 1
        try:
            out = m(input_ids=ids, return_logits=True, return_hidden=True)
        except TypeError:
            try:
                out = m(input_ids=ids, output_hidden_states=True, output_attentions=self.config.output_attentions)
            except TypeError:
                out = m(ids)
        if torch.is_tensor(out):
            out = {"logits": out}
        res = {"logits": out["logits"] if isinstance(out, dict) else out.logits}
        hs = out.get("hidden_states") if isinstance(out, dict) else getattr(out, "hidden_states", None)
        res["hidden_states"] = [hs] if torch.is_tensor(hs) else (list(hs) if hs is not None else None)
        at = out.get("attentions") if isinstance(out, dict) else getattr(out, "attentions", None)
        res["attentions"] = list(at) if at is not None else None
        self._memo = (key, res)
        return res

    def get_logits(self, input_ids: Tensor) -> Tensor:
        return self._forward(input_ids)["logits"]

    def get_hidden_states(self, input_ids: Tensor) -> Optional[List[Tensor]]:
        return self._select(self._forward(input_ids)["hidden_states"])

    def get_attentions(self, input_ids: Tensor) -> Optional[List[Tensor]]:
        return self._select(self._forward(input_ids)["attentions"])

    def is_available(self) -> bool:
        return self._model is not None or bool(self.config.model_path)

    def close(self) -> None:
        self._model, self._memo = None, None
        if torch.cuda.is_available():
            torch.cuda.empty_cache()


class _NetworkProvider(PiscesLxTeacherProvider):
    def __init__(self, config: PiscesLxTeacherConfig, transport: Optional[Transport] = None, sleep: Callable[[float], None] = time.sleep):
        super().__init__(config)
        self.transport, self._sleep = transport or _default_transport, sleep
        self.retries = 0

    def _headers(self) -> Dict[str, str]:
        h = {"Content-Type": "application/json"}
        if self.config.api_key:
            h["Authorization"] = f"Bearer {self.config.api_key}"
        return h

    def _post(self, url: str, payload: Dict[str, Any]) -> Dict[str, Any]:
        last: Optional[BaseException] = None
        for attempt in range(max(self.config.max_retries, 1)):
            try:
                self.calls += 1
                return self.transport(url, payload, self._headers(), float(self.config.timeout))
            except Exception as e:                                                     # the transport decides what a failure is
                last = e
                self.retries += 1
                if attempt + 1 < max(self.config.max_retries, 1):
                    self._sleep(min(0.5 * 2 ** attempt, 8.0))
        raise RuntimeError(f"teacher request to {url} failed after {self.config.max_retries} attempts: {last}")


class PiscesLxServerTeacherProvider(_NetworkProvider):
    """An inference server with ``POST /v1/distill/forward`` ({"input_ids", "output_hidden_states", "output_attentions"} ->
    {"logits", "hidden_states"?, "attentions"?}) and ``GET``-like ``/health`` (asked through the same transport)."""

    def _request(self, input_ids: Tensor, **kwargs: Any) -> Dict[str, Any]:
        if not self.config.server_url:
            raise ValueError("a server teacher needs config.server_url")
        return self._post(f"{self.config.server_url.rstrip('/')}/v1/distill/forward", {"input_ids": input_ids.tolist(), **kwargs})

    def get_logits(self, input_ids: Tensor) -> Tensor:
        return torch.tensor(self._request(input_ids)["logits"], dtype=torch.float32)

    def _layers(self, input_ids: Tensor, key: str, flag: str) -> Optional[List[Tensor]]:
        r = self._request(input_ids, **{flag: True}).get(key)
        return self._select([torch.tensor(x, dtype=torch.float32) for x in r]) if r is not None else None

    def get_hidden_states(self, input_ids: Tensor) -> Optional[List[Tensor]]:
        return self._layers(input_ids, "hidden_states", "output_hidden_states")

    def get_attentions(self, input_ids: Tensor) -> Optional[List[Tensor]]:
        return self._layers(input_ids, "attentions", "output_attentions")

    def is_available(self) -> bool:
        if not self.config.server_url:
            return False
        try:
            self.transport(f"{self.config.server_url.rstrip('/')}/health", {}, self._headers(), min(float(self.config.timeout), 5.0))
            return True
        except Exception:
            return False


class PiscesLxRemoteTeacherProvider(_NetworkProvider):
    """A completion API that scores a given text and returns, per position, the log-probabilities of its top tokens
    (``{"choices": [{"logprobs": {"top_logprobs": [{token_id_or_text: logprob, ...}, ...]}}]}``).  Token keys that are not
    integers are mapped through ``tokenizer.encode`` (first id)."""

    def __init__(self, config: PiscesLxTeacherConfig, tokenizer: Any = None, transport: Optional[Transport] = None, sleep: Callable[[float], None] = time.sleep):
        super().__init__(config, transport, sleep)
        self.tokenizer = tokenizer

    @staticmethod
    def _normalize_base_url(base_url: str) -> str:
        u = base_url.strip().rstrip("/")
        if not u.startswith(("http://", "https://")):
            u = "https://" + u
        return u if u.endswith("/v1") else u + "/v1"

    def _url(self) -> str:
        if not self.config.base_url:
            raise ValueError("a remote teacher needs config.base_url")
        return self._normalize_base_url(self.config.base_url) + "/completions"

    def _token_id(self, key: Any) -> Optional[int]:
        try:
            return int(key)
        except (TypeError, ValueError):
            if self.tokenizer is None:
                return None
            ids = list(self.tokenizer.encode(str(key)))
            return int(ids[0]) if ids else None

    def get_sparse_targets(self, input_ids: Tensor) -> Tuple[Tensor, Tensor]:
        """(ids [B, T, k], log-probabilities [B, T, k]); missing slots hold id -1 and -inf."""
        k = self.config.top_logprobs
        B, T = input_ids.shape
        ids = torch.full((B, T, k), -1, dtype=torch.long)
        lps = torch.full((B, T, k), float("-inf"))
        for b in range(B):
            row = input_ids[b].tolist()
            prompt = self.tokenizer.decode(row) if self.tokenizer is not None else row
            r = self._post(self._url(), {"model": self.config.model_name, "prompt": prompt, "max_tokens": 0, "echo": True, "logprobs": k})
            tops = r["choices"][0]["logprobs"]["top_logprobs"]
            for t, d in enumerate(tops[:T]):
                if not d:
                    continue
                pairs = [(self._token_id(tok), float(lp)) for tok, lp in d.items()]
                pairs = sorted([p for p in pairs if p[0] is not None], key=lambda p: -p[1])[:k]
                for j, (i, lp) in enumerate(pairs):
                    ids[b, t, j], lps[b, t, j] = i, lp
        return ids, lps

    def get_logits(self, input_ids: Tensor) -> Tensor:
        V = self.config.vocab_size or (len(self.tokenizer) if self.tokenizer is not None else None)
        if not V:
            raise ValueError("dense logits from a remote teacher need config.vocab_size or a tokenizer")
        ids, lps = self.get_sparse_targets(input_ids)
        valid = ids >= 0
        mass = torch.where(valid, lps.exp(), torch.zeros_like(lps)).sum(-1, keepdim=True).clamp(max=1.0 - 1e-6)
        rest = torch.log((1.0 - mass) / (V - valid.sum(-1, keepdim=True)).clamp_min(1))
        dense = rest.expand(-1, -1, V).clone()
        dense.scatter_(-1, ids.clamp_min(0), torch.where(valid, lps, dense.gather(-1, ids.clamp_min(0))))
        return dense

    def generate_for_distillation(self, prompts: List[str], max_tokens: int = 256, temperature: float = 0.7) -> List[Dict[str, Any]]:
        """Teacher-written answers for sequence-level distillation: ``[{"prompt", "response"}]`` (a failed prompt is skipped and
        counted in ``self.retries``)."""
        out = []
        for p in prompts:
            try:
                r = self._post(self._url(), {"model": self.config.model_name, "prompt": p, "max_tokens": max_tokens, "temperature": temperature})
                out.append({"prompt": p, "response": r["choices"][0].get("text", "")})
            except RuntimeError:
                continue
        return out

    def is_available(self) -> bool:
        return bool(self.config.base_url and self.config.model_name)


class PiscesLxTeacherProviderFactory:
    _registry: Dict[str, type] = {"local": PiscesLxLocalTeacherProvider, "server": PiscesLxServerTeacherProvider, "remote": PiscesLxRemoteTeacherProvider}

    @classmethod
    def create(cls, config: PiscesLxTeacherConfig, model_class: Any = None, tokenizer: Any = None, **kw: Any) -> PiscesLxTeacherProvider:
        t = config.provider_type.lower()
        if t not in cls._registry:
            raise ValueError(f"Unknown provider type: {t}. Available: {list(cls._registry)}")
        pc = cls._registry[t]
        if t == "local":
            return pc(config, model_class=model_class, tokenizer=tokenizer, **kw)
        if t == "remote":
            return pc(config, tokenizer=tokenizer, **kw)
        return pc(config, **kw)

    @classmethod
    def register(cls, name: str, provider_class: type) -> None:
        if not (isinstance(provider_class, type) and issubclass(provider_class, PiscesLxTeacherProvider)):
            raise TypeError("a provider class must derive from PiscesLxTeacherProvider")
        cls._registry[name.lower()] = provider_class

    @classmethod
    @contextlib.contextmanager
    def create_with_cleanup(cls, config: PiscesLxTeacherConfig, **kw: Any) -> Iterator[PiscesLxTeacherProvider]:
        p = cls.create(config, **kw)
        try:
            yield p
        finally:
            p.close()
