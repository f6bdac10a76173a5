"""Tokenizer wrapper.

``YvTokenizer`` loads a byte-level BPE ``tokenizer.json`` (the reference ships one with 154 820 entries + 36
added special tokens = 154 856 ids, model/tokenizer/tokenizer.py:86-712) through the ``tokenizers`` runtime when
a tokenizer directory is available (``tokenizer/`` beside ``manage.py`` or ``$PISCESLX_TOKENIZER``), and falls
back to a self-contained byte tokenizer otherwise, so that every entry point works offline.  Special-token names
follow the reference's ``YvSpecialTokens`` (model/tokenizer/special_tokens.py).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Union

import torch

REFERENCE_VOCAB_SIZE = 154856


@dataclass
class YvSpecialTokens:
    pad: str = "<|pad|>"
    bos: str = "<|bos|>"
    eos: str = "<|eos|>"
    unk: str = "<|unk|>"
    image: str = "<|image|>"
    audio: str = "<|audio|>"
    video: str = "<|video|>"
    think_start: str = "<think>"
    think_end: str = "</think>"
    tool_start: str = "<tool>"
    tool_end: str = "</tool>"
    agent_start: str = "<ag>"
    agent_end: str = "</ag>"

    def all(self) -> List[str]:
        return list(self.__dict__.values())


class _ByteTokenizer:
    """UTF-8 bytes + special tokens: ids 0..3 = pad/bos/eos/unk, 4..259 = bytes, then the remaining specials."""

    def __init__(self, specials: YvSpecialTokens):
        names = specials.all()
        self.special_to_id: Dict[str, int] = {names[0]: 0, names[1]: 1, names[2]: 2, names[3]: 3}
        for i, n in enumerate(names[4:]):
            self.special_to_id[n] = 260 + i
        self.id_to_special = {v: k for k, v in self.special_to_id.items()}
        self.vocab_size = 260 + len(names) - 4

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        i = 0
        specials = sorted(self.special_to_id, key=len, reverse=True)
        while i < len(text):
            for s in specials:
                if text.startswith(s, i):
                    out.append(self.special_to_id[s])
                    i += len(s)
                    break
            else:
                out.extend(4 + b for b in text[i].encode("utf-8"))
                i += 1
        return out

    def decode(self, ids: Iterable[int], skip_special: bool = True) -> str:
        buf = bytearray()
        parts: List[str] = []
        for t in ids:
            t = int(t)
            if 4 <= t < 260:
                buf.append(t - 4)
            else:
                if buf:
                    parts.append(buf.decode("utf-8", errors="replace"))
                    buf = bytearray()
                if not skip_special and t in self.id_to_special:
                    parts.append(self.id_to_special[t])
        if buf:
            parts.append(buf.decode("utf-8", errors="replace"))
        return "".join(parts)


class YvTokenizer:
    _instance: Optional["YvTokenizer"] = None

    def __init__(self, path: Optional[Union[str, Path]] = None, specials: Optional[YvSpecialTokens] = None):
        self.special_tokens = specials or YvSpecialTokens()
        self.backend = None
        self.path = None
        cand = [path, os.environ.get("PISCESLX_TOKENIZER"), Path(__file__).resolve().parents[2] / "tokenizer"]
        for c in cand:
            if c and (Path(c) / "tokenizer.json").exists():
                self.path = Path(c)
                break
        if self.path is not None:
            try:
                from tokenizers import Tokenizer
                self.backend = Tokenizer.from_file(str(self.path / "tokenizer.json"))
            except Exception:
                self.backend = None
        self._bytes = _ByteTokenizer(self.special_tokens) if self.backend is None else None
        self.pad_token_id, self.bos_token_id, self.eos_token_id, self.unk_token_id = 0, 1, 2, 3
        if self.backend is not None:
            for name, attr in (("pad", "pad_token_id"), ("bos", "bos_token_id"), ("eos", "eos_token_id")):
                tid = self.backend.token_to_id(getattr(self.special_tokens, name))
                if tid is not None:
                    setattr(self, attr, tid)

    @classmethod
    def instance(cls) -> "YvTokenizer":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def __len__(self) -> int:
        return self.vocab_size

    @property
    def vocab_size(self) -> int:
        if self.backend is not None:
            return self.backend.get_vocab_size(with_added_tokens=True)
        return self._bytes.vocab_size

    def encode(self, text: str, add_bos: bool = False, add_eos: bool = False) -> List[int]:
        ids = self.backend.encode(text).ids if self.backend is not None else self._bytes.encode(text)
        if add_bos:
            ids = [self.bos_token_id] + ids
        if add_eos:
            ids = ids + [self.eos_token_id]
        return ids

    def decode(self, ids: Union[Sequence[int], torch.Tensor], skip_special_tokens: bool = True) -> str:
        if torch.is_tensor(ids):
            ids = ids.tolist()
        if self.backend is not None:
            return self.backend.decode(list(ids), skip_special_tokens=skip_special_tokens)
        return self._bytes.decode(ids, skip_special_tokens)

    def __call__(self, texts: Union[str, List[str]], max_length: Optional[int] = None, padding: bool = True,
                 return_tensors: Optional[str] = "pt") -> Dict[str, torch.Tensor]:
        if isinstance(texts, str):
            texts = [texts]
        enc = [self.encode(t)[: max_length] if max_length else self.encode(t) for t in texts]
        L = max(len(e) for e in enc) if padding else None
        ids, mask = [], []
        for e in enc:
            pad = (L - len(e)) if L is not None else 0
            ids.append(e + [self.pad_token_id] * pad)
            mask.append([1] * len(e) + [0] * pad)
        if return_tensors == "pt":
            return {"input_ids": torch.tensor(ids, dtype=torch.long), "attention_mask": torch.tensor(mask, dtype=torch.long)}
        return {"input_ids": ids, "attention_mask": mask}

    def apply_chat_template(self, messages: List[Dict[str, str]]) -> str:
        """``[role]: content`` lines joined by newlines (the reference server builds prompts this way,
        tools/infer/server.py:1077-1084)."""
        return "\n".join(f"[{m.get('role', 'user')}]: {m.get('content', '')}" for m in messages)
