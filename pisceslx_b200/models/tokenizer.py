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

    def __init__(self, path: Optional[Union[str, Path]] = None, specials: Optional[YvSpecialTokens] = None,
                 use_files: bool = True):
        """``use_files=False`` skips the tokenizer directories and gives the built-in byte tokenizer (273 ids): what a
        model with a vocabulary smaller than the shipped file's needs."""
        self.special_tokens = specials or YvSpecialTokens()
        self.backend = None
        self.path = None
        cand = [path, os.environ.get("PISCESLX_TOKENIZER"), Path(__file__).resolve().parents[2] / "tokenizer"] \
            if use_files else []
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

    @classmethod
    def for_vocab(cls, vocab_size: int) -> "YvTokenizer":
        """The shared tokenizer when its ids fit a model with ``vocab_size`` embeddings, else the byte tokenizer."""
        tok = cls.instance()
        return tok if tok.vocab_size <= vocab_size else cls(use_files=False)

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

    # ---- the rest of the reference surface (model/tokenizer/tokenizer.py:355-712) --------------------------------
    def encode_batch(self, texts: List[str], add_bos: bool = False, add_eos: bool = False) -> List[List[int]]:
        return [self.encode(t, add_bos, add_eos) for t in texts]

    def batch_decode(self, batch: Sequence[Sequence[int]], skip_special_tokens: bool = True) -> List[str]:
        return [self.decode(ids, skip_special_tokens) for ids in batch]

    def add_tokens(self, new_tokens: List[str]) -> int:
        """Append tokens that are not in the vocabulary yet; returns how many were added."""
        if self.backend is not None:
            return int(self.backend.add_tokens([t for t in new_tokens if self.backend.token_to_id(t) is None]))
        added = 0
        for t in new_tokens:
            if t not in self._bytes.special_to_id:
                tid = self._bytes.vocab_size
                self._bytes.special_to_id[t] = tid
                self._bytes.id_to_special[tid] = t
                self._bytes.vocab_size += 1
                added += 1
        return added

    def get_special_token_id(self, token: str) -> Optional[int]:
        if self.backend is not None:
            return self.backend.token_to_id(token)
        return self._bytes.special_to_id.get(token)

    def get_vocab(self) -> Dict[str, int]:
        if self.backend is not None:
            return dict(self.backend.get_vocab(with_added_tokens=True))
        v = {f"<0x{b:02X}>": 4 + b for b in range(256)}
        v.update(self._bytes.special_to_id)
        return v

    def convert_ids_to_tokens(self, ids: Sequence[int]) -> List[str]:
        if self.backend is not None:
            return [self.backend.id_to_token(int(i)) or self.special_tokens.unk for i in ids]
        inv = {i: t for t, i in self.get_vocab().items()}
        return [inv.get(int(i), self.special_tokens.unk) for i in ids]

    def convert_tokens_to_string(self, tokens: List[str]) -> str:
        ids = [self.get_special_token_id(t) if self.backend is not None else self.get_vocab().get(t) for t in tokens]
        return self.decode([i for i in ids if i is not None], skip_special_tokens=False)

    def save_pretrained(self, save_directory: Union[str, Path]) -> None:
        d = Path(save_directory)
        d.mkdir(parents=True, exist_ok=True)
        if self.backend is not None:
            self.backend.save(str(d / "tokenizer.json"))
        cfg = {"backend": "tokenizers" if self.backend is not None else "bytes", "model_max_length": 131072,
               "pad_token": self.special_tokens.pad, "bos_token": self.special_tokens.bos,
               "eos_token": self.special_tokens.eos, "unk_token": self.special_tokens.unk,
               "extra_special_tokens": self.special_tokens.all(), "vocab_size": self.vocab_size}
        (d / "tokenizer_config.json").write_text(json.dumps(cfg, indent=2))

    def _named_id(self, *names: str) -> int:
        for n in names:
            tid = self.get_special_token_id(n)
            if tid is not None:
                return tid
        return self.unk_token_id

    im_start_id = property(lambda self: self._named_id("<|im_start|>", self.special_tokens.bos))
    im_end_id = property(lambda self: self._named_id("<|im_end|>", self.special_tokens.eos))
    vision_start_id = property(lambda self: self._named_id("<|vision_start|>", self.special_tokens.image))
    vision_end_id = property(lambda self: self._named_id("<|vision_end|>", self.special_tokens.image))
    image_pad_id = property(lambda self: self._named_id("<|image_pad|>", self.special_tokens.image))
    video_pad_id = property(lambda self: self._named_id("<|video_pad|>", self.special_tokens.video))

    @classmethod
    def reset_instance(cls) -> None:
        cls._instance = None


# ----------------------------------------------------------------------------------------------------------------------
# building a tokenizer file
# ----------------------------------------------------------------------------------------------------------------------
CHAT_SPECIALS = ["<|endoftext|>", "<|system|>", "<|user|>", "<|assistant|>", "<|observation|>", "<|im_start|>",
                 "<|im_end|>", "<|vision_start|>", "<|vision_end|>", "<|vision_pad|>", "<|image_pad|>", "<|video_pad|>",
                 "<|begin_of_image|>", "<|end_of_image|>", "<|begin_of_audio|>", "<|end_of_audio|>", "[MASK]"]


def train_tokenizer(files: Sequence[Union[str, Path]], out_dir: Union[str, Path], vocab_size: int = 8192,
                    specials: Optional[YvSpecialTokens] = None, min_frequency: int = 2) -> Path:
    """Train a byte-level BPE tokenizer (every byte is in the alphabet, so any text round-trips) on ``files`` and
    write ``tokenizer.json`` + ``tokenizer_config.json`` to ``out_dir``.  The special tokens come first, so pad / bos /
    eos / unk are ids 0..3 like in the built-in byte tokenizer.  ``python -m pisceslx_b200.models.tokenizer --help``
    is the command-line form; the file shipped in ``tokenizer/`` was made by it from this repository's own sources."""
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    sp = specials or YvSpecialTokens()
    names = sp.all() + [t for t in CHAT_SPECIALS if t not in sp.all()]
    tok = Tokenizer(models.BPE(unk_token=None))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=vocab_size, min_frequency=min_frequency, special_tokens=names,
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tok.train([str(f) for f in files], trainer)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    tok.save(str(out / "tokenizer.json"))
    cfg = {"backend": "tokenizers", "model_max_length": 131072, "pad_token": sp.pad, "bos_token": sp.bos,
           "eos_token": sp.eos, "unk_token": sp.unk, "extra_special_tokens": names,
           "vocab_size": tok.get_vocab_size(with_added_tokens=True), "trained_on": len(files)}
    (out / "tokenizer_config.json").write_text(json.dumps(cfg, indent=2))
    return out


# ----------------------------------------------------------------------------------------------------------------------
# extended vocabulary
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class YvExtendedTokenizerConfig:
    target_vocab_size: int = 160000
    num_scientific_tokens: int = 28000
    num_code_tokens: int = 24000
    num_multilingual_tokens: int = 20000
    num_domain_tokens: int = 18000


class YvTokenizer160K(YvTokenizer):
    """Tokenizer whose vocabulary is widened to ``target_vocab_size`` with generated scientific, code, multilingual and
    domain tokens (reference model/tokenizer/tokenizer.py:746-1065 grows a ~70K base to 160K the same way).  The added
    tokens are whole-string entries: the BPE backend matches them before splitting, the byte fallback treats them like
    special tokens.  Each category occupies one contiguous id range (``get_domain_token_ids``); existing special ids
    keep their values."""

    def __init__(self, config: Optional[YvExtendedTokenizerConfig] = None,
                 path: Optional[Union[str, Path]] = None, **kw):
        super().__init__(path, **kw)
        self.config = config or YvExtendedTokenizerConfig()
        self.base_vocab_size = self.vocab_size
        self._domain_token_ranges: Dict[str, range] = {}
        self._extend()

    # generators: deterministic families of strings, cut to the configured count
    @staticmethod
    def _scientific() -> Iterable[str]:
        greek = "αβγδεζηθικλμνξοπρστυφχψωΑΒΓΔΕΖΗΘΙΚΛΜΝΞΟΠΡΣΤΥΦΧΨΩ"
        ops = ["∑", "∏", "∫", "∂", "∇", "√", "∞", "≈", "≠", "≤", "≥", "±", "×", "÷", "∈", "∉", "⊂", "⊆", "∪", "∩", "→", "⇒", "⇔", "∀", "∃"]
        units = ["m", "kg", "s", "A", "K", "mol", "cd", "Hz", "N", "Pa", "J", "W", "C", "V", "F", "Ω", "T", "eV"]
        yield from ops
        for g in greek:
            yield g
            for i in range(10):
                yield f"{g}_{i}"
                yield f"{g}^{i}"
        for pre in ("", "k", "M", "G", "T", "m", "μ", "n", "p"):
            for u in units:
                yield f" {pre}{u}"
                for e in (2, 3, -1, -2):
                    yield f" {pre}{u}^{e}"
        for f in ("sin", "cos", "tan", "log", "ln", "exp", "det", "dim", "ker", "lim", "max", "min", "sup", "inf", "arg"):
            for v in "xyzntabkθφ":
                yield f"\\{f}({v})"
                yield f"{f}({v})"
        i = 0
        while True:
            yield f"\\sym{{{i}}}"
            i += 1

    @staticmethod
    def _code() -> Iterable[str]:
        kws = ["def", "class", "return", "import", "from", "async", "await", "lambda", "yield", "fn", "let", "mut", "impl",
               "struct", "enum", "match", "pub", "func", "var", "const", "static", "void", "int", "float", "double", "template",
               "typename", "namespace", "public", "private", "protected", "interface", "package", "try", "catch", "finally"]
        ops = ["==", "!=", "<=", ">=", "->", "=>", "::", "&&", "||", "<<", ">>", "+=", "-=", "*=", "/=", "//", "/*", "*/", "**", "?.", "??", "...", "#!", "{}", "[]", "()"]
        yield from ops
        for k in kws:
            yield f"{k} "
            yield f" {k} "
            yield f"\n{k} "
            for ind in (4, 8, 12):
                yield " " * ind + k + " "
        i = 0
        while True:
            yield f"__code_{i}__"
            i += 1

    @staticmethod
    def _multilingual() -> Iterable[str]:
        blocks = [(0x0400, 0x04FF), (0x0600, 0x06FF), (0x0900, 0x097F), (0x0E00, 0x0E7F), (0x3040, 0x30FF), (0xAC00, 0xD7A3), (0x4E00, 0x9FFF)]
        for lo, hi in blocks:
            for cp in range(lo, hi + 1):
                ch = chr(cp)
                if ch.isprintable():
                    yield ch
        i = 0
        while True:
            yield f"<lang_{i}>"
            i += 1

    @staticmethod
    def _domain() -> Iterable[str]:
        stems = ["cardio", "neuro", "hepato", "nephro", "derma", "onco", "immuno", "patho", "pharmaco", "toxico", "litig", "arbitr",
                 "statut", "juris", "tort", "equit", "liquid", "amortiz", "deriv", "collater", "securit", "hedg"]
        suff = ["logy", "pathy", "itis", "osis", "ectomy", "gram", "ation", "ative", "ize", "ized", "izing", "or", "al", "ic"]
        for s in stems:
            for u in suff:
                yield f" {s}{u}"
        i = 0
        while True:
            yield f"<domain_{i}>"
            i += 1

    def _extend(self) -> None:
        cfg = self.config
        plan = [("scientific", self._scientific(), cfg.num_scientific_tokens), ("code", self._code(), cfg.num_code_tokens),
                ("multilingual", self._multilingual(), cfg.num_multilingual_tokens), ("domain", self._domain(), cfg.num_domain_tokens)]
        for name, gen, count in plan:
            room = max(0, min(count, cfg.target_vocab_size - self.vocab_size))
            start = self.vocab_size
            batch: List[str] = []
            known = self.get_vocab()
            for tok in gen:
                if len(batch) >= room:
                    break
                if tok not in known:
                    known[tok] = -1
                    batch.append(tok)
            self.add_tokens(batch)
            self._domain_token_ranges[name] = range(start, self.vocab_size)
        # whatever is still missing up to the target is filled with reserved entries, as the reference's merge pass does
        rest = cfg.target_vocab_size - self.vocab_size
        if rest > 0:
            start = self.vocab_size
            self.add_tokens([f"<reserved_{i}>" for i in range(rest)])
            self._domain_token_ranges["reserved"] = range(start, self.vocab_size)

    def get_domain_token_ids(self, domain: str) -> List[int]:
        return list(self._domain_token_ranges.get(domain, range(0)))

    def get_extended_vocab_size(self) -> int:
        return self.vocab_size

    def get_extended_vocab(self) -> Dict[str, int]:
        lo = self.base_vocab_size
        return {t: i for t, i in self.get_vocab().items() if i >= lo}

    @property
    def is_extended(self) -> bool:
        return self.vocab_size > self.base_vocab_size


def _main() -> None:
    import argparse
    ap = argparse.ArgumentParser(description="train a byte-level BPE tokenizer file for YvTokenizer")
    ap.add_argument("--files", nargs="+", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--vocab-size", type=int, default=8192)
    a = ap.parse_args()
    print(train_tokenizer(a.files, a.out, a.vocab_size))


if __name__ == "__main__":
    _main()
