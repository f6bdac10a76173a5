"""Text quality signals for data cleaning (reference tools/data/clean/quality.py:73-470,
tools/data/clean/pipeline.py:48-200): script / language detection, keyword domain classification, perplexity,
readability, an incremental-processing ledger and the quality-aware cleaner that uses them.

Everything works offline.  The perplexity calculator scores with a caller-supplied ``token_logprobs(text) ->
sequence of log-probabilities`` (the framework's own model through the serving engine, for instance); without one
it falls back to the unigram / bigram entropy estimate, as the reference does when its hub download fails
(quality.py:292-306)."""
from __future__ import annotations

import hashlib
import json
import math
import os
import re
import threading
from collections import Counter
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

from .cleaning import PiscesLxDataExactDeduplicator, PiscesLxDataMinHashDeduplicator


class PiscesLxLanguageType(str, Enum):
    ENGLISH = "english"
    CHINESE = "chinese"
    JAPANESE = "japanese"
    KOREAN = "korean"
    ARABIC = "arabic"
    RUSSIAN = "russian"
    FRENCH = "french"
    GERMAN = "german"
    SPANISH = "spanish"
    CODE = "code"
    MIXED = "mixed"
    UNKNOWN = "unknown"


class PiscesLxDataLanguageDetector:
    """Script ranges first (a script with more than a tenth of the letters counts; two such scripts are MIXED, except
    that kana decides JAPANESE even beside Han characters, which Japanese text always contains), then code keywords,
    then stop-word overlap among Latin-script languages."""

    _CHAR_RANGES = {
        PiscesLxLanguageType.CHINESE: ((0x4E00, 0x9FFF), (0x3400, 0x4DBF), (0x20000, 0x2A6DF)),
        PiscesLxLanguageType.JAPANESE: ((0x3040, 0x309F), (0x30A0, 0x30FF)),
        PiscesLxLanguageType.KOREAN: ((0xAC00, 0xD7AF), (0x1100, 0x11FF)),
        PiscesLxLanguageType.ARABIC: ((0x0600, 0x06FF), (0x0750, 0x077F)),
        PiscesLxLanguageType.RUSSIAN: ((0x0400, 0x04FF),),
    }
    _CODE_KEYWORDS = ("def ", "class ", "import ", "from ", "return ", "function ", "const ", "let ", "var ", "public ",
                      "private ", "void ", "int ", "string ", "bool ", "if (", "for (", "while (", "#include", "namespace ",
                      "package ", "func ", "fn ", "async ", "await ", "yield ", "lambda ", "->", "=>", "print(", "console.log",
                      "System.out", "printf")
    _STOP = {PiscesLxLanguageType.FRENCH: {"le", "la", "les", "de", "du", "des", "et", "est", "en", "que", "qui", "dans", "pour"},
             PiscesLxLanguageType.GERMAN: {"der", "die", "das", "und", "ist", "von", "zu", "den", "mit", "sich", "auf", "nicht"},
             PiscesLxLanguageType.SPANISH: {"el", "la", "los", "las", "de", "en", "que", "y", "es", "por", "con", "para", "como"}}

    @classmethod
    def _detect_code(cls, text: str) -> float:
        low = text.lower()
        return sum(1 for kw in cls._CODE_KEYWORDS if kw.lower() in low) / len(cls._CODE_KEYWORDS)

    @classmethod
    def _detect_latin_language(cls, text: str) -> PiscesLxLanguageType:
        words = set(re.findall(r"[^\W\d_]+", text.lower()))
        overlap = {lang: len(words & sw) / len(sw) for lang, sw in cls._STOP.items()}
        best = max(overlap, key=overlap.get)
        return best if overlap[best] >= 0.15 else PiscesLxLanguageType.ENGLISH

    @classmethod
    def detect(cls, text: Any) -> PiscesLxLanguageType:
        if not isinstance(text, str) or not text.strip():
            return PiscesLxLanguageType.UNKNOWN
        text = text.strip()
        symbols = sum(text.count(c) for c in "{}();=<>[]")
        if cls._detect_code(text) > 0.12 or (cls._detect_code(text) > 0.05 and symbols / len(text) > 0.03):
            return PiscesLxLanguageType.CODE
        counts: Counter = Counter()
        alpha = 0
        for ch in text:
            if ch.isalpha():
                alpha += 1
                cp = ord(ch)
                for lang, ranges in cls._CHAR_RANGES.items():
                    if any(a <= cp <= b for a, b in ranges):
                        counts[lang] += 1
                        break
        if alpha == 0:
            return PiscesLxLanguageType.UNKNOWN
        found = [lang for lang, c in counts.items() if c / alpha > 0.1]
        if PiscesLxLanguageType.JAPANESE in found and set(found) <= {PiscesLxLanguageType.JAPANESE, PiscesLxLanguageType.CHINESE}:
            return PiscesLxLanguageType.JAPANESE
        latin = sum(1 for c in text if c.isalpha() and ord(c) < 0x250) / alpha
        if len(found) > 1 or (len(found) == 1 and latin > 0.3):
            return PiscesLxLanguageType.MIXED
        if found:
            return found[0]
        return cls._detect_latin_language(text) if latin > 0.8 else PiscesLxLanguageType.UNKNOWN


class PiscesLxDataDomainClassifier:
    """Keyword overlap per domain: 0.6 x coverage of the domain's keyword set + 0.4 x density in the text; the best
    domain wins unless its score stays under 0.01 (then "general")."""

    _DOMAIN_KEYWORDS: Dict[str, frozenset] = {k: frozenset(v.split()) for k, v in {
        "code": "function class method variable array object string integer boolean loop condition algorithm api database "
                "server client request response debug compile runtime library framework module def import return const",
        "math": "equation formula calculate solve theorem proof integral derivative matrix vector polynomial algebra geometry "
                "calculus probability statistics coefficient exponential logarithm",
        "science": "experiment hypothesis theory research study analysis observation result conclusion molecule atom cell "
                   "organism species evolution physics chemistry biology laboratory",
        "medical": "patient treatment diagnosis symptom medicine doctor hospital disease therapy drug dosage clinical surgery "
                   "prescription health medical vaccine virus bacteria infection chronic",
        "finance": "investment market stock trading financial portfolio asset equity bond dividend interest bank loan credit "
                   "debt revenue profit loss currency exchange inflation gdp economic",
        "legal": "law court judge attorney lawyer contract lawsuit verdict defendant plaintiff legal rights violation penalty "
                 "regulation compliance jurisdiction statute amendment constitution",
        "education": "student teacher school university education learning curriculum exam grade course lesson homework "
                     "assignment lecture professor academic degree diploma scholarship enrollment",
        "technology": "software hardware computer internet network digital technology device application platform cloud "
                      "security encryption artificial intelligence machine automation",
        "news": "breaking report journalist headline article news update coverage broadcast media press announced confirmed "
                "according sources official statement spokesperson incident",
        "social": "friend family relationship social community people person life love happiness emotion feeling experience "
                  "memory story journey together share connect support care",
    }.items()}

    @classmethod
    def get_multi_domain_scores(cls, text: Any) -> Dict[str, float]:
        if not isinstance(text, str) or not text:
            return {}
        words = re.findall(r"[a-z]+", text.lower())
        if not words:
            return {d: 0.0 for d in cls._DOMAIN_KEYWORDS}
        bag = Counter(words)
        out = {}
        for d, kws in cls._DOMAIN_KEYWORDS.items():
            hit_types = sum(1 for k in kws if k in bag)
            hit_tokens = sum(bag[k] for k in kws if k in bag)
            out[d] = 0.6 * hit_types / len(kws) + 0.4 * hit_tokens / len(words)
        return out

    @classmethod
    def classify(cls, text: Any) -> Tuple[str, float]:
        s = cls.get_multi_domain_scores(text)
        if not s:
            return "general", 0.0
        best = max(s, key=s.get)
        return (best, s[best]) if s[best] >= 0.01 else ("general", s[best])


class PiscesLxDataPerplexityCalculator:
    """``calculate(text)``: exp(-mean log-probability) under ``token_logprobs`` when one is given, otherwise the mean
    of 2^H(unigrams) and 2^H(bigrams) of the text's own words (a repetitiveness measure: low for boilerplate)."""

    def __init__(self, token_logprobs: Optional[Callable[[str], Sequence[float]]] = None, max_chars: int = 20000):
        self._lp, self.max_chars = token_logprobs, max_chars

    @staticmethod
    def _entropy(items: Sequence[Any]) -> float:
        n = len(items)
        return -sum(c / n * math.log2(c / n) for c in Counter(items).values())

    @classmethod
    def _estimate_perplexity(cls, text: str) -> float:
        words = re.findall(r"\w+", text.lower())
        if not words:
            return float("inf")
        ppl = 2 ** cls._entropy(words)
        if len(words) > 1:
            ppl = 0.5 * (ppl + 2 ** cls._entropy(list(zip(words[:-1], words[1:]))))
        return ppl

    def calculate(self, text: Any) -> Optional[float]:
        if not isinstance(text, str) or not text.strip():
            return None
        text = text[: self.max_chars]
        if self._lp is not None:
            lps = [float(x) for x in self._lp(text)]
            if lps:
                return math.exp(-sum(lps) / len(lps))
        return self._estimate_perplexity(text)


class PiscesLxDataReadabilityScorer:
    """Flesch reading ease mapped to [0, 1] for alphabetic languages; for Chinese / Japanese / Korean a score from the
    sentence length in characters (20-40 characters per sentence reads best)."""

    @staticmethod
    def _count_syllables(word: str) -> int:
        word = word.lower()
        n, prev = 0, False
        for ch in word:
            v = ch in "aeiouy"
            n += int(v and not prev)
            prev = v
        if word.endswith("e") and not word.endswith("le"):
            n -= 1
        return max(1, n)

    @classmethod
    def _calculate_english_readability(cls, text: str) -> float:
        sentences = [s for s in re.split(r"[.!?]+", text) if s.strip()]
        words = re.findall(r"[^\W\d_]+", text)
        if not sentences or not words:
            return 0.0
        syll = sum(cls._count_syllables(w) for w in words)
        flesch = 206.835 - 1.015 * len(words) / len(sentences) - 84.6 * syll / len(words)
        return max(0.0, min(100.0, flesch)) / 100.0

    @staticmethod
    def _calculate_asian_readability(text: str) -> float:
        chars = [c for c in text if not c.isspace()]
        if not chars:
            return 0.0
        sentences = [s for s in re.split(r"[。！？!?\.]+", text) if s.strip()]
        per = len(chars) / max(len(sentences), 1)
        return max(0.0, min(1.0, 1.0 - abs(per - 30.0) / 120.0))

    @classmethod
    def calculate(cls, text: Any, language: Any = "english") -> float:
        if not isinstance(text, str) or not text.strip():
            return 0.0
        lang = getattr(language, "value", language)
        return cls._calculate_asian_readability(text) if lang in ("chinese", "japanese", "korean") \
            else cls._calculate_english_readability(text)


# ---------------------------------------------------------------------------------------------------------------------------
class PiscesLxCleaningMode(str, Enum):
    LOCAL = "local"
    MULTIPROCESS = "multiprocess"


@dataclass
class PiscesLxDataCleaningConfig:
    batch_size: int = 1000
    max_workers: int = 4
    quality_threshold: float = 0.5
    min_text_length: int = 1
    max_text_length: int = 65536
    enable_quality_scoring: bool = True
    enable_incremental: bool = False
    checkpoint_interval: int = 5000
    mode: PiscesLxCleaningMode = PiscesLxCleaningMode.LOCAL
    preserve_metadata: bool = True
    dedup_enabled: bool = False
    dedup_method: str = "minhash"              # "exact" | "minhash"
    dedup_threshold: float = 0.8
    allowed_languages: Optional[Tuple[str, ...]] = None


class PiscesLxDataIncrementalState:
    """Ledger of the files already cleaned (path -> content hash) so that a re-run only touches new or changed files.
    Written atomically; safe to share between threads."""

    def __init__(self, state_path: str):
        self.state_path = state_path
        self.processed_files: Dict[str, str] = {}
        self.processed_samples = 0
        self.last_checkpoint = 0
        self._lock = threading.Lock()
        if os.path.exists(state_path):
            try:
                with open(state_path, encoding="utf-8") as f:
                    d = json.load(f)
                self.processed_files = dict(d.get("processed_files", {}))
                self.processed_samples = int(d.get("processed_samples", 0))
                self.last_checkpoint = int(d.get("last_checkpoint", 0))
            except (OSError, ValueError):
                pass                                           # an unreadable ledger means: start over

    @staticmethod
    def _compute_file_hash(file_path: str) -> str:
        h = hashlib.blake2b(digest_size=16)
        with open(file_path, "rb") as f:
            for chunk in iter(lambda: f.read(1 << 20), b""):
                h.update(chunk)
        return h.hexdigest()

    def is_processed(self, file_path: str) -> bool:
        if not os.path.exists(file_path):
            return False
        digest = self._compute_file_hash(file_path)
        with self._lock:
            return self.processed_files.get(file_path) == digest

    def mark_processed(self, file_path: str, sample_count: int = 0) -> None:
        digest = self._compute_file_hash(file_path)
        with self._lock:
            self.processed_files[file_path] = digest
            self.processed_samples += sample_count

    def save_state(self) -> None:
        with self._lock:
            os.makedirs(os.path.dirname(os.path.abspath(self.state_path)), exist_ok=True)
            tmp = self.state_path + ".tmp"
            with open(tmp, "w", encoding="utf-8") as f:
                json.dump({"processed_files": self.processed_files, "processed_samples": self.processed_samples,
                           "last_checkpoint": self.last_checkpoint}, f, indent=2)
            os.replace(tmp, self.state_path)


_CTRL = re.compile(r"[\x00-\x08\x0b\x0c\x0e-\x1f\x7f-\x9f]")


class PiscesLxDataQualityAwareCleaner:
    """normalise -> length limits -> quality score -> keep or filter, with counters.  The score combines the share of
    letters, the lexical variety, the word-length plausibility, the readability and (inverted) repetitiveness."""

    def __init__(self, config: Optional[PiscesLxDataCleaningConfig] = None,
                 perplexity: Optional[PiscesLxDataPerplexityCalculator] = None):
        self.config = config or PiscesLxDataCleaningConfig()
        self.perplexity = perplexity or PiscesLxDataPerplexityCalculator()
        self._stats = {"total_processed": 0, "high_quality": 0, "medium_quality": 0, "low_quality": 0, "filtered_out": 0,
                       "duplicates": 0}
        c = self.config
        self._dedup = None
        if c.dedup_enabled:
            self._dedup = PiscesLxDataExactDeduplicator() if c.dedup_method == "exact" else \
                PiscesLxDataMinHashDeduplicator(threshold=c.dedup_threshold)

    @staticmethod
    def _normalize_text(text: Any) -> str:
        t = _CTRL.sub("", str(text).strip())
        t = re.sub(r"\s+", " ", t)
        t = re.sub(r"([.!?])\1+", r"\1", t)                   # "!!!" -> "!"
        return re.sub(r"(.)\1{4,}", r"\1\1\1", t).strip()     # "soooooo" -> "sooo"

    def quality_score(self, text: str, language: PiscesLxLanguageType) -> Dict[str, float]:
        n = max(len(text), 1)
        cjk = language in (PiscesLxLanguageType.CHINESE, PiscesLxLanguageType.JAPANESE, PiscesLxLanguageType.KOREAN)
        units = [c for c in text if not c.isspace()] if cjk else text.split()
        alpha = sum(c.isalpha() for c in text) / n
        variety = len(set(units)) / max(len(units), 1)
        mwl = 1.0 if cjk else (sum(map(len, units)) / max(len(units), 1))
        word_ok = 1.0 if cjk or 3 <= mwl <= 10 else 0.3
        read = PiscesLxDataReadabilityScorer.calculate(text, language)
        ppl = self.perplexity._estimate_perplexity(text) if not cjk else float(len(set(units)))
        rep = min(1.0, math.log2(ppl + 1) / 6.0) if math.isfinite(ppl) else 0.0      # 64 distinct patterns saturate
        score = 0.3 * min(alpha / 0.7, 1.0) + 0.25 * min(variety / (0.3 if cjk else 0.5), 1.0) + 0.15 * word_ok + 0.15 * read + 0.15 * rep
        floor = 0.1 if cjk else 0.2
        if len(units) >= 8 and variety < floor:               # a handful of tokens repeated over and over
            score *= variety / floor
        return {"quality_score": score, "alpha_ratio": alpha, "variety": variety, "readability": read, "perplexity": ppl}

    def clean_with_quality(self, text: Any) -> Tuple[str, float, Dict[str, Any]]:
        """Returns (text, score, metrics); a filtered sample has a ``reason`` in its metrics and, when it is empty or
        too short, an empty text."""
        c = self.config
        if not isinstance(text, str) or not text:
            return "", 0.0, {"reason": "empty_or_invalid"}
        t = self._normalize_text(text)
        if len(t) < c.min_text_length:
            return "", 0.0, {"reason": "too_short", "length": len(t)}
        t = t[: c.max_text_length]
        lang = PiscesLxDataLanguageDetector.detect(t)
        m: Dict[str, Any] = {"length": len(t), "word_count": len(t.split()), "language": lang.value,
                             "char_diversity": len(set(t.lower())) / max(len(t), 1)}
        if c.allowed_languages is not None and lang.value not in c.allowed_languages:
            self._stats["filtered_out"] += 1
            return t, 0.0, {**m, "reason": "language"}
        if self._dedup is not None and not self._dedup.is_new(t):
            self._stats["duplicates"] += 1
            return t, 0.0, {**m, "reason": "duplicate"}
        if c.enable_quality_scoring:
            m.update(self.quality_score(t, lang))
            m["domain"] = PiscesLxDataDomainClassifier.classify(t)[0]
        else:
            m["quality_score"] = 1.0
        s = m["quality_score"]
        if s < c.quality_threshold:
            self._stats["filtered_out"] += 1
            return t, s, {**m, "reason": "low_quality"}
        self._stats["high_quality" if s >= 0.8 else ("medium_quality" if s >= 0.5 else "low_quality")] += 1
        self._stats["total_processed"] += 1
        return t, s, m

    def clean(self, texts: Iterable[Any]) -> Iterator[Tuple[str, Dict[str, Any]]]:
        """The kept samples with their metrics."""
        for x in texts:
            t, _, m = self.clean_with_quality(x)
            if t and "reason" not in m:
                yield t, m

    def clean_files(self, paths: Sequence[str], out_path: str, state: Optional[PiscesLxDataIncrementalState] = None,
                    text_key: str = "text") -> Dict[str, int]:
        """JSON-lines or plain-text files -> one JSON-lines file of kept samples (appended).  With a ledger, files whose
        content has not changed since they were processed are skipped and the ledger is saved every
        ``checkpoint_interval`` samples and at the end."""
        kept = skipped = seen = 0
        os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
        with open(out_path, "a", encoding="utf-8") as out:
            for p in paths:
                if state is not None and state.is_processed(p):
                    skipped += 1
                    continue
                n_file = 0
                with open(p, encoding="utf-8", errors="replace") as f:
                    for line in f:
                        line = line.strip()
                        if not line:
                            continue
                        meta: Dict[str, Any] = {}
                        if line.startswith("{"):
                            try:
                                meta = json.loads(line)
                                line = str(meta.get(text_key, ""))
                            except ValueError:
                                meta = {}
                        seen += 1
                        t, s, m = self.clean_with_quality(line)
                        if t and "reason" not in m:
                            rec = {text_key: t, "quality": round(s, 4), "language": m["language"], "domain": m.get("domain")}
                            if self.config.preserve_metadata:
                                rec.update({k: v for k, v in meta.items() if k not in rec})
                            out.write(json.dumps(rec, ensure_ascii=False) + "\n")
                            kept += 1
                            n_file += 1
                        if state is not None and seen - state.last_checkpoint >= self.config.checkpoint_interval:
                            state.last_checkpoint = seen
                            state.save_state()
                if state is not None:
                    state.mark_processed(p, n_file)
        if state is not None:
            state.save_state()
        return {"files_skipped": skipped, "samples_seen": seen, "samples_kept": kept}

    def get_stats(self) -> Dict[str, int]:
        return dict(self._stats)
