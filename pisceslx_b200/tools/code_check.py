"""Source checks and the staged self-test (reference tools/check/base.py:51-537, checks_style.py, checks_hygiene.py,
import_census.py, tools/test/core.py, report.py, stages/*.py).

Two small tools a maintainer runs on a checkout, both without a GPU:

* source checks: every rule is one class with ``inspect(source) -> [violation]``; files are read and parsed once and shared by
  all rules (the scanner caches text, lines and the AST).
* staged self-test: environment -> imports -> structure -> config -> model -> forward -> generation -> optimization ->
  memory, each stage a callable returning a result record; a failed stage marks the stages that depend on it as skipped
  rather than running them into the same error."""
from __future__ import annotations

import ast
import importlib
import json
import re
import sys
import time
from dataclasses import asdict, dataclass, field
from enum import Enum
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple


# ---- source checks ------------------------------------------------------------------------------------------------------------
class PiscesLxRuleId:
    HEADER = "header.missing"
    PROJECT_NAME = "style.project_name"
    ABSOLUTE_PATH = "hygiene.absolute_path"
    MODALITY = "hygiene.modality_literal"
    RESIDUAL = "hygiene.residual_system"
    SYNTAX = "parse.syntax_error"

    @classmethod
    def all_rules(cls) -> Tuple[str, ...]:
        return tuple(v for k, v in vars(cls).items() if k.isupper() and isinstance(v, str))


class PiscesLxSeverity:
    ERROR, WARNING = "error", "warning"


class PiscesLxStandardHeader:
    """The leading comment / docstring block every source file is expected to carry; ``required`` lists phrases of which each must appear."""

    def __init__(self, required: Sequence[str] = ()):
        self.required = tuple(required)

    @staticmethod
    def normalize(text: str) -> str:
        return re.sub(r"\s+", " ", re.sub(r"^[#\s]+", "", text, flags=re.M)).strip().lower()

    @staticmethod
    def extract_leading_block(text: str) -> str:
        lines, out = text.splitlines(), []
        i = 1 if lines and lines[0].startswith("#!") else 0
        while i < len(lines) and (lines[i].startswith("#") or not lines[i].strip()):
            out.append(lines[i])
            i += 1
        if not any(l.strip() for l in out):
            try:
                return ast.get_docstring(ast.parse(text)) or ""
            except SyntaxError:
                return ""
        return "\n".join(out)

    def missing(self, text: str) -> List[str]:
        block = self.normalize(self.extract_leading_block(text))
        if not self.required:
            return [] if block else ["a leading comment or docstring"]
        return [r for r in self.required if self.normalize(r) not in block]


@dataclass
class PiscesLxViolation:
    rule: str
    path: Path
    line: int
    message: str
    severity: str = PiscesLxSeverity.ERROR

    def render(self, root: Path) -> str:
        try:
            rel = self.path.relative_to(root)
        except ValueError:
            rel = self.path
        return f"{rel}:{self.line}: [{self.severity}] {self.rule}: {self.message}"


class PiscesLxSourceFile:
    def __init__(self, path: Path, root: Path):
        self.path, self.root = Path(path), Path(root)
        self._text: Optional[str] = None
        self._tree: Any = None
        self.parse_error = ""

    @property
    def text(self) -> str:
        if self._text is None:
            self._text = self.path.read_text(encoding="utf-8", errors="replace")
        return self._text

    @property
    def lines(self) -> List[str]:
        return self.text.splitlines()

    @property
    def tree(self) -> Optional[ast.Module]:
        if self._tree is None and not self.parse_error:
            try:
                self._tree = ast.parse(self.text)
            except SyntaxError as e:
                self.parse_error = f"line {e.lineno}: {e.msg}"
        return self._tree

    @property
    def is_init(self) -> bool:
        return self.path.name == "__init__.py"

    def line_source(self, line: int) -> str:
        ls = self.lines
        return ls[line - 1] if 0 < line <= len(ls) else ""


class PiscesLxRepositoryScanner:
    SKIP = {".git", "__pycache__", "build", "dist", ".venv", "node_modules", "_work"}

    def __init__(self, root: Path, explicit_paths: Iterable[Path] = ()):
        self.root = Path(root)
        paths = [Path(p) for p in explicit_paths] or [self.root]
        found = set()
        for p in paths:
            if p.is_file() and p.suffix == ".py":
                found.add(p)
            elif p.is_dir():
                found.update(q for q in p.rglob("*.py") if not (set(q.relative_to(p).parts[:-1]) & self.SKIP))
        self.files = tuple(PiscesLxSourceFile(p, self.root) for p in sorted(found))


class PiscesLxAstWalker:
    @staticmethod
    def iter_classes(tree: ast.Module) -> Iterator[ast.ClassDef]:
        return (n for n in ast.walk(tree) if isinstance(n, ast.ClassDef))

    @staticmethod
    def iter_functions(tree: ast.Module) -> Iterator[ast.AST]:
        return (n for n in ast.walk(tree) if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef)))

    @staticmethod
    def parents(tree: ast.Module) -> Dict[ast.AST, ast.AST]:
        return {c: p for p in ast.walk(tree) for c in ast.iter_child_nodes(p)}

    @classmethod
    def enclosing_classes(cls, tree: ast.Module) -> Dict[ast.AST, Tuple[str, ...]]:
        out: Dict[ast.AST, Tuple[str, ...]] = {}

        def visit(node: ast.AST, chain: Tuple[str, ...]) -> None:
            for c in ast.iter_child_nodes(node):
                out[c] = chain
                visit(c, chain + (c.name,) if isinstance(c, ast.ClassDef) else chain)
        visit(tree, ())
        return out

    @staticmethod
    def is_inside_class(node: ast.AST, parents: Dict[ast.AST, ast.AST]) -> bool:
        while node in parents:
            node = parents[node]
            if isinstance(node, ast.ClassDef):
                return True
        return False

    @staticmethod
    def _is_main_test(test: ast.expr) -> bool:
        return (isinstance(test, ast.Compare) and isinstance(test.left, ast.Name) and test.left.id == "__name__" and len(test.comparators) == 1
                and isinstance(test.comparators[0], ast.Constant) and test.comparators[0].value == "__main__")

    @classmethod
    def is_inside_main_guard(cls, node: ast.AST, parents: Dict[ast.AST, ast.AST]) -> bool:
        while node in parents:
            node = parents[node]
            if isinstance(node, ast.If) and cls._is_main_test(node.test):
                return True
        return False


class PiscesLxRegexLibrary:
    ABSOLUTE_PATHS = (re.compile(r"""["'](/home/|/Users/|/root/|[A-Z]:\\\\)[^"']*["']"""),)
    TODO = re.compile(r"#\s*(TODO|FIXME|XXX)\b", re.I)

    @classmethod
    def absolute_path_patterns(cls) -> Tuple[re.Pattern, ...]:
        return cls.ABSOLUTE_PATHS

    @staticmethod
    def matches_any(text: str, patterns: Sequence[re.Pattern]) -> bool:
        return any(p.search(text) for p in patterns)


class PiscesLxStandardCheck:
    rule, severity = "", PiscesLxSeverity.ERROR

    def inspect(self, source: PiscesLxSourceFile) -> List[PiscesLxViolation]:
        raise NotImplementedError

    def run(self, scanner: PiscesLxRepositoryScanner) -> List[PiscesLxViolation]:
        out = []
        for s in scanner.files:
            if s.tree is None and s.parse_error:
                continue
            out += self.inspect(s)
        return out

    def _v(self, s: PiscesLxSourceFile, line: int, msg: str) -> PiscesLxViolation:
        return PiscesLxViolation(self.rule, s.path, line, msg, self.severity)


class PiscesLxCopyrightHeaderCheck(PiscesLxStandardCheck):
    rule = PiscesLxRuleId.HEADER

    def __init__(self, header: Optional[PiscesLxStandardHeader] = None):
        self.header = header or PiscesLxStandardHeader()

    def inspect(self, s: PiscesLxSourceFile) -> List[PiscesLxViolation]:
        if not s.text.strip():
            return []
        miss = self.header.missing(s.text)
        return [self._v(s, 1, "header lacks " + "; ".join(miss))] if miss else []


class PiscesLxProjectNameCheck(PiscesLxStandardCheck):
    """Public classes carry one of the project's prefixes; private (underscore) and nested classes are exempt."""

    rule, severity = PiscesLxRuleId.PROJECT_NAME, PiscesLxSeverity.WARNING

    def __init__(self, prefixes: Sequence[str] = ("PiscesLx", "Yv", "POPSS"), exempt: Sequence[str] = ()):
        self.prefixes, self.exempt = tuple(prefixes), set(exempt)

    def inspect(self, s: PiscesLxSourceFile) -> List[PiscesLxViolation]:
        return [self._v(s, n.lineno, f"class {n.name} has none of the prefixes {', '.join(self.prefixes)}") for n in s.tree.body
                if isinstance(n, ast.ClassDef) and not n.name.startswith("_") and n.name not in self.exempt and not n.name.startswith(self.prefixes)]


class PiscesLxAbsolutePathCheck(PiscesLxStandardCheck):
    rule = PiscesLxRuleId.ABSOLUTE_PATH

    def inspect(self, s: PiscesLxSourceFile) -> List[PiscesLxViolation]:
        pats = PiscesLxRegexLibrary.absolute_path_patterns()
        return [self._v(s, i, "machine-specific absolute path") for i, l in enumerate(s.lines, 1) if PiscesLxRegexLibrary.matches_any(l, pats)]


class PiscesLxModalityCheck(PiscesLxStandardCheck):
    """Comparisons against a bare modality string (``x == "image"``) outside the module that defines the enumeration: use the enumeration."""

    rule, severity = PiscesLxRuleId.MODALITY, PiscesLxSeverity.WARNING
    NAMES = {"text", "image", "audio", "video", "document"}

    def __init__(self, defining_modules: Sequence[str] = ("core_types.py", "types.py")):
        self.defining = set(defining_modules)

    def inspect(self, s: PiscesLxSourceFile) -> List[PiscesLxViolation]:
        if s.path.name in self.defining:
            return []
        out = []
        for n in ast.walk(s.tree):
            if isinstance(n, ast.Compare) and any(isinstance(op, (ast.Eq, ast.NotEq)) for op in n.ops):
                for c in [n.left, *n.comparators]:
                    if isinstance(c, ast.Constant) and c.value in self.NAMES and "modal" in ast.unparse(n).lower():
                        out.append(self._v(s, n.lineno, f"compares against the literal {c.value!r}"))
        return out


class PiscesLxResidualSystemCheck(PiscesLxStandardCheck):
    """Leftovers: imports of modules that were removed (``removed`` maps module -> replacement) and marker comments."""

    rule = PiscesLxRuleId.RESIDUAL

    def __init__(self, removed: Optional[Dict[str, str]] = None, flag_markers: bool = False):
        self.removed, self.flag_markers = dict(removed or {}), flag_markers

    def inspect(self, s: PiscesLxSourceFile) -> List[PiscesLxViolation]:
        out = []
        for n in ast.walk(s.tree):
            mods = [a.name for a in n.names] if isinstance(n, ast.Import) else [n.module or ""] if isinstance(n, ast.ImportFrom) else []
            for m in mods:
                for gone, repl in self.removed.items():
                    if m == gone or m.startswith(gone + ".") or m.endswith("." + gone):
                        out.append(self._v(s, n.lineno, f"imports removed module {gone}" + (f"; use {repl}" if repl else "")))
        if self.flag_markers:
            out += [self._v(s, i, "marker comment left in") for i, l in enumerate(s.lines, 1) if PiscesLxRegexLibrary.TODO.search(l)]
        return out


@dataclass
class PiscesLxCheckReport:
    root: Path
    violations: List[PiscesLxViolation]
    checks_run: int
    files_scanned: int
    duration_s: float

    @property
    def errors(self) -> List[PiscesLxViolation]:
        return [v for v in self.violations if v.severity == PiscesLxSeverity.ERROR]

    @property
    def warnings(self) -> List[PiscesLxViolation]:
        return [v for v in self.violations if v.severity == PiscesLxSeverity.WARNING]

    def by_rule(self) -> Dict[str, int]:
        out: Dict[str, int] = {}
        for v in self.violations:
            out[v.rule] = out.get(v.rule, 0) + 1
        return out

    @property
    def exit_code(self) -> int:
        return 1 if self.errors else 0

    def render(self, verbose: bool = True, max_rows: int = 0) -> str:
        rows = [v.render(self.root) for v in sorted(self.violations, key=lambda v: (str(v.path), v.line))]
        if max_rows:
            rows = rows[:max_rows]
        head = f"{self.files_scanned} files, {self.checks_run} checks, {len(self.errors)} errors, {len(self.warnings)} warnings in {self.duration_s:.2f}s"
        return "\n".join(([*rows, ""] if verbose else []) + [head] + [f"  {r}: {n}" for r, n in sorted(self.by_rule().items())])


class PiscesLxCheckRunner:
    def __init__(self, root: Path, checks: Optional[Sequence[PiscesLxStandardCheck]] = None):
        self.root = Path(root)
        self.checks = list(checks) if checks is not None else [PiscesLxCopyrightHeaderCheck(), PiscesLxAbsolutePathCheck(), PiscesLxResidualSystemCheck()]

    def run(self, paths: Iterable[Path] = ()) -> PiscesLxCheckReport:
        t0 = time.perf_counter()
        sc = PiscesLxRepositoryScanner(self.root, paths)
        v = [PiscesLxViolation(PiscesLxRuleId.SYNTAX, s.path, 1, s.parse_error) for s in sc.files if s.tree is None and s.parse_error]
        for c in self.checks:
            v += c.run(sc)
        return PiscesLxCheckReport(self.root, v, len(self.checks), len(sc.files), time.perf_counter() - t0)


class PiscesLxImportCensusCli:
    """Counts what a source tree imports: per top-level package, how many files import it, and which are neither standard library nor the tree's own."""

    def __init__(self, root: Path, own: Sequence[str] = ("pisceslx_b200",)):
        self.root, self.own = Path(root), set(own)

    def census(self) -> Dict[str, Any]:
        counts: Dict[str, set] = {}
        sc = PiscesLxRepositoryScanner(self.root)
        for s in sc.files:
            if s.tree is None:
                continue
            for n in ast.walk(s.tree):
                mods = [a.name for a in n.names] if isinstance(n, ast.Import) else [n.module] if isinstance(n, ast.ImportFrom) and n.level == 0 and n.module else []
                for m in mods:
                    counts.setdefault(m.split(".")[0], set()).add(str(s.path))
        std = set(sys.stdlib_module_names)
        table = {k: len(v) for k, v in sorted(counts.items(), key=lambda kv: -len(kv[1]))}
        return {"files": len(sc.files), "imports": table, "third_party": [k for k in table if k not in std and k not in self.own], "stdlib": [k for k in table if k in std]}

    def run(self, argv: Optional[Sequence[str]] = None, out: Callable[[str], None] = print) -> int:
        c = self.census()
        if argv and "--json" in argv:
            out(json.dumps(c, indent=1))
        else:
            out(f"{c['files']} files")
            for k in c["third_party"]:
                out(f"  {k:<24}{c['imports'][k]:>5} files")
        return 0


# ---- staged self-test ---------------------------------------------------------------------------------------------------------
class PiscesLxTestStatus(str, Enum):
    PASSED, FAILED, SKIPPED, WARNING = "passed", "failed", "skipped", "warning"


@dataclass
class PiscesLxTestResult:
    name: str
    status: PiscesLxTestStatus
    seconds: float = 0.0
    message: str = ""
    details: Dict[str, Any] = field(default_factory=dict)


@dataclass
class PiscesLxTestReport:
    results: List[PiscesLxTestResult] = field(default_factory=list)

    def add(self, r: PiscesLxTestResult) -> None:
        self.results.append(r)

    def count(self, status: PiscesLxTestStatus) -> int:
        return sum(r.status == status for r in self.results)

    @property
    def ok(self) -> bool:
        return self.count(PiscesLxTestStatus.FAILED) == 0

    def to_dict(self) -> Dict[str, Any]:
        return {"ok": self.ok, "results": [{**asdict(r), "status": r.status.value} for r in self.results]}

    def render(self) -> str:
        rows = [f"{r.status.value.upper():<8}{r.name:<16}{r.seconds:7.2f}s  {r.message}" for r in self.results]
        return "\n".join(rows + [f"{self.count(PiscesLxTestStatus.PASSED)} passed, {self.count(PiscesLxTestStatus.FAILED)} failed, {self.count(PiscesLxTestStatus.SKIPPED)} skipped"])

    def save(self, path: str) -> str:
        Path(path).write_text(json.dumps(self.to_dict(), indent=1, default=str))
        return path


class _StageChecker:
    name, requires = "", ()

    def check(self, ctx: Dict[str, Any]) -> Dict[str, Any]:
        raise NotImplementedError


class PiscesLxEnvironmentChecker(_StageChecker):
    name = "environment"

    def check(self, ctx):
        import torch
        d = {"python": sys.version.split()[0], "torch": torch.__version__, "cuda": torch.cuda.is_available()}
        if d["cuda"]:
            d["device"], d["capability"] = torch.cuda.get_device_name(0), list(torch.cuda.get_device_capability(0))
        if sys.version_info < (3, 10):
            raise RuntimeError("Python 3.10 or newer is needed")
        return d


class PiscesLxImportChecker(_StageChecker):
    name, requires = "imports", ("environment",)
    MODULES = ("pisceslx_b200", "pisceslx_b200.config", "pisceslx_b200.models.model", "pisceslx_b200.engine", "pisceslx_b200.serve", "pisceslx_b200.optim", "pisceslx_b200.quant", "pisceslx_b200.data")

    def __init__(self, modules: Optional[Sequence[str]] = None):
        self.modules = tuple(modules or self.MODULES)

    def check(self, ctx):
        bad = {}
        for m in self.modules:
            try:
                importlib.import_module(m)
            except Exception as e:
                bad[m] = f"{type(e).__name__}: {e}"
        if bad:
            raise RuntimeError("; ".join(f"{k} ({v})" for k, v in bad.items()))
        return {"modules": len(self.modules)}


class PiscesLxStructureChecker(_StageChecker):
    name, requires = "structure", ("imports",)
    EXPECTED = ("models", "ops", "parallel", "engine", "serve", "optim", "quant", "data", "tools", "utils", "third_party")

    def check(self, ctx):
        import pisceslx_b200
        root = Path(pisceslx_b200.__file__).parent
        miss = [d for d in self.EXPECTED if not (root / d / "__init__.py").exists()]
        if miss:
            raise RuntimeError("missing packages: " + ", ".join(miss))
        return {"packages": len(self.EXPECTED), "root": root.name}


class PiscesLxConfigChecker(_StageChecker):
    name, requires = "config", ("imports",)

    def check(self, ctx):
        from ..config import YvConfig
        cfg = ctx.get("config") or YvConfig(vocab_size=512, hidden_size=64, n_layer=2, n_head=4, n_kv_head=2, intermediate_size=128, max_position_embeddings=128)
        if cfg.hidden_size % cfg.n_head:
            raise RuntimeError("hidden_size is not a multiple of n_head")
        ctx["config"] = cfg
        n = cfg.count_parameters()
        return {"parameters": n["total"] if isinstance(n, dict) else int(n)}


class PiscesLxModelChecker(_StageChecker):
    name, requires = "model", ("config",)

    def check(self, ctx):
        import torch
        from ..models.model import YvModelForCausalLM
        torch.manual_seed(0)
        ctx["model"] = YvModelForCausalLM(ctx["config"]).to(ctx.get("device", "cpu"))
        return {"parameters": sum(p.numel() for p in ctx["model"].parameters())}


def _logits(out: Any):
    return out["logits"] if isinstance(out, dict) else out.logits if hasattr(out, "logits") else out[0] if isinstance(out, (tuple, list)) else out


class PiscesLxForwardChecker(_StageChecker):
    name, requires = "forward", ("model",)

    def check(self, ctx):
        import torch
        m, cfg = ctx["model"], ctx["config"]
        ids = torch.randint(0, cfg.vocab_size, (2, 16), device=next(m.parameters()).device)
        lg = _logits(m(ids, return_logits=True))
        if tuple(lg.shape) != (2, 16, cfg.vocab_size) or not bool(torch.isfinite(lg).all()):
            raise RuntimeError(f"logits {tuple(lg.shape)} wrong or not finite")
        loss = torch.nn.functional.cross_entropy(lg[:, :-1].reshape(-1, cfg.vocab_size).float(), ids[:, 1:].reshape(-1))
        loss.backward()
        g = [p.grad for p in m.parameters() if p.grad is not None]
        m.zero_grad(set_to_none=True)
        if not g:
            raise RuntimeError("no parameter received a gradient")
        return {"loss": float(loss.detach()), "tensors_with_grad": len(g)}


class PiscesLxGenerationChecker(_StageChecker):
    name, requires = "generation", ("forward",)

    def check(self, ctx):
        import torch
        m, cfg = ctx["model"].eval(), ctx["config"]
        ids = torch.randint(0, cfg.vocab_size, (1, 4), device=next(m.parameters()).device)
        with torch.no_grad():
            for _ in range(4):
                ids = torch.cat([ids, _logits(m(ids, return_logits=True))[:, -1].argmax(-1, keepdim=True)], 1)
        m.train()
        return {"tokens": ids.shape[1]}


class PiscesLxOptimizationChecker(_StageChecker):
    name, requires = "optimization", ("forward",)

    def check(self, ctx):
        import torch
        m, cfg = ctx["model"], ctx["config"]
        opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
        ids = torch.randint(0, cfg.vocab_size, (2, 16), device=next(m.parameters()).device)
        losses = []
        for _ in range(4):
            lg = _logits(m(ids, return_logits=True))
            loss = torch.nn.functional.cross_entropy(lg[:, :-1].reshape(-1, cfg.vocab_size).float(), ids[:, 1:].reshape(-1))
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
            losses.append(float(loss.detach()))
        if not losses[-1] < losses[0]:
            raise RuntimeError(f"loss did not fall on a repeated batch: {losses}")
        return {"first": losses[0], "last": losses[-1]}


class PiscesLxMemoryOptChecker(_StageChecker):
    name, requires = "memory_opt", ("model",)

    def check(self, ctx):
        import torch
        from torch.utils.checkpoint import checkpoint
        lin = torch.nn.Linear(16, 16)
        x = torch.randn(4, 16, requires_grad=True)
        a = lin(x).relu().sum()
        b = checkpoint(lambda t: lin(t).relu(), x, use_reentrant=False).sum()
        if not torch.allclose(a, b):
            raise RuntimeError("recomputation changed the result")
        return {"checkpoint_matches": True}


class PiscesLxRegressionSuiteChecker(_StageChecker):
    """Runs the repository's CPU tests that match ``pattern`` through pytest, when a ``tests`` folder sits beside the package."""

    name, requires = "regressions", ("imports",)

    def __init__(self, pattern: str = "test_config", tests_dir: Optional[str] = None):
        self.pattern, self.tests_dir = pattern, tests_dir

    def check(self, ctx):
        import subprocess
        import pisceslx_b200
        d = Path(self.tests_dir) if self.tests_dir else Path(pisceslx_b200.__file__).parent.parent / "tests"
        if not d.is_dir():
            return {"skipped": "no tests folder"}
        p = subprocess.run([sys.executable, "-m", "pytest", str(d), "-q", "-x", "-m", "not gpu", "-k", self.pattern], capture_output=True, text=True, timeout=900)
        if p.returncode not in (0, 5):
            raise RuntimeError(p.stdout[-500:])
        return {"summary": p.stdout.strip().splitlines()[-1] if p.stdout.strip() else ""}


class PiscesLxTestRunner:
    DEFAULT = (PiscesLxEnvironmentChecker, PiscesLxImportChecker, PiscesLxStructureChecker, PiscesLxConfigChecker, PiscesLxModelChecker,
               PiscesLxForwardChecker, PiscesLxGenerationChecker, PiscesLxOptimizationChecker, PiscesLxMemoryOptChecker)

    def __init__(self, stages: Optional[Sequence[_StageChecker]] = None, context: Optional[Dict[str, Any]] = None):
        self.stages = list(stages) if stages is not None else [c() for c in self.DEFAULT]
        self.context = dict(context or {})

    def run(self, only: Optional[Sequence[str]] = None) -> PiscesLxTestReport:
        rep, status = PiscesLxTestReport(), {}
        for st in self.stages:
            if only and st.name not in only and not any(st.name in getattr(o, "requires", ()) for o in self.stages if o.name in only):
                continue
            blocked = [r for r in st.requires if status.get(r) in (PiscesLxTestStatus.FAILED, PiscesLxTestStatus.SKIPPED)]
            if blocked:
                res = PiscesLxTestResult(st.name, PiscesLxTestStatus.SKIPPED, message="needs " + ", ".join(blocked))
            else:
                t0 = time.perf_counter()
                try:
                    d = st.check(self.context)
                    res = PiscesLxTestResult(st.name, PiscesLxTestStatus.PASSED, time.perf_counter() - t0, details=d or {})
                except Exception as e:
                    res = PiscesLxTestResult(st.name, PiscesLxTestStatus.FAILED, time.perf_counter() - t0, f"{type(e).__name__}: {e}")
            status[st.name] = res.status
            rep.add(res)
        return rep


class PiscesLxTestCli:
    def run(self, argv: Optional[Sequence[str]] = None, out: Callable[[str], None] = print) -> int:
        import argparse
        ap = argparse.ArgumentParser(prog="pisceslx test")
        ap.add_argument("--stage", action="append")
        ap.add_argument("--json")
        ap.add_argument("--device", default="cpu")
        a = ap.parse_args(list(argv or []))
        rep = PiscesLxTestRunner(context={"device": a.device}).run(a.stage)
        out(rep.render())
        if a.json:
            rep.save(a.json)
        return 0 if rep.ok else 1
