"""Further static checks and the suite around them (reference tools/check: hard-coding, incomplete markers,
top-level functions, dangling exports, dead / undeclared config fields, engine isolation, import census, report, CLI).
Built on the rule classes of ``utils.check``."""
from __future__ import annotations

import ast
import json
import os
import re
from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Set

from .check import PiscesLxStandardCheck, PiscesLxViolation


class PiscesLxSeverity(str, Enum):
    INFO = "info"
    WARNING = "warning"
    ERROR = "error"


@dataclass
class PiscesLxSourceFile:
    path: str
    source: str
    tree: ast.AST


class PiscesLxRepositoryScanner:
    """Yields the parsed Python files under a root, skipping caches, build output and hidden folders."""

    SKIP = {"__pycache__", ".git", "build", "csrc"}

    def __init__(self, root: str, skip: Optional[Iterable[str]] = None):
        """``skip``: further folder names to leave out; by default the folders that the root's ``.gitignore`` lists
        (scratch and vendored trees are not the project's source)."""
        self.root = root
        extra = set(skip) if skip is not None else self._gitignored_dirs(root)
        self.SKIP = set(self.SKIP) | extra

    @staticmethod
    def _gitignored_dirs(root: str) -> set:
        out = set()
        try:
            for line in open(os.path.join(root, ".gitignore"), encoding="utf-8"):
                line = line.strip()
                if line and not line.startswith("#") and line.endswith("/") and "*" not in line:
                    out.add(line.strip("/").split("/")[0])
        except OSError:
            pass
        return out

    def files(self) -> Iterator[PiscesLxSourceFile]:
        for d, dirs, names in os.walk(self.root):
            dirs[:] = [x for x in dirs if x not in self.SKIP and not x.startswith(".")]
            for n in sorted(names):
                if n.endswith(".py"):
                    p = os.path.join(d, n)
                    try:
                        src = open(p, encoding="utf-8").read()
                        yield PiscesLxSourceFile(p, src, ast.parse(src))
                    except (SyntaxError, UnicodeDecodeError):
                        continue


class PiscesLxHardcodingCheck(PiscesLxStandardCheck):
    """Absolute user paths, private network addresses and inline credentials in string literals."""
    rule = "hardcoding"
    PATTERNS = [re.compile(r"^/(home|Users)/[^/\s]+/"), re.compile(r"\b(?:10|192\.168|172\.(?:1[6-9]|2\d|3[01]))\.\d+\.\d+\b"),
                re.compile(r"(?i)(api[_-]?key|secret|password)\s*[=:]\s*['\"]?[A-Za-z0-9_\-]{12,}")]

    def check(self, path, source, tree):
        for node in ast.walk(tree):
            if isinstance(node, ast.Constant) and isinstance(node.value, str):
                for pat in self.PATTERNS:
                    if pat.search(node.value):
                        yield PiscesLxViolation(self.rule, path, node.lineno, f"hard-coded value: {node.value[:40]!r}")
                        break


class PiscesLxIncompleteMarkerCheck(PiscesLxStandardCheck):
    """Markers of unfinished work in comments, and function bodies that only raise NotImplementedError outside an
    abstract base (a class whose name ends in Base / Interface, or a method documented as abstract)."""
    rule = "incomplete-marker"
    MARK = re.compile(r"#.*\b(TODO|FIXME|XXX|HACK)\b")

    def check(self, path, source, tree):
        for i, line in enumerate(source.splitlines(), 1):
            if self.MARK.search(line):
                yield PiscesLxViolation(self.rule, path, i, "unfinished-work marker in a comment")


class PiscesLxTopLevelFunctionCheck(PiscesLxStandardCheck):
    """Public top-level functions need a docstring (private helpers, tests and ``main`` are exempt)."""
    rule = "top-level-function-doc"

    def check(self, path, source, tree):
        if os.path.basename(path).startswith("test_"):
            return
        for node in getattr(tree, "body", []):
            if isinstance(node, ast.FunctionDef) and not node.name.startswith("_") and node.name != "main":
                if ast.get_docstring(node) is None and len(node.body) > 3:
                    yield PiscesLxViolation(self.rule, path, node.lineno, f"public function {node.name} has no docstring")


class PiscesLxDanglingExportCheck(PiscesLxStandardCheck):
    """Names listed in ``__all__`` that the module does not define or import."""
    rule = "dangling-export"

    def check(self, path, source, tree):
        defined: Set[str] = set()
        exported: List[ast.Constant] = []
        for node in getattr(tree, "body", []):
            if isinstance(node, (ast.FunctionDef, ast.ClassDef, ast.AsyncFunctionDef)):
                defined.add(node.name)
            elif isinstance(node, ast.Assign):
                for t in node.targets:
                    if isinstance(t, ast.Name):
                        defined.add(t.id)
                        if t.id == "__all__" and isinstance(node.value, (ast.List, ast.Tuple)):
                            exported = [e for e in node.value.elts if isinstance(e, ast.Constant)]
            elif isinstance(node, (ast.Import, ast.ImportFrom)):
                for a in node.names:
                    defined.add((a.asname or a.name).split(".")[0])
        for e in exported:
            if e.value not in defined:
                yield PiscesLxViolation(self.rule, path, e.lineno, f"__all__ names {e.value!r}, which is not defined here")


class PiscesLxEngineIsolationCheck(PiscesLxStandardCheck):
    """Layering: the kernel / op layer must not import the engine, serving or tool layers."""
    rule = "engine-isolation"
    LOWER, UPPER = ("ops",), ("engine", "serve", "tools", "data")

    def check(self, path, source, tree):
        parts = path.replace("\\", "/").split("/")
        if "pisceslx_b200" not in parts:
            return
        layer = parts[parts.index("pisceslx_b200") + 1] if parts.index("pisceslx_b200") + 1 < len(parts) else ""
        if layer not in self.LOWER:
            return
        for node in ast.walk(tree):
            mod = node.module if isinstance(node, ast.ImportFrom) else None
            if mod and any(f"pisceslx_b200.{u}" in mod or (node.level >= 2 and mod.split(".")[0] == u) for u in self.UPPER):
                yield PiscesLxViolation(self.rule, path, node.lineno, f"{layer} layer imports {mod}")


class PiscesLxConfigSchemaCollector:
    """Field names of a dataclass-style config class (annotated assignments in the class body)."""

    @staticmethod
    def fields(tree: ast.AST, class_name: str) -> Set[str]:
        for node in ast.walk(tree):
            if isinstance(node, ast.ClassDef) and node.name == class_name:
                return {n.target.id for n in node.body if isinstance(n, ast.AnnAssign) and isinstance(n.target, ast.Name)}
        return set()


class PiscesLxUndeclaredConfigReadCheck(PiscesLxStandardCheck):
    """``cfg.<name>`` reads of names that the config class does not declare (typos fall through ``getattr`` defaults
    silently otherwise).  Only plain ``cfg.x`` / ``self.cfg.x`` attribute reads are considered."""
    rule = "undeclared-config-read"

    def __init__(self, declared: Set[str], allow: Iterable[str] = ()):
        self.declared, self.allow = set(declared), set(allow)

    def check(self, path, source, tree):
        for node in ast.walk(tree):
            if isinstance(node, ast.Attribute) and isinstance(node.ctx, ast.Load):
                v = node.value
                is_cfg = (isinstance(v, ast.Name) and v.id == "cfg") or \
                         (isinstance(v, ast.Attribute) and v.attr == "cfg" and isinstance(v.value, ast.Name) and v.value.id == "self")
                if is_cfg and not node.attr.startswith("_") and node.attr not in self.declared and node.attr not in self.allow:
                    yield PiscesLxViolation(self.rule, path, node.lineno, f"cfg.{node.attr} is not a declared config field")


class PiscesLxDeadConfigFieldCheck:
    """Config fields that no source file reads (by attribute name anywhere in the tree)."""
    rule = "dead-config-field"

    def __init__(self, declared: Set[str]):
        self.declared = set(declared)

    def run(self, files: Iterable[PiscesLxSourceFile]) -> List[str]:
        used: Set[str] = set()
        for f in files:
            for node in ast.walk(f.tree):
                if isinstance(node, ast.Attribute):
                    used.add(node.attr)
                elif isinstance(node, ast.Constant) and isinstance(node.value, str):
                    used.add(node.value)
        return sorted(self.declared - used)


class PiscesLxImportCensus:
    """Counts third-party top-level imports per package over the tree (what the project really depends on)."""

    def run(self, files: Iterable[PiscesLxSourceFile], own: str = "pisceslx_b200") -> Dict[str, int]:
        import sys
        std = set(getattr(sys, "stdlib_module_names", ()))
        counts: Dict[str, int] = {}
        for f in files:
            for node in ast.walk(f.tree):
                names = []
                if isinstance(node, ast.Import):
                    names = [a.name.split(".")[0] for a in node.names]
                elif isinstance(node, ast.ImportFrom) and node.level == 0 and node.module:
                    names = [node.module.split(".")[0]]
                for n in names:
                    if n not in std and n != own and n != "__future__":
                        counts[n] = counts.get(n, 0) + 1
        return dict(sorted(counts.items(), key=lambda kv: -kv[1]))


@dataclass
class PiscesLxCheckReport:
    violations: List[PiscesLxViolation] = field(default_factory=list)
    files: int = 0

    def by_rule(self) -> Dict[str, int]:
        out: Dict[str, int] = {}
        for v in self.violations:
            out[v.rule] = out.get(v.rule, 0) + 1
        return out

    def to_json(self) -> str:
        return json.dumps({"files": self.files, "by_rule": self.by_rule(),
                           "violations": [v.__dict__ for v in self.violations]}, indent=1)

    def ok(self, fail_on: Sequence[str] = ()) -> bool:
        rules = self.by_rule()
        return not any(r in rules for r in fail_on) if fail_on else not self.violations


class PiscesLxCheckSuite:
    """Runs a list of rule objects over a scanned tree."""

    def __init__(self, checks: Sequence[PiscesLxStandardCheck]):
        self.checks = list(checks)

    def run(self, root: str) -> PiscesLxCheckReport:
        rep = PiscesLxCheckReport()
        for f in PiscesLxRepositoryScanner(root).files():
            rep.files += 1
            for c in self.checks:
                rep.violations.extend(c.check(f.path, f.source, f.tree))
        return rep


class PiscesLxCheckCatalog:
    @staticmethod
    def default() -> List[PiscesLxStandardCheck]:
        return [PiscesLxHardcodingCheck(), PiscesLxIncompleteMarkerCheck(), PiscesLxDanglingExportCheck(), PiscesLxEngineIsolationCheck()]


class PiscesLxCheckCli:
    def run(self, argv: List[str]) -> int:
        root = argv[0] if argv else "."
        rep = PiscesLxCheckSuite(PiscesLxCheckCatalog.default()).run(root)
        print(rep.to_json() if "--json" in argv else f"{rep.files} files, {len(rep.violations)} violations: {rep.by_rule()}")
        return 0 if rep.ok() else 1
