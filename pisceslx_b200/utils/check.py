"""Static conformance checks (reference ``python -m tools.check``, tools/check/*): AST / regex rules over the source
tree - class naming, no stdlib ``logging`` in engine code, no silent ``except: pass``, no detached scalars fed to
``backward``, dangling intra-package imports, and this repository's own rule that comments never point at build
documents."""
from __future__ import annotations

import ast
import os
import re
from dataclasses import dataclass
from typing import Callable, Dict, Iterator, List


@dataclass
class PiscesLxViolation:
    rule: str
    path: str
    line: int
    message: str


class PiscesLxStandardCheck:
    rule = "base"

    def check(self, path: str, source: str, tree: ast.AST) -> Iterator[PiscesLxViolation]:
        return iter(())


class PiscesLxSilentExceptCheck(PiscesLxStandardCheck):
    rule = "silent-except"

    def check(self, path, source, tree):
        for node in ast.walk(tree):
            if isinstance(node, ast.ExceptHandler) and node.type is None:
                if all(isinstance(s, ast.Pass) for s in node.body):
                    yield PiscesLxViolation(self.rule, path, node.lineno, "bare 'except: pass' hides failures")


class PiscesLxStdlibLoggingCheck(PiscesLxStandardCheck):
    rule = "stdlib-logging"

    def check(self, path, source, tree):
        for node in ast.walk(tree):
            if isinstance(node, ast.Import) and any(a.name == "logging" for a in node.names):
                yield PiscesLxViolation(self.rule, path, node.lineno, "use PiscesLxLogger instead of stdlib logging")


class PiscesLxClassNamingCheck(PiscesLxStandardCheck):
    rule = "class-naming"
    ok = re.compile(r"^(_?Yv|_?PiscesLx|_[A-Z]|[A-Z][A-Za-z0-9]+(Error|Fn|Config|Sampler|Dataset|Stage|Buffer|Heap|Plan|Context|State|Request)$)")

    def check(self, path, source, tree):
        for node in ast.walk(tree):
            if isinstance(node, ast.ClassDef) and not self.ok.match(node.name):
                yield PiscesLxViolation(self.rule, path, node.lineno, f"class {node.name} lacks the Yv / PiscesLx prefix")


class PiscesLxDetachedScalarCheck(PiscesLxStandardCheck):
    rule = "detached-scalar"

    def check(self, path, source, tree):
        for node in ast.walk(tree):
            if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr == "backward":
                v = node.func.value
                if isinstance(v, ast.Call) and isinstance(v.func, ast.Attribute) and v.func.attr in ("item", "detach"):
                    yield PiscesLxViolation(self.rule, path, node.lineno, "backward() on a detached value")


class PiscesLxBuildDocReferenceCheck(PiscesLxStandardCheck):
    rule = "build-doc-reference"
    # any all-capitals markdown file of the repository root other than the README (planning and review documents)
    pat = re.compile(r"\b(?!README\b)[A-Z]{5,}\.md\b")

    def check(self, path, source, tree):
        for i, line in enumerate(source.splitlines(), 1):
            if self.pat.search(line):
                yield PiscesLxViolation(self.rule, path, i, "source must not point at build documents")


class PiscesLxDanglingImportCheck(PiscesLxStandardCheck):
    rule = "dangling-import"

    def __init__(self, root: str):
        self.root = root

    def check(self, path, source, tree):
        for node in ast.walk(tree):
            if isinstance(node, ast.ImportFrom) and node.module and node.level == 0 and node.module.startswith("pisceslx_b200"):
                rel = node.module.replace(".", os.sep)
                base = os.path.join(self.root, rel)
                if not (os.path.isdir(base) or os.path.exists(base + ".py")):
                    yield PiscesLxViolation(self.rule, path, node.lineno, f"module {node.module} does not exist")


def run_checks(root: str, verbose: bool = True) -> int:
    checks: List[PiscesLxStandardCheck] = [PiscesLxSilentExceptCheck(), PiscesLxStdlibLoggingCheck(),
                                           PiscesLxDetachedScalarCheck(), PiscesLxBuildDocReferenceCheck(),
                                           PiscesLxDanglingImportCheck(root)]
    violations: List[PiscesLxViolation] = []
    for base in ("pisceslx_b200", "tests"):
        for dirpath, _, files in os.walk(os.path.join(root, base)):
            for f in files:
                if not f.endswith(".py"):
                    continue
                path = os.path.join(dirpath, f)
                src = open(path).read()
                if os.path.basename(path) == "check.py":
                    continue
                try:
                    tree = ast.parse(src)
                except SyntaxError as e:
                    violations.append(PiscesLxViolation("syntax", path, e.lineno or 0, str(e)))
                    continue
                for c in checks:
                    violations.extend(c.check(os.path.relpath(path, root), src, tree))
    if verbose:
        for v in violations:
            print(f"{v.path}:{v.line}: [{v.rule}] {v.message}")
        print(f"{len(violations)} violation(s)")
    return 1 if violations else 0
