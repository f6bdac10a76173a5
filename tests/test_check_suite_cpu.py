"""CPU tests of the static check suite: every rule on a small synthetic tree, then the suite on the package itself."""
from __future__ import annotations

import ast
import os

from pisceslx_b200.utils import check_suite as C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(check, src, path="pkg/mod.py"):
    return list(check.check(path, src, ast.parse(src)))


def test_individual_rules():
    v = _run(C.PiscesLxHardcodingCheck(), 'p = "/home/alice/data"\nh = "10.1.2.3"\nk = "api_key=abcdef0123456789"\nok = "/tmp/x"\n')
    assert [x.line for x in v] == [1, 2, 3]
    assert len(_run(C.PiscesLxIncompleteMarkerCheck(), "x = 1  # TODO later\ny = 2  # todo lower case is prose\n")) == 1
    src = 'def public(a):\n    a += 1\n    a += 2\n    a += 3\n    return a\n\ndef _private(a):\n    a += 1\n    a += 2\n    a += 3\n    return a\n\ndef documented(a):\n    """doc"""\n    return a\n'
    assert [x.message for x in _run(C.PiscesLxTopLevelFunctionCheck(), src)] == ["public function public has no docstring"]
    assert _run(C.PiscesLxTopLevelFunctionCheck(), src, "tests/test_x.py") == []
    v = _run(C.PiscesLxDanglingExportCheck(), '__all__ = ["a", "b", "c"]\nfrom m import a\ndef b():\n    pass\n')
    assert len(v) == 1 and "'c'" in v[0].message
    iso = C.PiscesLxEngineIsolationCheck()
    assert len(_run(iso, "from pisceslx_b200.engine.trainer import YvTrainer\n", "x/pisceslx_b200/ops/f.py")) == 1
    assert len(_run(iso, "from ..serve import engine\n", "x/pisceslx_b200/ops/f.py")) == 1
    assert _run(iso, "from pisceslx_b200.engine.trainer import YvTrainer\n", "x/pisceslx_b200/serve/f.py") == []
    tree = ast.parse("class Cfg:\n    hidden: int = 1\n    layers: int = 2\n    unused_field: int = 3\n")
    declared = C.PiscesLxConfigSchemaCollector.fields(tree, "Cfg")
    assert declared == {"hidden", "layers", "unused_field"}
    v = _run(C.PiscesLxUndeclaredConfigReadCheck(declared), "def f(cfg, self):\n    return cfg.hidden + cfg.hiden + self.cfg.layers + self.cfg.depth\n")
    assert sorted(x.message for x in v) == ["cfg.depth is not a declared config field", "cfg.hiden is not a declared config field"]
    user = C.PiscesLxSourceFile("u.py", "", ast.parse("def f(cfg):\n    return cfg.hidden * cfg.layers\n"))
    assert C.PiscesLxDeadConfigFieldCheck(declared).run([user]) == ["unused_field"]


def test_scanner_census_suite_and_cli_on_a_synthetic_tree(tmp_path, capsys):
    (tmp_path / "pkg").mkdir()
    (tmp_path / "pkg" / "__pycache__").mkdir()
    (tmp_path / "pkg" / "a.py").write_text("import numpy as np\nimport os\nfrom torch import nn\nimport torch\nx = 1  # FIXME\n")
    (tmp_path / "pkg" / "b.py").write_text('__all__ = ["missing"]\nimport torch\n')
    (tmp_path / "pkg" / "broken.py").write_text("def (:\n")
    (tmp_path / "pkg" / "__pycache__" / "c.py").write_text("import shouldnotbeseen\n")
    files = list(C.PiscesLxRepositoryScanner(str(tmp_path)).files())
    assert sorted(os.path.basename(f.path) for f in files) == ["a.py", "b.py"]
    assert C.PiscesLxImportCensus().run(files) == {"torch": 3, "numpy": 1}
    rep = C.PiscesLxCheckSuite(C.PiscesLxCheckCatalog.default()).run(str(tmp_path))
    assert rep.files == 2 and rep.by_rule() == {"incomplete-marker": 1, "dangling-export": 1}
    assert not rep.ok() and rep.ok(fail_on=["hardcoding"]) and '"files": 2' in rep.to_json()
    assert C.PiscesLxCheckCli().run([str(tmp_path)]) == 1
    assert "2 files, 2 violations" in capsys.readouterr().out


def test_package_passes_its_own_layering_export_and_hardcoding_rules():
    rep = C.PiscesLxCheckSuite([C.PiscesLxEngineIsolationCheck(), C.PiscesLxDanglingExportCheck(), C.PiscesLxHardcodingCheck()]
                               ).run(os.path.join(ROOT, "pisceslx_b200"))
    assert rep.files > 80 and rep.violations == [], [f"{v.path}:{v.line} {v.message}" for v in rep.violations[:10]]
