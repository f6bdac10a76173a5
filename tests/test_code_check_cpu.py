"""Source checks and the staged self-test."""
import ast
import json
from pathlib import Path

from pisceslx_b200.tools.code_check import (PiscesLxAbsolutePathCheck, PiscesLxAstWalker, PiscesLxCheckRunner, PiscesLxCopyrightHeaderCheck, PiscesLxImportCensusCli,
                                            PiscesLxModalityCheck, PiscesLxProjectNameCheck, PiscesLxRegexLibrary, PiscesLxResidualSystemCheck, PiscesLxRuleId,
                                            PiscesLxStandardHeader, PiscesLxTestCli, PiscesLxTestRunner, PiscesLxTestStatus, _StageChecker)


def _tree(tmp_path):
    (tmp_path / "pkg").mkdir()
    (tmp_path / "pkg" / "good.py").write_text('"""Licensed under Apache. A good module."""\nimport os\nimport numpy\n\nclass PiscesLxThing:\n    pass\n')
    (tmp_path / "pkg" / "bad.py").write_text('import old_system.api\nimport numpy as np\nP = "/home/someone/data"\n\nclass Loose:\n    class Inner: pass\n\ndef f(modality):\n    return modality == "image"\n# TODO remove\n')
    (tmp_path / "pkg" / "broken.py").write_text("def (:\n")
    (tmp_path / "pkg" / "__pycache__").mkdir()
    (tmp_path / "pkg" / "__pycache__" / "x.py").write_text("zzz(")
    return tmp_path


def test_checks_and_report(tmp_path):
    root = _tree(tmp_path)
    checks = [PiscesLxCopyrightHeaderCheck(PiscesLxStandardHeader(["licensed under apache"])), PiscesLxProjectNameCheck(), PiscesLxAbsolutePathCheck(), PiscesLxModalityCheck(),
              PiscesLxResidualSystemCheck({"old_system": "new_system"}, flag_markers=True)]
    rep = PiscesLxCheckRunner(root, checks).run()
    by = rep.by_rule()
    assert rep.files_scanned == 3 and by[PiscesLxRuleId.SYNTAX] == 1 and by[PiscesLxRuleId.HEADER] == 1 and by[PiscesLxRuleId.PROJECT_NAME] == 1
    assert by[PiscesLxRuleId.ABSOLUTE_PATH] == 1 and by[PiscesLxRuleId.MODALITY] == 1 and by[PiscesLxRuleId.RESIDUAL] == 2 and rep.exit_code == 1
    assert all("good.py" not in v.render(root) for v in rep.violations) and len(rep.warnings) == 2
    text = rep.render()
    assert "pkg/bad.py:3: [error] hygiene.absolute_path" in text and "use new_system" in text and rep.render(verbose=False).count("\n") < text.count("\n")
    assert PiscesLxCheckRunner(root).run([root / "pkg" / "good.py"]).exit_code == 0 and set(PiscesLxRuleId.all_rules()) >= set(by)


def test_header_walker_regex_census(tmp_path):
    h = PiscesLxStandardHeader()
    assert h.extract_leading_block("#!/usr/bin/env python\n# Copyright X\n#  All rights\n\nimport os\n").startswith("# Copyright") and h.missing("import os\n") and not h.missing("# hi\nimport os")
    assert PiscesLxStandardHeader.normalize("#  A\n#   B") == "a b"
    t = ast.parse("class A:\n    class B:\n        def m(self): pass\ndef g(): pass\nif __name__ == '__main__':\n    x = 1\n")
    assert [c.name for c in PiscesLxAstWalker.iter_classes(t)] == ["A", "B"] and len(list(PiscesLxAstWalker.iter_functions(t))) == 2
    par = PiscesLxAstWalker.parents(t)
    m = next(n for n in ast.walk(t) if isinstance(n, ast.FunctionDef) and n.name == "m")
    g = next(n for n in ast.walk(t) if isinstance(n, ast.FunctionDef) and n.name == "g")
    x = next(n for n in ast.walk(t) if isinstance(n, ast.Assign))
    assert PiscesLxAstWalker.is_inside_class(m, par) and not PiscesLxAstWalker.is_inside_class(g, par)
    assert PiscesLxAstWalker.is_inside_main_guard(x, par) and not PiscesLxAstWalker.is_inside_main_guard(g, par) and PiscesLxAstWalker.enclosing_classes(t)[m] == ("A", "B")
    assert PiscesLxRegexLibrary.matches_any('p = "/Users/me/x"', PiscesLxRegexLibrary.absolute_path_patterns()) and not PiscesLxRegexLibrary.matches_any('p = "data/x"', PiscesLxRegexLibrary.absolute_path_patterns())
    root = _tree(tmp_path)
    cli = PiscesLxImportCensusCli(root, own=("pkg",))
    c = cli.census()
    assert c["imports"]["numpy"] == 2 and "numpy" in c["third_party"] and "os" in c["stdlib"] and "old_system" in c["third_party"]
    lines = []
    assert cli.run(["--json"], lines.append) == 0 and json.loads(lines[0])["files"] == 3


def test_staged_selftest_runs_and_skips_dependants(tmp_path):
    rep = PiscesLxTestRunner().run()
    assert rep.ok and rep.count(PiscesLxTestStatus.PASSED) == 9, rep.render()
    opt = next(r for r in rep.results if r.name == "optimization")
    assert opt.details["last"] < opt.details["first"]

    class Boom(_StageChecker):
        name = "model"
        requires = ()

        def check(self, ctx):
            raise ValueError("no weights")

    class After(_StageChecker):
        name, requires = "forward", ("model",)

        def check(self, ctx):
            raise AssertionError("must not run")

    class After2(After):
        name, requires = "generation", ("forward",)

    r2 = PiscesLxTestRunner([Boom(), After(), After2()]).run()
    assert [r.status for r in r2.results] == [PiscesLxTestStatus.FAILED, PiscesLxTestStatus.SKIPPED, PiscesLxTestStatus.SKIPPED] and not r2.ok and "no weights" in r2.render()
    out = []
    assert PiscesLxTestCli().run(["--stage", "environment", "--json", str(tmp_path / "r.json")], out.append) == 0
    assert json.loads(Path(tmp_path / "r.json").read_text())["ok"] and "PASSED" in out[0]
