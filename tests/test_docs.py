"""The list of environment variables in docs/environment.md stays in step with the parser."""
import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parent.parent


def test_every_parsed_variable_is_documented():
    doc = (ROOT / "docs" / "environment.md").read_text()
    parsed = set(re.findall(r'"(CCL_[A-Z0-9_]+)"', (ROOT / "csrc" / "core" / "env.cpp").read_text()))
    assert len(parsed) > 80
    missing = sorted(n for n in parsed if n not in doc)
    assert not missing, f"not documented: {missing}"


def test_documented_variables_exist_in_the_sources():
    doc = (ROOT / "docs" / "environment.md").read_text()
    names = set(re.findall(r"`(CCL_[A-Z0-9_]+)`", doc))
    sources = ""
    for pat in ("csrc/**/*.cpp", "csrc/**/*.cu", "csrc/**/*.hpp", "oneccl_b200/**/*.py"):
        for f in ROOT.glob(pat):
            sources += f.read_text(errors="ignore")
    # families written with a placeholder or composed at run time (CCL_<COLL>, CCL_CUDA_<COLL>, ..._SCALEOUT)
    unknown = sorted(n for n in names if n not in sources and not n.endswith("_"))
    assert not unknown, f"documented but not read anywhere: {unknown}"
