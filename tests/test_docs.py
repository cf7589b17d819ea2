"""The commands and paths the documentation names exist: modules given to ``python -m`` import and have an entry point, script
and source paths are files of this tree, spec keys used in examples are keys of the spec."""
import importlib
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = ["README.md", "DESIGN.md"]


def _text(name):
    with open(os.path.join(ROOT, name), encoding="utf-8") as fh:
        return fh.read()


@pytest.mark.parametrize("doc", DOCS)
def test_modules_named_in_commands_exist(doc):
    mods = set(re.findall(r"python -m (parameter_golf_b200(?:\.[a-z_]+)+)", _text(doc)))
    assert mods, doc
    for mod in sorted(mods):
        m = importlib.import_module(mod)
        assert any(hasattr(m, f) for f in ("main", "_main")), f"{doc}: {mod} has no command-line entry"


@pytest.mark.parametrize("doc", DOCS)
def test_paths_named_in_the_docs_exist(doc):
    text = _text(doc)
    paths = set(re.findall(r"`((?:bench|tests|specs|profiles|parameter_golf_b200)/[A-Za-z0-9_./-]+\.(?:py|cu|cuh|cpp|h|inc|toml|json|md|sh))`", text))
    paths |= {"parameter_golf_b200/" + p for p in re.findall(r"`((?:csrc|models|ops|parallel|quant|eval|data|optim|utils)/[A-Za-z0-9_]+\.(?:py|cu|cuh|cpp|h|inc))`", text)}
    assert len(paths) > 10, doc
    missing = sorted(p for p in paths if not os.path.exists(os.path.join(ROOT, p)))
    assert not missing, f"{doc} names files that do not exist: {missing}"


def test_spec_keys_used_in_the_docs_are_real_keys():
    from parameter_golf_b200.spec import RunSpec
    keys = {k for k, _, _ in RunSpec().describe_keys()}
    sections = ("model.", "train.", "quant.", "eval.")
    used = set()
    for doc in DOCS:
        for k in re.findall(r"`((?:model|train|quant|eval)\.[a-z_][a-z0-9_.]*)", _text(doc)):
            used.add(k.rstrip("."))
    assert len(used) > 40
    unknown = sorted(k for k in used if k not in keys and not any(x.startswith(k + ".") for x in keys) and not k.endswith(("_", ".py")))
    # prefixes written with a trailing wildcard in prose (train.lawa_*, train.swa_*, eval.doc_*) name families of keys
    unknown = [k for k in unknown if not any(x.startswith(k) for x in keys)]
    assert not unknown, unknown
