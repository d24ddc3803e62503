"""CPU checks of the drop-in boundary: the shared library loads and exports
every symbol include/mk_cuda.h declares, and refuses to run without a GPU."""
import os
import re

import pytest

from conftest import ROOT


def _declared():
    src = open(os.path.join(ROOT, "include", "mk_cuda.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(mk_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_are_exported_and_bound():
    from microkimi_b200 import lib
    L = lib.load()
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(L, n), f"{n} declared in mk_cuda.h but not exported"
        assert n in lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(lib.SIGNATURES) == names


def test_reference_side_binding_lists_every_entry_point():
    """The `src/cuda.rs` block a maintainer of the engine would add declares every function of the header."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    missing = [n for n in _declared() if not re.search(r"\bfn %s\(" % n, text)]
    assert not missing, missing


def test_no_cpu_fallback_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import microkimi_b200 as mk
    with pytest.raises(mk.lib.MkError):
        mk.Context(0)


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "microkimi_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"
