"""The C-ABI library builds, loads and exports every symbol that include/ptxfe.h declares; without a GPU its entry
points fail loudly instead of falling back to a CPU path."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "ptxfe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ptxfe_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import zluda_b200
    lib = zluda_b200.lib()
    names = declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n


def test_no_cpu_fallback_without_a_device():
    import torch
    import zluda_b200
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(zluda_b200.PtxfeError):
        zluda_b200.Context(0)
    with pytest.raises(zluda_b200.PtxfeError):
        zluda_b200.parse_module_checked(".version 7.8\n.target sm_80\n")


def test_product_does_not_reference_the_oracle():
    for d, _, files in os.walk(os.path.join(ROOT, "zluda_b200")):
        for f in files:
            if f.endswith((".py", ".h", ".cu", ".cpp", ".inc")):
                s = open(os.path.join(d, f), errors="replace").read()
                assert "oracle/" not in s.replace("../oracle/gen", "").replace('"oracle", "gen"', "") or f in ("build.py", "gen_tables.py"), f
