"""The C-ABI library builds, loads and exports every symbol include/fmb200.h declares (no compute calls)."""
import os
import re

from conftest import ROOT


def test_library_exports_every_declared_symbol():
    from fastmace_b200 import _lib, build
    build.build()
    lib = _lib.load()
    header = open(os.path.join(ROOT, "include", "fmb200.h")).read()
    declared = set(re.findall(r"FMB_API\s+[\w\s\*]+?\b(fmb_\w+)\s*\(", header))
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.fmb_version() >= 100


def test_no_cpu_fallback():
    import pytest
    import torch
    from fastmace_b200 import _lib
    from fastmace_b200.model import SMALL, init_weights
    from fastmace_b200.structures import nacl
    if torch.cuda.is_available():
        pytest.skip("checks the refusal on a CPU-only host")
    from fastmace_b200.forcefield import B200ForceField
    s = nacl((1, 1, 1), 0.0, 0)
    with pytest.raises(_lib.Fmb200Error):
        B200ForceField(SMALL, init_weights(SMALL, 0), s.numbers, s.cell)
