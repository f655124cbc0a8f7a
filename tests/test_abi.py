"""CPU tests of the drop-in boundary: the library loads and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "nanoserve_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:ns|b2)_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_reference_symbols():
    syms = _declared_symbols()
    # the six names the reference's binding resolves (python/nanoserve/ops.py:19-26)
    for name in ("ns_rmsnorm", "ns_rope", "ns_swiglu", "ns_flash_fwd", "ns_w4_quantize", "ns_w4_linear"):
        assert name in syms


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(lib_path)
    missing = [s for s in _declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_binding_signatures_cover_the_header(lib_path):
    from nanoserve_b200 import ops
    assert sorted(ops.SIGNATURES) == _declared_symbols()
    lib = ops.load_library(lib_path)
    assert lib.b2_version().decode().startswith("nanoserve-b200")


def test_missing_library_fails_loudly(tmp_path):
    from nanoserve_b200 import ops
    with pytest.raises(FileNotFoundError):
        ops.Kernels(str(tmp_path / "libnanoserve.so"))


def test_no_cpu_path():
    import torch
    from nanoserve_b200 import ops
    with pytest.raises(RuntimeError):
        ops.Kernels._cuda(torch.zeros(1))
