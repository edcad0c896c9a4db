"""CPU: the C-ABI library loads, exports every function the header declares, and the host-side
argument checks that need no GPU behave like the reference's TORCH_CHECKs."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    src = open(os.path.join(ROOT, "include", "triteia_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(trb_\w+)\s*\(", src)))


def test_header_and_binding_list_the_same_functions():
    from triteia_b200 import _lib

    assert declared_functions() == sorted(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol():
    from triteia_b200 import _lib

    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), name


def test_host_only_entry_points():
    from triteia_b200._lib import lib, status_string

    assert lib.trb_version() >= 100
    assert lib.trb_sgmv_tmp_size(16) == 16 * 60  # same rule as the reference (sgmv.cuh:48-52)
    assert lib.trb_route_max_tiles(128, 64, 8) == 128 // 8 + 64
    assert lib.trb_sbmm_indexed_scratch_bytes(128, 4096, 64) >= 128 * 4096 * 2
    assert "shape" in status_string(1) and status_string(0) == "ok"


def test_cpu_tensors_are_rejected_not_computed():
    from triteia_b200.capi import mul_2_4
    from triteia_b200.ops import matmul_4bit_2_4, gen_sparse_quant4_NT

    torch.manual_seed(0)
    _, q, s, meta = gen_sparse_quant4_NT(256, 128, device="cpu")
    x = torch.randn(4, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA"):
        matmul_4bit_2_4(q, x, meta, s)
    with pytest.raises(RuntimeError, match="CUDA"):
        mul_2_4(x, q, meta, torch.empty(4, 256, dtype=torch.float16), s, torch.zeros(32, dtype=torch.int32))


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    import importlib
    from triteia_b200 import _lib

    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU"):
        _lib._load()
    importlib.reload(_lib)
