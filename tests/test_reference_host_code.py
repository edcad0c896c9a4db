"""GPU: the reference's own Python host code running over this library.

The drop-in claim is that the reference's `triteia.python.ops` works unchanged when the module it
imports as `triteia_cuda` is this package's shim.  This test does exactly that: it needs a checkout
of the reference (environment variable TRITEIA_REFERENCE = its root directory) AND a CUDA device; it
is skipped when either is missing.  The reference's contract applies to its functions: per-channel
scales, indices grouped by delta with the -1 run first.
"""
import os
import sys
import types

import numpy as np
import pytest
import torch

from oracle import ops as oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_ops(cuda):
    root = os.environ.get("TRITEIA_REFERENCE", "")
    if not root or not os.path.isdir(os.path.join(root, "triteia", "python", "ops")):
        pytest.skip("no reference checkout (set TRITEIA_REFERENCE)")
    from triteia_b200 import triteia_cuda as shim

    saved = {k: sys.modules.get(k) for k in ("triteia_cuda", "pynvml")}
    sys.modules["triteia_cuda"] = shim
    try:
        import pynvml
        pynvml.nvmlInit()
    except Exception:                        # no NVML here: the reference only reads the GPU's name from it
        nv = types.ModuleType("pynvml")
        nv.nvmlInit = lambda: None
        nv.nvmlDeviceGetHandleByIndex = lambda i: None
        nv.nvmlDeviceGetName = lambda h: "NVIDIA B200"
        sys.modules["pynvml"] = nv
    sys.path.insert(0, root)
    try:
        import triteia.python.ops as ops
        yield ops
    finally:
        sys.path.remove(root)
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
        for k in [k for k in sys.modules if k == "triteia" or k.startswith("triteia.")]:
            sys.modules.pop(k)


def _np(t):
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def test_reference_sbmm_native_over_the_shim(ref_ops, cuda):
    import triteia_b200.ops as ours
    qs, metas, ss = ours.random_packed_deltas(5, 256, 512, groupsize=-1, device=cuda, seed=1, scale_lo=0.005, scale_hi=0.02)
    x = torch.randn(40, 256, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(1))
    idx = torch.from_numpy(np.sort(np.random.default_rng(1).integers(-1, 5, 40)).astype(np.int32)).to(cuda)
    y = ref_ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx)
    ref = oracle.sbmm(_np(qs), _np(x), _np(metas), _np(ss), _np(idx))
    assert oracle.row_rel_err(_np(y), ref).max() <= 1e-2
    y2 = ref_ops.sbmm_4bit_2_4_forloop(qs, x, metas, ss, idx)
    assert oracle.row_rel_err(_np(y2), ref).max() <= 1e-2


def test_reference_ldmm_and_sgmv_over_the_shim(ref_ops, cuda):
    import triteia_b200.ops as ours
    M, D, K, N, r, T = 3, 3, 768, 768, 16, 48
    qs, metas, ss = ours.random_packed_deltas(D, K, N, groupsize=-1, device=cuda, seed=2, scale_lo=0.005, scale_hi=0.02)
    g = torch.Generator(cuda).manual_seed(2)
    A = (torch.randn(M, K, r, device=cuda, generator=g) / K ** 0.5).half()
    B = (torch.randn(M, r, N, device=cuda, generator=g) / r ** 0.5).half()
    x = torch.randn(T, K, device=cuda, generator=g).half()
    idx = torch.from_numpy(np.sort(np.random.default_rng(2).integers(-1, M + D, T)).astype(np.int32)).to(cuda)
    y = ref_ops.ldmm(idx, x, A, B, qs, metas, ss)
    ref = oracle.ldmm(_np(idx), _np(x), _np(A), _np(B), _np(qs), _np(metas), _np(ss))
    assert oracle.row_rel_err(_np(y), ref).max() <= 1e-2
    lidx = torch.from_numpy(np.sort(np.random.default_rng(3).integers(-1, M, T)).astype(np.int32)).to(cuda)
    y = ref_ops.lora_sgmv(A, B, x, lidx)
    ref = oracle.lora(_np(A), _np(B), _np(x), _np(lidx))
    assert oracle.row_rel_err(_np(y), ref).max() <= 1e-2
