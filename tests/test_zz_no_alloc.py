"""GPU: the scratch-free entry point trb_sbmm_indexed_static against trb_sbmm_indexed.

Some hosts of the library cannot allocate device memory for it (their own arena owns all of HBM,
or their plugin contract bans cudaMalloc after start-up).  For them the working memory of the
fused indexed delta matmul is a fixed array inside the library; this test calls that entry point
through the C ABI twice in a row, with different batches, and compares each result with the
caller-allocated entry point on the same inputs.  The file name sorts last on purpose.
"""
import numpy as np
import pytest
import torch

from oracle import ops as oracle

pytestmark = pytest.mark.gpu


def _run_both(L, qs, metas, ss, x, idx, groupsize):
    T, K = x.shape
    D, _, N = ss.shape
    dev = x.device
    y_ref = torch.full((T, N), 7.0, dtype=torch.float16, device=dev)
    y_new = torch.full((T, N), 7.0, dtype=torch.float16, device=dev)
    nbytes = L.lib.trb_sbmm_indexed_scratch_bytes(T, K, D)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    L.check(L.lib.trb_sbmm_indexed(L.ptr(x), L.ptr(qs), L.ptr(metas), L.ptr(ss), L.ptr(idx), L.ptr(y_ref), T, N, K, D, 0,
                                   groupsize, 0, L.ptr(scratch), nbytes, 0, L.stream_of(x)), "sbmm_indexed")
    L.check(L.lib.trb_sbmm_indexed_static(L.ptr(x), L.ptr(qs), L.ptr(metas), L.ptr(ss), L.ptr(idx), L.ptr(y_new), T, N, K,
                                          D, 0, groupsize, 0, 0, L.stream_of(x)), "sbmm_indexed_static")
    torch.cuda.synchronize()
    return y_ref, y_new


def test_static_scratch_entry_point_matches_twice(cuda):
    from triteia_b200 import _lib as L
    import triteia_b200.ops as ops

    K, N, D, groupsize = 512, 256, 6, 128
    qs, metas, ss = ops.random_packed_deltas(D, K, N, groupsize=groupsize, device=cuda, seed=3, scale_lo=0.005,
                                             scale_hi=0.02)
    for call, T in enumerate([48, 21]):          # second call: smaller batch over the first call's leftovers
        g = torch.Generator(cuda).manual_seed(100 + call)
        x = torch.randn(T, K, dtype=torch.float16, device=cuda, generator=g)
        idx = torch.from_numpy(np.random.default_rng(call).integers(-1, D, T).astype(np.int32)).to(cuda)
        y_ref, y_new = _run_both(L, qs, metas, ss, x, idx, groupsize)
        err = oracle.row_rel_err(y_new.float().cpu().numpy(), y_ref.float().cpu().numpy())
        assert err.max() <= 1e-2, f"call {call}: row rel err {err.max()}"
        assert torch.all(y_new[idx == -1] == 0)
        ref = oracle.sbmm(qs.cpu().numpy(), x.cpu().numpy(), metas.cpu().numpy(), ss.cpu().numpy(), idx.cpu().numpy())
        assert oracle.row_rel_err(y_new.float().cpu().numpy(), ref).max() <= 1e-2
    assert L.device_status(0) == 0


def test_static_scratch_rejects_oversize(cuda):
    from triteia_b200 import _lib as L

    cap = L.lib.trb_sbmm_indexed_static_capacity()
    assert cap == 4 * 1024 * 1024 + 64 * 1024
    assert L.lib.trb_sbmm_indexed_scratch_bytes(4096, 8192, 64) > cap
    one = torch.zeros(16, dtype=torch.uint8, device=cuda)
    rc = L.lib.trb_sbmm_indexed_static(L.ptr(one), L.ptr(one), L.ptr(one), L.ptr(one), L.ptr(one), L.ptr(one), 4096, 4096,
                                       8192, 64, 0, 128, 0, 0, L.stream_of(one))
    assert rc == L.ERR_SCRATCH
    assert "scratch" in L.status_string(rc)
