"""GPU parity: every operator of the path, called through the C ABI (ctypes shims of
triteia_b200), against the CPU oracle on the same seeded inputs.

Bars: bit-exact for routing, tile work lists and weight / metadata unpacking; for fp16 outputs
max relative error per output row <= 1e-2 against the fp32 dequantise-then-matmul oracle
(max_n |y - ref| / max_n |ref|), plus the reference's own metric mean|y - ref| / mean|ref|
< 0.002 where its tests use it (tests/ops/test_matmul.py:18-22, tests/ops/test_sbmm.py:47-61).
"""
import zlib

import numpy as np
import pytest
import torch

from oracle import delta_format as fmt
from oracle import ops as oracle

pytestmark = pytest.mark.gpu

ROW_TOL = 1e-2
MEAN_TOL = 2e-3


def _ops():
    import triteia_b200.ops as ops
    return ops


def _lib():
    from triteia_b200 import _lib
    return _lib


def check(y, ref, mean_tol=MEAN_TOL):
    y = y.float().cpu().numpy()
    assert np.isfinite(y).all()
    err = oracle.row_rel_err(y, ref)
    assert err.max() <= ROW_TOL, f"row rel err {err.max():.4g} (row {err.argmax()})"
    if mean_tol is not None and np.abs(ref).mean() > 0:
        assert oracle.mean_rel_err(y, ref) < mean_tol


def packed(n_out, k_in, groupsize, seed, num=None, dev="cuda"):
    ops = _ops()
    qs, metas, ss = ops.random_packed_deltas(num or 1, k_in, n_out, groupsize=groupsize, device=dev, seed=seed,
                                              scale_lo=0.005, scale_hi=0.02)
    if num is None:
        return qs[0], metas[0], ss[0]
    return qs, metas, ss


# ------------------------------------------------------------------ unpack (bit-exact)
@pytest.mark.parametrize("name", ["pack_a", "pack_b", "pack_c"])
def test_unpack_golden_bit_exact(cuda, golden, name):
    L = _lib()
    q = torch.from_numpy(golden[f"{name}_q"]).to(cuda)
    meta = torch.from_numpy(golden[f"{name}_meta"]).to(cuda)
    s = torch.from_numpy(golden[f"{name}_s"]).to(cuda)
    k, n = q.shape[0] * 32, q.shape[1] // 2
    w = torch.empty(k, n, dtype=torch.float16, device=cuda)
    L.check(L.lib.trb_unpack_2_4(L.ptr(q), L.ptr(meta), L.ptr(s), L.ptr(w), n, k, -1, 0, L.stream_of(w)), "unpack")
    ref = fmt.dequantize(golden[f"{name}_q"], golden[f"{name}_meta"], golden[f"{name}_s"])
    assert np.array_equal(w.cpu().numpy().view(np.uint16), ref.view(np.uint16))
    assert np.array_equal(w.cpu().numpy(), golden[f"{name}_uncompress"])


@pytest.mark.parametrize("groupsize", [-1, 128])
def test_unpack_random_bit_exact(cuda, groupsize):
    L = _lib()
    q, meta, s = packed(512, 384, groupsize, seed=5)
    w = torch.empty(384, 512, dtype=torch.float16, device=cuda)
    L.check(L.lib.trb_unpack_2_4(L.ptr(q), L.ptr(meta), L.ptr(s), L.ptr(w), 512, 384, groupsize, 0, L.stream_of(w)),
            "unpack")
    ref = fmt.dequantize(q.cpu().numpy(), meta.cpu().numpy(), s.cpu().numpy())
    assert np.array_equal(w.cpu().numpy().view(np.uint16), ref.view(np.uint16))


# ------------------------------------------------------------------ single matmul
@pytest.mark.parametrize("groupsize", [-1, 128])
@pytest.mark.parametrize("tokens", [1, 3, 8, 9, 16, 17, 31, 33, 64, 65, 130])
def test_matmul_small(cuda, tokens, groupsize):
    ops = _ops()
    q, meta, s = packed(256, 384, groupsize, seed=tokens)
    x = torch.randn(tokens, 384, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(tokens))
    y = ops.matmul_4bit_2_4(q, x, meta, s)
    assert y.shape == (tokens, 256) and y.dtype == torch.float16
    check(y, oracle.matmul_2_4(q.cpu().numpy(), x.cpu().numpy(), meta.cpu().numpy(), s.cpu().numpy()))


@pytest.mark.parametrize("name", ["pack_a", "pack_b", "pack_c"])
def test_matmul_reference_packed_tensors(cuda, golden, name):
    """Tensors produced by the reference's packer; oracle = fp32 matmul on its fp16 `uncompress`."""
    ops = _ops()
    q = torch.from_numpy(golden[f"{name}_q"]).to(cuda)
    meta = torch.from_numpy(golden[f"{name}_meta"]).to(cuda)
    s = torch.from_numpy(golden[f"{name}_s"]).to(cuda)
    k = q.shape[0] * 32
    x = torch.randn(16, k, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(1))
    y = ops.matmul_4bit_2_4(q, x, meta, s)
    ref = x.float().cpu().numpy() @ golden[f"{name}_uncompress"].astype(np.float32)
    check(y, ref)


def test_matmul_plumbing_config(cuda):
    """16 x 4096 x 4096, per-channel scales U(0.001, 0.01): the CPU-runnable benchmark config."""
    ops = _ops()
    qs, metas, ss = ops.random_packed_deltas(1, 4096, 4096, device=cuda, seed=0)
    x = torch.randn(16, 4096, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(0))
    y = ops.matmul_4bit_2_4(qs[0], x, metas[0], ss[0])
    y2 = ops.matmul_4bit_2_4(qs[0], x, metas[0], ss[0])
    assert torch.equal(y, y2)  # deterministic reduction order
    check(y, oracle.matmul_2_4(qs[0].cpu().numpy(), x.cpu().numpy(), metas[0].cpu().numpy(), ss[0].cpu().numpy()))


def test_matmul_leading_dims_and_module(cuda):
    ops = _ops()
    from triteia_b200.nn import sparse_low_precision_linear

    torch.manual_seed(3)
    unc, q, s, meta = ops.gen_sparse_quant4_NT(256, 256, device=cuda)
    x = torch.randn(2, 5, 256, dtype=torch.float16, device=cuda)
    y = ops.matmul_4bit_2_4(q, x, meta, s)
    assert y.shape == (2, 5, 256)
    ref = x.float().cpu().numpy().reshape(10, 256) @ unc.float().cpu().numpy()
    check(y.reshape(10, 256), ref)
    layer = sparse_low_precision_linear(256, 256).to(cuda)
    layer.pack(unc, s)
    assert torch.equal(layer.qweight, q) and torch.equal(layer.meta, meta)
    check(layer(x).reshape(10, 256), ref)


def test_matmul_errors(cuda):
    ops = _ops()
    from triteia_b200.capi import mul_2_4

    q, meta, s = packed(256, 128, -1, seed=1)
    x = torch.randn(4, 128, dtype=torch.float16, device=cuda)
    C = torch.empty(4, 256, dtype=torch.float16, device=cuda)
    with pytest.raises(RuntimeError, match="workspace"):
        mul_2_4(x, q, meta, C, s, torch.zeros(1, dtype=torch.int32, device=cuda))
    with pytest.raises(RuntimeError, match="contiguous"):
        mul_2_4(x.t().contiguous().t(), q, meta, C, s, torch.zeros(64, dtype=torch.int32, device=cuda))
    # K not a multiple of 128: problem-shape error with the reference's message
    with pytest.raises(RuntimeError, match="not compatible"):
        mul_2_4(x[:, :64].contiguous(), q[:2], meta[:, :4].contiguous(), C, s,
                torch.zeros(64, dtype=torch.int32, device=cuda))
    # zero tokens: nothing to do
    y0 = ops.matmul_4bit_2_4(q, x[:0], meta, s)
    assert y0.shape == (0, 256)


# ------------------------------------------------------------------ router (bit-exact)
def run_route(idx_np, num_deltas, tile, offset=0):
    L = _lib()
    dev = torch.device("cuda:0")
    T = len(idx_np)
    idx = torch.from_numpy(np.asarray(idx_np, dtype=np.int32)).to(dev)
    max_tiles = L.lib.trb_route_max_tiles(T, num_deltas, tile)
    nseg = max(1, min(T, num_deltas))
    perm = torch.full((max(T, 1),), -7, dtype=torch.int32, device=dev)
    seg = [torch.full((nseg,), -7, dtype=torch.int32, device=dev) for _ in range(3)]
    til = [torch.full((max(max_tiles, 1),), -7, dtype=torch.int32, device=dev) for _ in range(3)]
    cnt = torch.full((4,), -7, dtype=torch.int32, device=dev)
    L.check(L.lib.trb_route(L.ptr(idx), T, num_deltas, tile, offset, L.ptr(perm), *[L.ptr(t) for t in seg],
                            *[L.ptr(t) for t in til], L.ptr(cnt), 0, L.stream_of(cnt)), "route")
    c = cnt.cpu().numpy()
    R, NT = int(c[0]), int(c[1])
    return (perm.cpu().numpy()[:T], [t.cpu().numpy()[:R] for t in seg], [t.cpu().numpy()[:NT] for t in til], c)


def oracle_tiles(u, st, c, tile):
    td, ts, tc = [], [], []
    for d, a, n in zip(u, st, c):
        for off in range(0, n, tile):
            td.append(d); ts.append(a + off); tc.append(min(tile, n - off))
    return np.array(td, np.int32), np.array(ts, np.int32), np.array(tc, np.int32)


ROUTE_CASES = {
    "sorted": lambda r: np.sort(r.integers(-1, 64, 128)),
    "shuffled": lambda r: r.integers(-1, 64, 128),
    "all_base": lambda r: np.full(37, -1),
    "one_delta": lambda r: np.full(50, 3),
    "single_token": lambda r: np.array([5]),
    "empty": lambda r: np.zeros(0, dtype=np.int64),
    "distinct": lambda r: r.permutation(64),
    "ragged_big": lambda r: r.integers(-1, 1000, 5000),
    "many_tokens": lambda r: r.integers(-1, 32, 8192),
    "zipf": lambda r: np.minimum(r.zipf(1.5, 512) - 1, 127),
}


@pytest.mark.parametrize("case", list(ROUTE_CASES))
@pytest.mark.parametrize("tile", [8, 64])
def test_route_bit_exact(cuda, case, tile):
    rng = np.random.default_rng(zlib.crc32(case.encode()) % 1000)
    idx = ROUTE_CASES[case](rng).astype(np.int32)
    D = 1024 if case == "ragged_big" else 128
    perm, seg, til, cnt = run_route(idx, D, tile)
    operm, u, st, c = oracle.route_any(idx)
    assert np.array_equal(perm, operm)
    assert np.array_equal(seg[0], u) and np.array_equal(seg[1], st) and np.array_equal(seg[2], c)
    td, ts, tc = oracle_tiles(u, st, c, tile)
    assert np.array_equal(til[0], td) and np.array_equal(til[1], ts) and np.array_equal(til[2], tc)
    assert cnt[2] == (idx == -1).sum() and cnt[3] == 0


def test_route_offset_and_out_of_range(cuda):
    idx = np.array([-1, 0, 9, 4, 5, 5, 12, 4, 3, -5], dtype=np.int32)   # deltas are ids 4..7 (offset 4, D = 4)
    perm, seg, til, cnt = run_route(idx, 4, 8, offset=4)
    mapped = np.where((idx - 4 >= 0) & (idx - 4 < 4), idx - 4, -1)
    operm, u, st, c = oracle.route_any(mapped)
    assert np.array_equal(perm, operm) and np.array_equal(seg[0], u) and np.array_equal(seg[2], c)
    assert cnt[3] == 3  # 9, 12 and -5 are outside [-1, offset + D)


# ------------------------------------------------------------------ sbmm
def sbmm_inputs(T, D, K, N, groupsize, seed, base=False, sort=True, frac_base=0.1):
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(seed)
    qs, metas, ss = packed(N, K, groupsize, seed=seed, num=D)
    x = torch.randn(T, K, dtype=torch.float16, device=dev, generator=torch.Generator(dev).manual_seed(seed))
    idx = rng.integers(0, D, T)
    idx[rng.random(T) < frac_base] = -1
    if sort:
        idx = np.sort(idx)
    bw = None
    if base:
        bw = (torch.randn(N, K, device=dev, generator=torch.Generator(dev).manual_seed(seed + 1)) * 0.02).half()
    return qs, metas, ss, x, torch.from_numpy(idx.astype(np.int32)).to(dev), bw


def sbmm_ref(qs, metas, ss, x, idx, bw):
    return oracle.sbmm(qs.cpu().numpy(), x.cpu().numpy(), metas.cpu().numpy(), ss.cpu().numpy(), idx.cpu().numpy(),
                       None if bw is None else bw.cpu().numpy())


@pytest.mark.parametrize("groupsize", [-1, 128])
@pytest.mark.parametrize("sort", [True, False])
@pytest.mark.parametrize("base", [False, True])
def test_sbmm_native(cuda, groupsize, sort, base):
    ops = _ops()
    qs, metas, ss, x, idx, bw = sbmm_inputs(40, 6, 256, 512, groupsize, seed=7, base=base, sort=sort)
    y = ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx, base_weight=bw)
    ref = sbmm_ref(qs, metas, ss, x, idx, bw)
    check(y, ref, mean_tol=None if base else MEAN_TOL)
    if not base:
        assert torch.all(y[idx == -1] == 0)
    y2 = ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx, base_weight=bw)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("variant", ["forloop", "multilaunch", "segments"])
def test_sbmm_reference_call_sequences(cuda, variant):
    ops = _ops()
    qs, metas, ss, x, idx, bw = sbmm_inputs(30, 5, 256, 256, -1, seed=9)
    fn = {"forloop": ops.sbmm_4bit_2_4_forloop, "multilaunch": ops.sbmm_4bit_2_4_multilaunch,
          "segments": ops.sbmm_4bit_2_4_segments}[variant]
    check(fn(qs, x, metas, ss, idx), sbmm_ref(qs, metas, ss, x, idx, None))


def test_sbmm_reference_test_shape_uniform(cuda):
    """("uniform", 10 requests, 5 models, 256 x 512), sorted — tests/ops/test_sbmm.py:15-31."""
    ops = _ops()
    qs, metas, ss, x, idx, _ = sbmm_inputs(10, 5, 256, 512, -1, seed=11)
    check(ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx), sbmm_ref(qs, metas, ss, x, idx, None))


@pytest.mark.parametrize("case", ["all_base", "one_delta", "one_token", "hot_delta", "every_delta_once"])
def test_sbmm_edge_cases(cuda, case):
    ops = _ops()
    qs, metas, ss, x, idx, _ = sbmm_inputs(96, 8, 128, 256, -1, seed=13, sort=False)
    if case == "all_base":
        idx[:] = -1
    elif case == "one_delta":
        idx[:] = 5
    elif case == "one_token":
        x, idx = x[:1].contiguous(), idx[:1]
    elif case == "hot_delta":
        idx[:80] = 2          # 80 tokens of one delta: several token tiles
    elif case == "every_delta_once":
        x, idx = x[:8].contiguous(), torch.arange(8, dtype=torch.int32, device=cuda)
    y = ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx)
    check(y, sbmm_ref(qs, metas, ss, x, idx, None), mean_tol=None)


def test_sbmm_decode_config_shape(cuda):
    """The headline sbmm configuration at reduced delta count: 128 tokens, 4096 x 4096, group 128, 10% base."""
    ops = _ops()
    qs, metas, ss, x, idx, _ = sbmm_inputs(128, 8, 4096, 4096, 128, seed=17, sort=False)
    y = ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx)
    check(y, sbmm_ref(qs, metas, ss, x, idx, None))


def test_sbmm_linearity_full_size(cuda):
    """Size-independent properties at the full 64-delta configuration: f(2x) == 2 f(x) bit for bit
    (scaling by 2 is exact in fp16 and fp32 outside the fp16 subnormal range of the output), and
    permuting the tokens permutes the rows."""
    ops = _ops()
    qs, metas, ss, x, idx, _ = sbmm_inputs(128, 64, 4096, 4096, 128, seed=19, sort=False)
    y = ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx)
    y2 = ops.sbmm_4bit_2_4_native(qs, (x * 2).contiguous(), metas, ss, idx)
    normal = y.abs() >= 1e-3          # fp16 results below 2**-14 round on a fixed grid, not a relative one
    assert torch.equal(y2[normal], (y * 2)[normal])
    assert torch.allclose(y2.float(), 2 * y.float(), rtol=0, atol=2e-7)
    p = torch.randperm(128, device=cuda, generator=torch.Generator(cuda).manual_seed(1))
    yp = ops.sbmm_4bit_2_4_native(qs, x[p].contiguous(), metas, ss, idx[p].contiguous())
    assert torch.equal(yp, y[p])


# ------------------------------------------------------------------ prefill-sized tiles (tcgen05 kernel)
@pytest.mark.parametrize("groupsize", [-1, 128])
@pytest.mark.parametrize("tokens", [40, 256, 300, 700])
def test_matmul_prefill_tiles(cuda, tokens, groupsize):
    ops = _ops()
    q, meta, s = packed(384, 512, groupsize, seed=tokens)
    x = torch.randn(tokens, 512, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(tokens))
    y = ops.matmul_4bit_2_4(q, x, meta, s)
    check(y, oracle.matmul_2_4(q.cpu().numpy(), x.cpu().numpy(), meta.cpu().numpy(), s.cpu().numpy()))
    assert torch.equal(y, ops.matmul_4bit_2_4(q, x, meta, s))


@pytest.mark.parametrize("groupsize", [-1, 128])
@pytest.mark.parametrize("base", [False, True])
def test_sbmm_prefill_segments(cuda, groupsize, base):
    """Contiguous segments of a few hundred tokens per delta (the prefill configuration's shape)."""
    ops = _ops()
    D, K, N = 3, 384, 256
    qs, metas, ss = packed(N, K, groupsize, seed=23, num=D)
    counts = [300, 129, 512]
    idx = np.concatenate([np.full(30, -1)] + [np.full(c, d) for d, c in enumerate(counts)]).astype(np.int32)
    T = len(idx)
    x = torch.randn(T, K, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(5))
    idx_t = torch.from_numpy(idx).to(cuda)
    bw = (torch.randn(N, K, device=cuda, generator=torch.Generator(cuda).manual_seed(6)) * 0.02).half() if base else None
    y = ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx_t, base_weight=bw)
    check(y, sbmm_ref(qs, metas, ss, x, idx_t, bw), mean_tol=None if base else MEAN_TOL)
    p = torch.randperm(T, device=cuda, generator=torch.Generator(cuda).manual_seed(2))
    yp = ops.sbmm_4bit_2_4_native(qs, x[p].contiguous(), metas, ss, idx_t[p].contiguous(), base_weight=bw)
    assert torch.equal(yp, y[p])


# ------------------------------------------------------------------ bmm
@pytest.mark.parametrize("b", [1, 4, 16])
def test_bmm(cuda, b):
    ops = _ops()
    qs, metas, ss = packed(256, 512, -1, seed=b, num=b)
    x = torch.randn(b, 1, 512, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(b))
    y = ops.bmm_4bit_2_4(qs, x, metas, ss)
    assert y.shape == (b, 1, 256)
    ref = np.stack([oracle.matmul_2_4(qs[i].cpu().numpy(), x[i].cpu().numpy(), metas[i].cpu().numpy(),
                                      ss[i].cpu().numpy()) for i in range(b)])
    check(y.reshape(b, 256), ref.reshape(b, 256), mean_tol=1e-3)
    check(ops.bmm_4bit_2_4_forloop(qs, x, metas, ss).reshape(b, 256), ref.reshape(b, 256), mean_tol=1e-3)


# ------------------------------------------------------------------ LoRA
def lora_inputs(T, M, H1, H2, r, seed, dtype=torch.float16):
    dev = torch.device("cuda:0")
    g = torch.Generator(dev).manual_seed(seed)
    A = (torch.randn(M, H1, r, device=dev, generator=g) / H1 ** 0.5).to(dtype)
    B = (torch.randn(M, r, H2, device=dev, generator=g) / r ** 0.5).to(dtype)
    x = torch.randn(T, H1, device=dev, generator=g).to(dtype)
    idx = np.sort(np.random.default_rng(seed).integers(-1, M, T)).astype(np.int32)
    return A, B, x, torch.from_numpy(idx).to(dev)


def lora_ref(A, B, x, idx, scale=1.0):
    return oracle.lora(A.float().cpu().numpy(), B.float().cpu().numpy(), x.float().cpu().numpy(), idx.cpu().numpy(),
                       scale=scale)


@pytest.mark.parametrize("rank", [8, 16, 32, 64])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_lora_bgmv(cuda, rank, dtype):
    ops = _ops()
    A, B, x, idx = lora_inputs(33, 5, 768, 768, rank, seed=rank, dtype=dtype)
    y = ops.lora_bgmv(A, B, x, idx, scale=0.5)
    ref = lora_ref(A, B, x, idx, 0.5)
    tol = 1e-2 if dtype == torch.float16 else 3e-2
    assert oracle.row_rel_err(y.float().cpu().numpy(), ref)[idx.cpu().numpy() >= 0].max() <= tol
    assert torch.all(y[idx == -1] == 0)


def test_lora_bgmv_capi_transposed_layouts(cuda):
    """The two-launch BGMV of the reference API (shrink into fp16 tmp, then expand)."""
    from triteia_b200.capi import add_lora_bgmv
    from triteia_b200 import _lib as L

    A, B, x, idx = lora_inputs(20, 4, 4096, 1024, 16, seed=2)
    keep = idx >= 0
    xk, ik = x[keep].contiguous(), idx[keep].long()
    wa_t = A.transpose(1, 2).contiguous().unsqueeze(1)
    wb_t = B.transpose(1, 2).contiguous().unsqueeze(1)
    y = torch.zeros(xk.shape[0], 1024, dtype=torch.float16, device=cuda)
    add_lora_bgmv(y, xk, wa_t, wb_t, ik, 0, 1.0)
    ref = lora_ref(A, B, xk, ik)
    check(y, ref, mean_tol=5e-3)
    # fused single-launch variant on the same layouts
    y2 = torch.zeros_like(y)
    L.check(L.lib.trb_lora_bgmv_fused(L.ptr(y2), L.ptr(xk), L.ptr(wa_t), L.ptr(wb_t), L.ptr(ik), xk.shape[0], 4096,
                                      1024, 16, 1, 0, 1.0, 0, 0, L.stream_of(y2)), "fused")
    check(y2, ref, mean_tol=5e-3)


@pytest.mark.parametrize("shape", [(768, 768), (256, 256), (4096, 1536)])
def test_lora_sgmv(cuda, shape):
    ops = _ops()
    A, B, x, idx = lora_inputs(150, 6, shape[0], shape[1], 64, seed=4)
    y = ops.lora_sgmv(A, B, x, idx)
    check(y, lora_ref(A, B, x, idx), mean_tol=5e-3)


def test_lora_golden(cuda, golden):
    ops = _ops()
    A, B = torch.from_numpy(golden["lora_A"]).to(cuda), torch.from_numpy(golden["lora_B"]).to(cuda)
    x, idx = torch.from_numpy(golden["lora_x"]).to(cuda), torch.from_numpy(golden["lora_idx"]).to(cuda)
    ref = oracle.lora(golden["lora_A"], golden["lora_B"], golden["lora_x"], golden["lora_idx"])
    check(ops.lora_bgmv(A, B, x, idx), ref, mean_tol=5e-3)
    check(ops.lora_sgmv(A, B, x, idx), ref, mean_tol=5e-3)


# ------------------------------------------------------------------ ldmm
@pytest.mark.parametrize("rank", [8, 16, 64])
@pytest.mark.parametrize("base", [False, True])
def test_ldmm(cuda, rank, base):
    ops = _ops()
    M, D, K, N, T = 5, 5, 768, 768, 60
    qs, metas, ss = packed(N, K, -1, seed=rank, num=D)
    A, B, x, _ = lora_inputs(T, M, K, N, rank, seed=rank)
    idx = torch.from_numpy(np.random.default_rng(rank).integers(-1, M + D, T).astype(np.int32)).to(cuda)
    bw = (torch.randn(N, K, device=cuda) * 0.02).half() if base else None
    y = ops.ldmm(idx, x, A, B, qs, metas, ss, base_weight=bw)
    ref = oracle.ldmm(idx.cpu().numpy(), x.cpu().numpy(), A.cpu().numpy(), B.cpu().numpy(), qs.cpu().numpy(),
                      metas.cpu().numpy(), ss.cpu().numpy(), None if bw is None else bw.cpu().numpy())
    check(y, ref, mean_tol=None)
    yb = ops.baseline_ldmm(idx, x, A, B, qs, metas, ss, base_weight=bw)
    check(yb, ref, mean_tol=None)
    assert torch.allclose(y.float(), yb.float(), rtol=5e-3, atol=5e-3)  # tests/ops/test_ldmm.py:73-77


def test_ldmm_golden_dispatch(cuda, golden):
    ops = _ops()
    t = lambda k: torch.from_numpy(golden[k]).to(cuda)
    y = ops.ldmm(t("ldmm_idx"), t("ldmm_x"), t("lora_A"), t("lora_B"), t("sbmm_q"), t("sbmm_meta"), t("sbmm_s"))
    ref = oracle.ldmm(golden["ldmm_idx"], golden["ldmm_x"], golden["lora_A"], golden["lora_B"], golden["sbmm_q"],
                      golden["sbmm_meta"], golden["sbmm_s"])
    check(y, ref, mean_tol=None)
    assert oracle.row_rel_err(y.float().cpu().numpy(), golden["ldmm_y"].astype(np.float32)).max() < 2e-2


def test_ldmm_float32_input_dtype(cuda):
    ops = _ops()
    qs, metas, ss = packed(256, 256, -1, seed=1, num=2)
    A, B, x, _ = lora_inputs(9, 2, 256, 256, 16, seed=1)
    idx = torch.tensor([0, 1, 2, 3, -1, 3, 0, 2, 1], dtype=torch.int32, device=cuda)
    y = ops.ldmm(idx, x.float(), A, B, qs, metas, ss)
    assert y.dtype == torch.float32


def test_no_device_side_timeouts(cuda):
    from triteia_b200 import _lib as L

    assert L.device_status(0) == 0


# ------------------------------------------------------------------ reference test shapes and full-size properties
def test_sbmm_reference_test_shape_zipf(cuda):
    """("zipf:1.5", 128 requests, 2 models, 4096 x 12288), sorted — tests/ops/test_sbmm.py:15-31."""
    ops = _ops()
    qs, metas, ss = packed(12288, 4096, -1, seed=31, num=2)
    np.random.seed(3)
    idx = torch.sort(ops.generate_model_distribution("zipf:1.5", 128, 2, device=cuda)).values.int()
    x = torch.randn(128, 4096, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(3))
    ref = sbmm_ref(qs, metas, ss, x, idx, None)
    for fn in (ops.sbmm_4bit_2_4_native, ops.sbmm_4bit_2_4_forloop, ops.sbmm_4bit_2_4_multilaunch):
        check(fn(qs, x, metas, ss, idx), ref)


def test_sbmm_tensor_parallel_chunks(cuda):
    """Column- and row-chunked packing (tests/ops/test_sbmm_tp.py:15-91): concatenated / summed per-chunk
    outputs equal the unchunked result."""
    ops = _ops()
    torch.manual_seed(5)
    D, K, N, tp = 3, 256, 512, 2
    uncs, col_parts, row_parts = [], [], []
    for d in range(D):
        unc, q, s, meta = ops.gen_sparse_quant4_NT(N, K, device=cuda)
        uncs.append(unc)
        col_parts.append(ops.torch_weight_to_sparse_marlin(unc, s, tp_size=tp, chunk_by="column"))
        row_parts.append(ops.torch_weight_to_sparse_marlin(unc, s, tp_size=tp, chunk_by="row"))
    x = torch.randn(10, K, dtype=torch.float16, device=cuda)
    idx = torch.tensor([-1, 0, 0, 1, 1, 1, 2, 2, 2, 2], dtype=torch.int32, device=cuda)
    ref = ops.sbmm_16bit_forloop(torch.stack(uncs), x, idx).float().cpu().numpy()
    cols = []
    for c in range(tp):
        qs = torch.stack([col_parts[d][0][c] for d in range(D)])
        ss = torch.stack([col_parts[d][1][c] for d in range(D)])
        ms = torch.stack([col_parts[d][2][c] for d in range(D)])
        cols.append(ops.sbmm_4bit_2_4_native(qs, x, ms, ss, idx))
    check(torch.cat(cols, dim=1), ref, mean_tol=5e-3)
    acc = 0
    for c in range(tp):
        qs = torch.stack([row_parts[d][0][c] for d in range(D)])
        ss = torch.stack([row_parts[d][1][c] for d in range(D)])
        ms = torch.stack([row_parts[d][2][c] for d in range(D)])
        acc = acc + ops.sbmm_4bit_2_4_native(qs, x[:, c * K // tp:(c + 1) * K // tp].contiguous(), ms, ss, idx).float()
    check(acc, ref, mean_tol=5e-3)


def test_bmm_reference_shape(cuda):
    """b in {4, 8, 16}, 512^3 — tests/ops/test_bmm.py:12-47 (mean-relative < 1e-3)."""
    ops = _ops()
    for b in (4, 8):
        qs, metas, ss = packed(512, 512, -1, seed=40 + b, num=b)
        x = torch.randn(b, 1, 512, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(b))
        y = ops.bmm_4bit_2_4(qs, x, metas, ss)
        ref = np.stack([oracle.matmul_2_4(qs[i].cpu().numpy(), x[i].cpu().numpy(), metas[i].cpu().numpy(),
                                          ss[i].cpu().numpy()) for i in range(b)]).reshape(b, 512)
        check(y.reshape(b, 512), ref, mean_tol=1e-3)


def test_ldmm_full_size_properties(cuda):
    """The ldmm benchmark configuration at full size (4096 -> 11008, 32 deltas + 32 rank-16 adapters, 256 tokens,
    Zipf(1.2) ids): agreement with the per-id loop path, doubling the input doubles the output, permuting
    tokens permutes rows; a sample of rows against the oracle."""
    ops = _ops()
    K, N, T, M, D, R = 4096, 11008, 256, 32, 32, 16
    qs, metas, ss = ops.random_packed_deltas(D, K, N, device=cuda, seed=2, scale_lo=0.001, scale_hi=0.01)
    g = torch.Generator(cuda).manual_seed(0)
    base = (torch.randn(N, K, device=cuda, generator=g) * 0.02).half()
    A = (torch.randn(M, K, R, device=cuda, generator=g) / K ** 0.5).half()
    B = (torch.randn(M, R, N, device=cuda, generator=g) / R ** 0.5).half()
    x = torch.randn(T, K, device=cuda, generator=g).half()
    rng = np.random.default_rng(0)
    p = np.arange(1, M + D + 1, dtype=np.float64) ** -1.2
    idx = torch.from_numpy(rng.permutation(M + D)[rng.choice(M + D, T, p=p / p.sum())].astype(np.int32)).to(cuda)
    y = ops.ldmm(idx, x, A, B, qs, metas, ss, base_weight=None)
    yb = ops.baseline_ldmm(idx, x, A, B, qs, metas, ss, base_weight=None)
    assert oracle.row_rel_err(y.float().cpu().numpy(), yb.float().cpu().numpy()).max() <= 1e-2
    y2 = ops.ldmm(idx, (x * 2).contiguous(), A, B, qs, metas, ss)
    normal = y.abs() >= 1e-2
    assert torch.allclose(y2.float()[normal], 2 * y.float()[normal], rtol=2e-3, atol=0)   # LoRA adds in fp16
    perm = torch.randperm(T, device=cuda, generator=torch.Generator(cuda).manual_seed(1))
    yp = ops.ldmm(idx[perm].contiguous(), x[perm].contiguous(), A, B, qs, metas, ss)
    assert torch.equal(yp, y[perm])
    yfull = ops.ldmm(idx, x, A, B, qs, metas, ss, base_weight=base)
    rows = [0, 17, 101, 255]
    sub = torch.tensor(rows, device=cuda)
    ref = oracle.ldmm(idx[sub].cpu().numpy(), x[sub].cpu().numpy(), A.cpu().numpy(), B.cpu().numpy(), qs.cpu().numpy(),
                      metas.cpu().numpy(), ss.cpu().numpy(), base.cpu().numpy())
    check(yfull[sub], ref, mean_tol=None)
    # 64 more rows over every id of the batch, three 128-column windows each (first, middle, last
    # stripe): base + adapter or delta, stated with the oracle's column-block decoder
    idx_np = idx.cpu().numpy()
    more = np.array(_sampled_rows(idx_np, per_id=3, seed=2))
    assert len(more) >= 64
    x32 = x[torch.from_numpy(more).to(cuda)].float().cpu().numpy()
    A32, B32, base32 = A.float().cpu().numpy(), B.float().cpu().numpy(), base.float().cpu().numpy()
    for blk0 in (0, 86, N // 64 - 2):
        c0, c1 = 64 * blk0, 64 * blk0 + 128
        ref = x32 @ base32[c0:c1].T
        delta_ids = np.where(idx_np[more] >= M, idx_np[more] - M, -1).astype(np.int32)
        ref += oracle.sbmm_rows(qs, x[torch.from_numpy(more).to(cuda)], metas, ss, delta_ids, np.arange(len(more)), blk0, 2)
        for i, t in enumerate(more):
            a = idx_np[t]
            if 0 <= a < M:
                ref[i] += (x32[i] @ A32[a]) @ B32[a][:, c0:c1]
        got = yfull[torch.from_numpy(more).to(cuda)][:, c0:c1].float().cpu().numpy()
        assert oracle.row_rel_err(got, ref).max() <= 1e-2


def test_sbmm_prefill_full_size_properties(cuda):
    """The prefill benchmark configuration (5120 -> 13824, group 128, 8192 tokens in 16 segments of 512, 16 of 32
    deltas resident here): the tcgen05 path against the oracle on a sample of rows, linearity, and equality
    with the small-tile kernel on a 24-token slice of the same deltas."""
    ops = _ops()
    K, N, T, SEG, D = 5120, 13824, 8192, 16, 16
    qs, metas, ss = ops.random_packed_deltas(D, K, N, groupsize=128, device=cuda, seed=1, scale_lo=0.001, scale_hi=0.01)
    x = torch.randn(T, K, device=cuda, generator=torch.Generator(cuda).manual_seed(0)).half()
    idx = torch.arange(SEG, device=cuda, dtype=torch.int32).repeat_interleave(T // SEG)
    y = ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx)
    y2 = ops.sbmm_4bit_2_4_native(qs, (x * 2).contiguous(), metas, ss, idx)
    normal = y.abs() >= 1e-3
    assert torch.equal(y2[normal], (y * 2)[normal])
    rows = torch.tensor([0, 511, 512, 4095, 8191], device=cuda)
    ref = oracle.sbmm(qs.cpu().numpy()[[0, 1, 7, 15]], x[rows].cpu().numpy(), metas.cpu().numpy()[[0, 1, 7, 15]],
                      ss.cpu().numpy()[[0, 1, 7, 15]], np.array([0, 0, 1, 2, 3]))
    check(y[rows], ref)
    # four rows of every segment, three 128-column windows (first, middle, last stripe)
    idx_np = idx.cpu().numpy()
    more = np.array(_sampled_rows(idx_np, per_id=4, seed=3))
    assert len(more) == 4 * SEG
    xm = x[torch.from_numpy(more).to(cuda)]
    for blk0 in (0, 107, N // 64 - 2):
        ref = oracle.sbmm_rows(qs, xm, metas, ss, idx_np[more], np.arange(len(more)), blk0, 2)
        got = y[torch.from_numpy(more).to(cuda)][:, 64 * blk0:64 * blk0 + 128].float().cpu().numpy()
        assert oracle.row_rel_err(got, ref).max() <= 1e-2
    small = torch.cat([torch.arange(0, 8), torch.arange(512, 520), torch.arange(8184, 8192)]).to(cuda)
    ys = ops.sbmm_4bit_2_4_native(qs, x[small].contiguous(), metas, ss, idx[small].contiguous())
    assert oracle.row_rel_err(ys.float().cpu().numpy(), y[small].float().cpu().numpy()).max() <= 2e-3


@pytest.mark.parametrize("rows,n", [(1, 8), (37, 256), (200, 11008)])
def test_row_checksum(cuda, rows, n):
    """fp32 per-row sums of an fp16 matrix: overwrite, then accumulate; identical from run to run."""
    from triteia_b200 import _lib

    g = torch.Generator(device="cuda").manual_seed(rows)
    y = torch.randn(rows, n, generator=g, device="cuda").half()
    sums = torch.full((rows,), 123.0, device="cuda")

    def call(acc):
        _lib.check(_lib.lib.trb_row_checksum(_lib.ptr(y), _lib.ptr(sums), rows, n, acc, _lib.dev_of(y),
                                             _lib.stream_of(y)), "row_checksum")
    call(0)
    ref = y.double().sum(dim=1)
    first = sums.clone()
    assert torch.allclose(first.double(), ref, rtol=1e-5, atol=1e-3)
    call(1)
    assert torch.allclose(sums.double(), 2 * ref, rtol=1e-5, atol=2e-3)
    call(0)
    assert torch.equal(sums, first)
    # bad shapes are refused before any launch
    assert _lib.lib.trb_row_checksum(_lib.ptr(y), _lib.ptr(sums), rows, n + 1, 0, _lib.dev_of(y), _lib.stream_of(y)) != 0


@pytest.mark.parametrize("segs,tokens", [(3, 5), (20, 40), (40, 100)])
def test_segment_list_tail_k_split(cuda, segs, tokens):
    """trb_sbmm_2_4_ksplit: few work items (every one is a split tail item), a mix, and a launch whose
    last round is split.  Against the oracle, against the unsplit entry point, twice for bit identity,
    and the counters are zero again afterwards."""
    import triteia_b200.ops as ops
    from triteia_b200 import _lib
    from triteia_b200.capi import sbmm_2_4

    K, N, g = 1024, 2048, 128
    qs, metas, ss = ops.random_packed_deltas(segs, K, N, groupsize=g, device=cuda, seed=segs, scale_lo=0.005, scale_hi=0.02)
    rng = np.random.default_rng(tokens)
    ids = np.sort(rng.integers(0, segs, tokens)).astype(np.int32)
    idx = torch.from_numpy(ids).to(cuda)
    x = torch.randn(tokens, K, device=cuda, generator=torch.Generator(cuda).manual_seed(1)).half()
    uniq, counts = torch.unique_consecutive(idx, return_counts=True)
    starts = (torch.cumsum(counts, 0) - counts).int()
    uniq, counts = uniq.int(), counts.int()
    nbytes = _lib.lib.trb_sbmm_ksplit_bytes()
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device=cuda)

    def split_call(y):
        _lib.check(_lib.lib.trb_sbmm_2_4_ksplit(_lib.ptr(x), _lib.ptr(qs), _lib.ptr(metas), _lib.ptr(y), _lib.ptr(ss),
                                                _lib.ptr(uniq), _lib.ptr(starts), _lib.ptr(counts), N, tokens, K,
                                                int(uniq.numel()), g, _lib.dev_of(y), _lib.stream_of(y),
                                                _lib.ptr(scratch), nbytes), "sbmm_2_4_ksplit")
    y1 = torch.full((tokens, N), 3.0, dtype=torch.float16, device=cuda)
    y2 = torch.full((tokens, N), -3.0, dtype=torch.float16, device=cuda)
    split_call(y1)
    split_call(y2)
    y0 = torch.empty(tokens, N, dtype=torch.float16, device=cuda)
    ws = torch.zeros(int(uniq.numel()), N // 8, dtype=torch.int32, device=cuda)
    sbmm_2_4(x, qs, metas, y0, ss, uniq, ws, starts, counts)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    assert int(scratch[:512].max()) == 0
    ref = oracle.sbmm(qs.cpu().numpy(), x.cpu().numpy(), metas.cpu().numpy(), ss.cpu().numpy(), ids)
    assert oracle.row_rel_err(y1.float().cpu().numpy(), ref).max() <= 1e-2
    assert oracle.row_rel_err(y1.float().cpu().numpy(), y0.float().cpu().numpy()).max() <= 1e-2
    # a scratch that is too small or misaligned is refused
    assert _lib.lib.trb_sbmm_2_4_ksplit(_lib.ptr(x), _lib.ptr(qs), _lib.ptr(metas), _lib.ptr(y1), _lib.ptr(ss),
                                        _lib.ptr(uniq), _lib.ptr(starts), _lib.ptr(counts), N, tokens, K,
                                        int(uniq.numel()), g, _lib.dev_of(y1), _lib.stream_of(y1), _lib.ptr(scratch),
                                        1024) == _lib.ERR_SCRATCH
    assert _lib.device_status(0) == 0


@pytest.mark.parametrize("k,n,groupsize", [(128, 256, -1), (512, 768, 128), (1024, 512, -1)])
def test_pack_kernel_bit_exact(cuda, k, n, groupsize):
    """The packer kernel against the torch packer (itself pinned on the reference's vectors) and the
    round trip through the on-GPU decoder."""
    from triteia_b200.ops.utils.sparsity import pack_2_4, pack_2_4_cuda
    from triteia_b200 import _lib

    g = torch.Generator(device="cuda").manual_seed(k + n)
    groups = 1 if groupsize == -1 else k // groupsize
    lev = torch.randint(1, 8, (k, n), generator=g, device=cuda) * (torch.randint(0, 2, (k, n), generator=g, device=cuda) * 2 - 1)
    keep = torch.rand(k // 4, 4, n, generator=g, device=cuda).argsort(dim=1).argsort(dim=1) < 2
    scales = (torch.rand(groups, n, generator=g, device=cuda) * 0.01 + 0.001).half()
    s_rows = scales if groups == 1 else scales.repeat_interleave(k // groups, dim=0)
    w = ((lev * keep.reshape(k, n)).half() * s_rows).half()
    q_ref, s_ref, m_ref = pack_2_4(w, scales)
    q, s, m = pack_2_4_cuda(w, scales)
    torch.cuda.synchronize()
    assert torch.equal(q, q_ref) and torch.equal(m, m_ref) and torch.equal(s, s_ref)
    out = torch.empty(k, n, dtype=torch.float16, device=cuda)
    _lib.check(_lib.lib.trb_unpack_2_4(_lib.ptr(q), _lib.ptr(m), _lib.ptr(s), _lib.ptr(out), n, k, groupsize, 0,
                                       _lib.stream_of(out)), "unpack")
    torch.cuda.synchronize()
    assert torch.equal(out, w)
    assert _lib.lib.trb_pack_2_4(_lib.ptr(w), _lib.ptr(scales), _lib.ptr(q), _lib.ptr(m), _lib.ptr(s), k + 1, n, groupsize, 0,
                                 _lib.stream_of(w)) == _lib.ERR_PROB_SHAPE


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_elementwise_neighbours(cuda, dtype):
    """gelu_quick, silu_and_mul and rotary_embedding (both styles, plain and batched) against fp32
    torch statements of the same formulas; tolerance = a few roundings of the 16-bit type."""
    from triteia_b200 import triteia_cuda as tc
    from triteia_b200.capi import QuickGELU, rotary_embedding, batched_rotary_embedding

    g = torch.Generator(device="cuda").manual_seed(3)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=4e-3, atol=4e-3)
    x = torch.randn(37, 11008, generator=g, device=cuda).to(dtype)
    y = QuickGELU()(x)
    assert torch.allclose(y.float(), x.float() * torch.sigmoid(1.702 * x.float()), **tol)
    gu = torch.randn(37, 2 * 1024, generator=g, device=cuda).to(dtype)
    out = torch.empty(37, 1024, dtype=dtype, device=cuda)
    tc.silu_and_mul(out, gu)
    ref = torch.nn.functional.silu(gu[:, :1024].float()) * gu[:, 1024:].float()
    assert torch.allclose(out.float(), ref, **tol)

    T, H, KVH, hs, rot, maxpos = 19, 8, 2, 64, 32, 100
    cache = torch.randn(2 * maxpos, rot, generator=g, device=cuda).clamp(-1, 1).to(dtype)
    pos = torch.randint(0, maxpos, (T,), generator=g, device=cuda, dtype=torch.int64)
    offs = torch.randint(0, 2, (T,), generator=g, device=cuda, dtype=torch.int64) * maxpos

    def ref_rot(t, rows, neox):
        t = t.float().reshape(T, -1, hs).clone()
        cos, sin = cache[rows, : rot // 2].float()[:, None, :], cache[rows, rot // 2:].float()[:, None, :]
        if neox:
            a, b = t[..., : rot // 2].clone(), t[..., rot // 2: rot].clone()
            t[..., : rot // 2], t[..., rot // 2: rot] = a * cos - b * sin, b * cos + a * sin
        else:
            a, b = t[..., 0:rot:2].clone(), t[..., 1:rot:2].clone()
            t[..., 0:rot:2], t[..., 1:rot:2] = a * cos - b * sin, b * cos + a * sin
        return t.reshape(T, -1)

    for neox in (True, False):
        q0 = torch.randn(T, H * hs, generator=g, device=cuda).to(dtype)
        k0 = torch.randn(T, KVH * hs, generator=g, device=cuda).to(dtype)
        q, k = q0.clone(), k0.clone()
        rotary_embedding(pos, q, k, hs, cache, neox)
        assert torch.allclose(q.float(), ref_rot(q0, pos, neox), **tol) and torch.allclose(k.float(), ref_rot(k0, pos, neox), **tol)
        q, k = q0.clone(), k0.clone()
        batched_rotary_embedding(pos, q, k, hs, cache, neox, rot, offs)
        assert torch.allclose(q.float(), ref_rot(q0, pos + offs, neox), **tol)
        assert torch.allclose(k.float(), ref_rot(k0, pos + offs, neox), **tol)
        assert torch.equal(q[:, rot:hs], q0[:, rot:hs])          # beyond rot_dim nothing moves


# ------------------------------------------------------------------ overlapping calls, full-size oracle comparisons
def _sampled_rows(idx_np, per_id=1, seed=0):
    rng = np.random.default_rng(seed)
    rows = []
    for d in np.unique(idx_np):
        cand = np.flatnonzero(idx_np == d)
        rows.extend(int(r) for r in rng.choice(cand, size=min(per_id, len(cand)), replace=False))
    return sorted(rows)


def test_sbmm_two_streams_do_not_share_scratch(cuda):
    """Two different batches in flight on two streams: the op keeps its working memory per stream
    (the reference allocates its workspace per call), so both results must match the oracle."""
    ops = _ops()
    qs, metas, ss, xa, ia, _ = sbmm_inputs(128, 16, 1024, 2048, 128, seed=41, sort=False)
    _, _, _, xb, ib, _ = sbmm_inputs(128, 16, 1024, 2048, 128, seed=42, sort=False)
    ib = torch.roll(ib, 7)
    sa, sb = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    outs = {}
    for rep in range(20):                      # interleaved launches, no synchronisation in between
        with torch.cuda.stream(sa):
            outs["a"] = ops.sbmm_4bit_2_4_native(qs, xa, metas, ss, ia)
        with torch.cuda.stream(sb):
            outs["b"] = ops.sbmm_4bit_2_4_native(qs, xb, metas, ss, ib)
    torch.cuda.synchronize()
    check(outs["a"], sbmm_ref(qs, metas, ss, xa, ia, None))
    check(outs["b"], sbmm_ref(qs, metas, ss, xb, ib, None))
    assert _lib().device_status(0) == 0


def test_sbmm_decode_full_size_against_oracle(cuda):
    """The headline configuration at its full size (64 deltas, 128 tokens, group 128, unsorted, tail K
    split active): one sampled row of every distinct id x 128 columns against the oracle, and rows
    with id -1 exactly zero."""
    ops = _ops()
    qs, metas, ss, x, idx, _ = sbmm_inputs(128, 64, 4096, 4096, 128, seed=23, sort=False)
    y = ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx)
    idx_np = idx.cpu().numpy()
    rows = _sampled_rows(idx_np, per_id=1, seed=1)
    for blk0 in (0, 31, 62):
        ref = oracle.sbmm_rows(qs, x, metas, ss, idx_np, rows, blk0=blk0, nblk=2)
        got = y[rows][:, 64 * blk0:64 * blk0 + 128].float().cpu().numpy()
        err = oracle.row_rel_err(got, ref)
        assert err.max() <= ROW_TOL, f"columns {64 * blk0}: row rel err {err.max():.4g}"
    assert torch.all(y[idx == -1] == 0)


# ------------------------------------------------------------------ base product on the library's own kernel
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("T,K,N", [(1, 128, 256), (40, 256, 512), (256, 4096, 1024), (300, 512, 11008), (700, 1024, 384)])
def test_base_gemm(cuda, T, K, N, dtype):
    """y = x @ W^T against an fp32 torch statement of the same product (the reference calls torch.matmul
    here: sbmm.py:90-93); fp16 / bf16 rounding of the output bounds the error."""
    from triteia_b200.ops.matmul._base import base_gemm
    g = torch.Generator(cuda).manual_seed(T + K + N)
    x = torch.randn(T, K, device=cuda, generator=g).to(dtype)
    w = (torch.randn(N, K, device=cuda, generator=g) * 0.05).to(dtype)
    y = base_gemm(x, w)
    ref = (x.float() @ w.float().t()).cpu().numpy()
    err = oracle.row_rel_err(y.float().cpu().numpy(), ref)
    assert err.max() <= (ROW_TOL if dtype == torch.float16 else 2e-2), f"row rel err {err.max():.4g}"
    y2 = base_gemm(x, w, out=y.clone(), accumulate=True)
    err2 = oracle.row_rel_err(y2.float().cpu().numpy(), 2 * ref)
    assert err2.max() <= 2e-2
    assert _lib().device_status(0) == 0


@pytest.mark.parametrize("M,rank", [(3, 8), (5, 16), (32, 16), (4, 64)])
def test_base_gemm_with_lora_expand(cuda, M, rank):
    """Base product and LoRA expand in one accumulator: shrink rows + trb_base_gemm against the oracle's
    lora statement (lora_forloop semantics, lora.py:4-20), ids outside [0, M) get the base only."""
    from triteia_b200.ops.matmul._base import base_gemm, lora_shrink_rows
    T, K, N = 100, 512, 768
    A, B, x, idx = lora_inputs(T, M, K, N, rank, seed=3 * M + rank)
    idx[::7] = -1
    idx[3::11] = M + 2                      # an id of the delta range: no adapter
    w = (torch.randn(N, K, device=cuda, generator=torch.Generator(cuda).manual_seed(5)) * 0.05).half()
    v = lora_shrink_rows(x, A, idx)
    y = base_gemm(x, w, lora_v=v, lora_b=B.view(M * rank, N))
    idx_np = idx.cpu().numpy().copy()
    idx_np[idx_np >= M] = -1
    ref = oracle.lora(A.cpu().numpy(), B.cpu().numpy(), x.cpu().numpy(), idx_np, base_weight=w.cpu().numpy())
    check(y, ref, mean_tol=None)
    assert _lib().device_status(0) == 0


# ------------------------------------------------------------------ tiles chosen per segment, long lists
def test_sbmm_zipf_batch_mixed_tiles(cuda):
    """A Zipf(1.5) batch of 512 tokens over 64 deltas through the one-call path: the hot deltas
    (more than 32 rows) go to the tcgen05 kernel in 256-token tiles, the others to the mma.sp kernel in
    8-token tiles, all inside one call.  Every row against the oracle; run twice, bit-identical."""
    ops = _ops()
    T, D, K, N = 512, 64, 512, 768
    qs, metas, ss = packed(N, K, 128, seed=51, num=D)
    rng = np.random.default_rng(51)
    p = np.arange(1, D + 1, dtype=np.float64) ** -1.5
    idx_np = rng.choice(D, T, p=p / p.sum()).astype(np.int32)
    idx_np[rng.choice(T, 20, replace=False)] = -1
    counts = np.bincount(idx_np[idx_np >= 0], minlength=D)
    assert counts.max() > 32 and ((counts > 8) & (counts <= 32)).any() and ((counts > 0) & (counts <= 8)).any()
    x = torch.randn(T, K, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(51))
    idx = torch.from_numpy(idx_np).to(cuda)
    y = ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx)
    check(y, sbmm_ref(qs, metas, ss, x, idx, None))
    assert torch.all(y[idx == -1] == 0)
    assert torch.equal(y, ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx))
    assert _lib().device_status(0) == 0


@pytest.mark.parametrize("count", [8, 9, 32, 33, 100, 256, 300])
@pytest.mark.parametrize("others", [6, 130])
def test_sbmm_segment_sizes_around_the_class_bounds(cuda, count, others):
    """One delta with `count` rows among `others` other rows: up to 32 rows it is cut into 8-token
    tiles; beyond that it goes to the tcgen05 kernel when the batch has more than 128 tokens."""
    ops = _ops()
    D, K, N = 6, 256, 512
    qs, metas, ss = packed(N, K, -1, seed=60 + count, num=D)
    idx_np = np.concatenate([np.full(count, 2), np.arange(others) % D, [-1, -1]]).astype(np.int32)
    np.random.default_rng(count).shuffle(idx_np)
    T = idx_np.size
    x = torch.randn(T, K, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(count))
    idx = torch.from_numpy(idx_np).to(cuda)
    y = ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx)
    check(y, sbmm_ref(qs, metas, ss, x, idx, None))


def test_sbmm_more_than_1024_segments(cuda):
    """2048 tokens over 1500 deltas in one call (more tiles than one launch's shared-memory table
    held before), and the same batch through the segment-list entry point, which splits lists of
    more than 1024 segments over several launches."""
    ops = _ops()
    T, D, K, N = 2048, 1500, 128, 256
    qs, metas, ss = packed(N, K, -1, seed=71, num=D)
    rng = np.random.default_rng(71)
    idx_np = np.sort(rng.integers(-1, D, T)).astype(np.int32)
    x = torch.randn(T, K, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(71))
    idx = torch.from_numpy(idx_np).to(cuda)
    ref = sbmm_ref(qs, metas, ss, x, idx, None)
    assert len(np.unique(idx_np[idx_np >= 0])) > 1024
    check(ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx), ref)
    check(ops.sbmm_4bit_2_4_segments(qs, x, metas, ss, idx), ref)
    assert _lib().device_status(0) == 0


# ------------------------------------------------------------------ bounded waits, converter on the device, reference host code
def test_bounded_wait_expires_and_reports(cuda):
    """A wait on a barrier nothing signals gives up after its poll limit, the kernel ends normally and
    the device error word carries TRB_ERR_TIMEOUT exactly once; the context stays usable."""
    L = _lib()
    assert L.device_status(0) == 0
    flag = torch.zeros(1, dtype=torch.int32, device=cuda)
    L.check(L.lib.trb_selftest_timeout(1000, L.ptr(flag), 0, L.stream_of(flag)), "selftest_timeout")
    assert L.device_status(0) == L.ERR_TIMEOUT
    assert int(flag.item()) == 1
    assert L.device_status(0) == 0
    qs, metas, ss, x, idx, _ = sbmm_inputs(16, 3, 128, 256, -1, seed=3)
    check(_ops().sbmm_4bit_2_4_native(qs, x, metas, ss, idx), sbmm_ref(qs, metas, ss, x, idx, None))
    assert L.device_status(0) == 0


def test_converter_on_device_through_sbmm(cuda):
    """A GPTQ-style module converted on the GPU (packer kernel for fp16 CUDA chunks), tp 1 and 2: the
    chunks pass the output check of verify_weights, and the tp-1 packed tensors pushed through sbmm as a
    one-delta set match the oracle on the dequantised source weight."""
    from tests.test_converter import _gptq_module
    from triteia_b200.converters.deltazip import convert_state_dict
    from triteia_b200.converters.verify_weights import check_output, check_tp_group_equal
    rng = np.random.default_rng(5)
    src = {}
    dense = {}
    for name, k, n in (("model.layers.0.self_attn.q_proj", 256, 512), ("model.layers.0.self_attn.k_proj", 256, 512),
                       ("model.layers.0.self_attn.v_proj", 256, 512), ("model.layers.0.self_attn.o_proj", 256, 512)):
        mod, d = _gptq_module(rng, k, n)
        dense[name] = d
        for key, t in mod.items():
            src[f"{name}.{key}"] = t.to(cuda)
    one = convert_state_dict(src, 1, use_kernel=True)
    two = convert_state_dict(src, 2, use_kernel=True)
    # a row-split module keeps all its scales in every chunk; nothing else may repeat across ranks
    assert all(comp == "scales" and mod.endswith("o_proj") for mod, comp, _, _ in check_tp_group_equal(two))
    for module in ("model.layers.0.self_attn.qkv_proj", "model.layers.0.self_attn.o_proj"):
        assert check_output(two, one, module, nr=64) < 1e-2
    q, m, s = (one[f"model.layers.0.self_attn.qkv_proj.0.{c}"] for c in ("qweight", "meta", "scales"))
    x = torch.randn(24, 256, dtype=torch.float16, device=cuda, generator=torch.Generator(cuda).manual_seed(1))
    idx = torch.zeros(24, dtype=torch.int32, device=cuda)
    y = _ops().sbmm_4bit_2_4_native(q[None], x, m[None], s[None], idx)
    w = np.concatenate([dense[f"model.layers.0.self_attn.{p}_proj"] for p in "qkv"], axis=1).astype(np.float32)
    check(y, x.float().cpu().numpy() @ w, mean_tol=None)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rank", [8, 16, 64])
def test_sgmv_stacked_ragged_segments(cuda, rank, dtype):
    """The tensor-core SGMV on stacked weights: ragged segments (one empty, one of a single row, one
    longer than a token tile), rows before the first segment untouched, shrink then expand against
    the oracle's lora statement."""
    from triteia_b200.ops.matmul.lora import sgmv_stacked
    M, K, N = 5, 512, 768
    lens = [7, 0, 1, 300, 40]
    lead = 5                                             # rows without an adapter in front
    T = lead + sum(lens)
    g = torch.Generator(cuda).manual_seed(rank)
    A = (torch.randn(M, K, rank, device=cuda, generator=g) / K ** 0.5).to(dtype)
    B = (torch.randn(M, rank, N, device=cuda, generator=g) / rank ** 0.5).to(dtype)
    x = torch.randn(T, K, device=cuda, generator=g).to(dtype)
    seg = torch.tensor(np.concatenate([[lead], lead + np.cumsum(lens)]).astype(np.int32), device=cuda)
    y0 = torch.randn(T, N, device=cuda, generator=g).to(dtype)
    y = y0.clone()
    v = torch.zeros(T, rank, dtype=dtype, device=cuda)
    sgmv_stacked(v, x, A, seg, accumulate=False)
    sgmv_stacked(y, v, B, seg, accumulate=True)
    idx = np.concatenate([np.full(lead, -1)] + [np.full(n, i) for i, n in enumerate(lens)])
    ref = y0.float().cpu().numpy() + oracle.lora(A.float().cpu().numpy(), B.float().cpu().numpy(), x.float().cpu().numpy(), idx)
    err = oracle.row_rel_err(y.float().cpu().numpy(), ref)
    assert err.max() <= (ROW_TOL if dtype == torch.float16 else 3e-2), f"row rel err {err.max():.4g}"
    assert torch.equal(y[:lead], y0[:lead])
    assert _lib().device_status(0) == 0
