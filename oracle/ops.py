"""CPU oracle, part 2: the operators of the indexed delta matmul path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and the cpu_baseline / reference legs of bench.py may
import this package; the product (triteia_b200) never does.

Every function is the fp32 "dequantise, then matmul" statement of one reference operator,
computed from the PACKED tensors (never from the generator's fp16 copy):

  matmul_2_4      triteia/python/ops/matmul/sparse_low_precision.py:5-24
  route_sorted    triteia/python/ops/matmul/sbmm.py:96,112-123 (unique_consecutive, drop the
                  leading -1 run, exclusive cumsum of counts)
  route_any       the same result for indices in any order: stable sort by (delta id) with
                  -1 first, then route_sorted (the fused entry points accept this)
  sbmm            triteia/python/ops/matmul/sbmm.py:7-23 (sbmm_16bit_forloop semantics)
  lora            triteia/python/ops/matmul/lora.py:4-20 (lora_forloop)
  bgmv            triteia/python/capi/punica.py:43-60 (docstring semantics of add_lora_bgmv)
  sgmv            triteia/python/capi/punica.py:13-27 (docstring semantics of add_lora_sgmv_cutlass)
  ldmm            triteia/python/ops/matmul/ldmm.py:22-46 (dispatch rule of baseline_ldmm)

Parity pin: tests/test_oracle_golden.py compares route_sorted, sbmm, lora and ldmm with
outputs of the reference's torch code stored in tests/golden/reference_vectors.npz.
SGMV runs inside an un-vendored CUTLASS grouped GEMM in the reference and its test asserts
nothing, so SGMV parity is pinned only through `lora` (same mathematical result).
"""
import numpy as np

from .delta_format import dequantize


def _f32(a):
    return np.asarray(a).astype(np.float32)


def matmul_2_4(qweight, x, meta, s):
    """y[T, N] = x[T, K] @ W[K, N] in fp32."""
    return _f32(x) @ _f32(dequantize(qweight, meta, s))


def route_sorted(indices):
    """indices int32 [T], grouped by delta id with the -1 run first.

    Returns (unique int32 [R], start int32 [R], count int32 [R]).
    """
    idx = np.asarray(indices).astype(np.int64)
    if idx.size == 0:
        z = np.zeros(0, dtype=np.int32)
        return z, z, z
    change = np.flatnonzero(np.diff(idx)) + 1
    starts = np.concatenate([[0], change])
    ends = np.concatenate([change, [idx.size]])
    uniq = idx[starts]
    keep = uniq != -1
    return (uniq[keep].astype(np.int32), starts[keep].astype(np.int32),
            (ends - starts)[keep].astype(np.int32))


def route_any(indices):
    """Any order.  Returns (perm int32 [T], unique, start, count) where perm lists the token
    positions in sorted order (stable, -1 first) and start/count index the sorted order."""
    idx = np.asarray(indices).astype(np.int64)
    perm = np.argsort(idx, kind="stable").astype(np.int32)
    u, st, c = route_sorted(idx[perm])
    return perm, u, st, c


def sbmm(qweights, xs, metas, ss, indices, base_weight=None):
    """y[t] = x[t] @ base.T + x[t] @ W[idx[t]] (idx >= 0); indices in any order."""
    xs32 = _f32(xs)
    n_out = np.asarray(ss).shape[2]
    y = xs32 @ _f32(base_weight).T if base_weight is not None else np.zeros((xs32.shape[0], n_out), np.float32)
    idx = np.asarray(indices)
    for d in np.unique(idx):
        if d < 0:
            continue
        w = _f32(dequantize(qweights[d], metas[d], ss[d]))
        m = idx == d
        y[m] += xs32[m] @ w
    return y


def sbmm_rows(qweights, xs, metas, ss, indices, rows, blk0=0, nblk=2, base_weight=None):
    """`sbmm` restricted to the token rows `rows` and output columns [64*blk0, 64*(blk0+nblk)):
    returns fp32 [len(rows), 64*nblk].  Full-size checks decode only these column blocks."""
    from .delta_format import column_blocks, to_numpy

    rows = np.asarray(rows)
    xs32 = _f32(to_numpy(xs)[rows])
    idx = to_numpy(indices)[rows]
    c0, c1 = 64 * blk0, 64 * (blk0 + nblk)
    y = (xs32 @ _f32(to_numpy(base_weight[c0:c1])).T if base_weight is not None
         else np.zeros((len(rows), c1 - c0), np.float32))
    for d in np.unique(idx):
        if d < 0:
            continue
        w = _f32(dequantize(*column_blocks(qweights[d], metas[d], ss[d], blk0, nblk)))
        m = idx == d
        y[m] += xs32[m] @ w
    return y


def sbmm_dense_f32(weights, x, rows_of):
    """The reference's torch check path on dequantised weights (sbmm_16bit_forloop,
    triteia/python/ops/matmul/sbmm.py:7-23) in fp32 on host tensors: for every delta d,
    y[rows_of[d]] += x[rows_of[d]] @ weights[d].  torch tensors in, torch tensor out; this is what
    the CPU timing legs of the benchmark run (all host threads, through torch.matmul)."""
    import torch

    y = torch.zeros(x.shape[0], weights[0].shape[1])
    for d, r in enumerate(rows_of):
        if len(r):
            y[r] += x[r] @ weights[d]
    return y


def lora(weights_a, weights_b, x, indices, base_weight=None, scale=1.0):
    """y[t] = x[t] @ base.T + scale * (x[t] @ A[idx[t]]) @ B[idx[t]]; A [M,H1,r], B [M,r,H2]."""
    x32 = _f32(x)
    h2 = np.asarray(weights_b).shape[2]
    y = x32 @ _f32(base_weight).T if base_weight is not None else np.zeros((x32.shape[0], h2), np.float32)
    idx = np.asarray(indices)
    for d in np.unique(idx):
        if d < 0:
            continue
        m = idx == d
        y[m] += scale * ((x32[m] @ _f32(weights_a[d])) @ _f32(weights_b[d]))
    return y


def bgmv(y, x, w_t_all, indices, layer_idx, scale):
    """One BGMV launch: y[i] += scale * W[idx[i], layer] @ x[i];  W [M, L, h_out, h_in]."""
    y = _f32(y).copy()
    x32 = _f32(x)
    for i, d in enumerate(np.asarray(indices)):
        y[i] += scale * (_f32(w_t_all[d, layer_idx]) @ x32[i])
    return y


def sgmv(y, x, weights, seg, layer_idx=0):
    """y[s[i]:s[i+1]] += x[s[i]:s[i+1]] @ W_i[layer];  weights: list of [L, d_in, d_out]."""
    y = _f32(y).copy()
    x32 = _f32(x)
    for i, w in enumerate(weights):
        a, b = int(seg[i]), int(seg[i + 1])
        if b > a:
            y[a:b] += x32[a:b] @ _f32(w[layer_idx])
    return y


def ldmm(indices, x, lwa, lwb, qweights, metas, ss, base_weight=None):
    """Index space: [0, M) = LoRA adapter, [M, M + D) = delta (M = number of adapters), -1 = base."""
    x32 = _f32(np.asarray(x).astype(np.float16))
    idx = np.asarray(indices).astype(np.int64)
    m_lora = np.asarray(lwa).shape[0]
    h2 = np.asarray(lwb).shape[2]
    y = x32 @ _f32(base_weight).T if base_weight is not None else np.zeros((x32.shape[0], h2), np.float32)
    for d in np.unique(idx):
        if d < 0:
            continue
        m = idx == d
        if d < m_lora:
            y[m] += (x32[m] @ _f32(lwa[d])) @ _f32(lwb[d])
        else:
            y[m] += x32[m] @ _f32(dequantize(qweights[d - m_lora], metas[d - m_lora], ss[d - m_lora]))
    return y


def row_rel_err(y, ref):
    """max_n |y - ref| / max_n |ref| per output row (the 1e-2 bound is stated on this)."""
    y = _f32(y)
    ref = _f32(ref)
    den = np.maximum(np.abs(ref).max(axis=-1), 1e-6)
    return np.abs(y - ref).max(axis=-1) / den


def mean_rel_err(y, ref):
    """mean|y - ref| / mean|ref| — the reference's own metric (tests/ops/test_matmul.py:18-22)."""
    return float(np.abs(_f32(y) - _f32(ref)).mean() / max(np.abs(_f32(ref)).mean(), 1e-12))
