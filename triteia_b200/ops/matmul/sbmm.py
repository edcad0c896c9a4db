"""Selective batched matmul (one token batch, one packed delta chosen per token).

Same names and signatures as triteia/python/ops/matmul/sbmm.py: `sbmm_16bit_forloop` :7,
`sbmm_4bit_2_4_forloop` :26, `sbmm_4bit_2_4_multilaunch` :54, `sbmm_4bit_2_4_native` :89.
The forloop and multilaunch variants keep the reference's structure (they are its slow
comparison paths); `native` is one router launch + one grouped-kernel launch with no host
synchronisation, accepts the indices in any order and honours per-group scales.
"""
import torch

from ... import _lib
from ..._lib import lib, ptr, stream_of, dev_of
from ...capi import mul_2_4, sbmm_2_4, sbmm_2_4_multilaunch
from ._base import base_gemm, base_or_zeros
from ._scratch import scratch


def _base(xs, base_weight, n_out):
    if base_weight is not None and not xs.is_cuda:
        return torch.matmul(xs, base_weight.t())       # sbmm_16bit_forloop also serves as a host-side check path
    return base_or_zeros(xs, base_weight, n_out)


def sbmm_16bit_forloop(weights, xs, indices, base_weight=None):
    """fp16 comparison path on uncompressed weights [D, K, N] (runs on any device)."""
    y = _base(xs, base_weight, weights.shape[2])
    for d in torch.unique(indices).tolist():
        if d != -1:
            m = indices == d
            y[m] += torch.matmul(xs[m], weights[d])
    return y


def sbmm_4bit_2_4_forloop(qweights, xs, metas, ss, indices, base_weight=None):
    y = _base(xs, base_weight, ss.shape[2])
    workspace = torch.zeros(y.shape[1] // 128 * 16, device=xs.device, dtype=torch.int32)
    for d in torch.unique(indices).tolist():
        if d != -1:
            m = indices == d
            inp = xs[m]
            out = torch.empty((inp.shape[0], y.shape[1]), dtype=xs.dtype, device=xs.device)
            mul_2_4(inp, qweights[d], metas[d], out, ss[d], workspace)
            y[m] += out
    return y


def _segments(indices):
    """(unique ids, starts, counts) of a grouped index vector, leading -1 run dropped."""
    uniq, counts = torch.unique_consecutive(indices, return_counts=True)
    starts = torch.cumsum(counts, 0) - counts
    keep = uniq != -1
    return uniq[keep].int(), starts[keep].int(), counts[keep].int()


def sbmm_4bit_2_4_multilaunch(qweights, xs, metas, ss, indices, base_weight=None):
    """indices must be grouped by delta id (as in the reference)."""
    y = _base(xs, base_weight, ss.shape[2])
    uniq, starts, counts = _segments(indices)
    if uniq.numel() == 0:
        return y
    workspace = torch.zeros(len(uniq), y.shape[1] // 8, device=xs.device, dtype=torch.int32)
    output = torch.zeros_like(y)
    sbmm_2_4_multilaunch(xs, qweights, metas, output, ss, uniq, workspace, starts, counts)
    y += output
    return y


def sbmm_indexed(xs, qweights, metas, ss, indices, y=None, index_offset=0):
    """Fused call: y[t] (+)= xs[t] @ delta[indices[t] - index_offset].  If `y` is given it is
    accumulated into, else a new tensor is returned (rows without a delta are zero)."""
    T, K = xs.shape
    D, G, N = ss.shape
    groupsize = -1 if G == 1 else K // G
    accumulate = y is not None
    if y is None:
        y = torch.empty(T, N, dtype=torch.float16, device=xs.device)
    if indices.dtype != torch.int32:
        indices = indices.to(torch.int32)
    nbytes = lib.trb_sbmm_indexed_scratch_bytes(T, K, D)
    buf = scratch(xs.device, nbytes)
    err = lib.trb_sbmm_indexed(ptr(xs), ptr(qweights), ptr(metas), ptr(ss), ptr(indices), ptr(y), T, N, K, D,
                               int(index_offset), groupsize, int(accumulate), ptr(buf), buf.numel(), dev_of(xs),
                               stream_of(xs))
    _lib.check(err, "sbmm_indexed")
    return y


class IndexedDeltaCall:
    """`sbmm_indexed(..., y=y)` in two steps, so that the router and the row gather (`plan`, which
    write nothing but the scratch) can run on another stream beside the kernel that produces y, and
    the grouped kernels (`run`) after both.  The scratch belongs to the stream that is current at
    construction; `plan` may be issued on any stream, the caller orders `run` after it."""

    def __init__(self, xs, qweights, metas, ss, indices, y, index_offset=0):
        T, K = xs.shape
        D, G, N = ss.shape
        if indices.dtype != torch.int32:
            indices = indices.to(torch.int32)
        self.t = (xs, qweights, metas, ss, indices, y)
        self.dims = (T, N, K, D, int(index_offset), -1 if G == 1 else K // G)
        self.buf = scratch(xs.device, lib.trb_sbmm_indexed_scratch_bytes(T, K, D))

    def _call(self, phase):
        xs, q, m, s, idx, y = self.t
        T, N, K, D, off, groupsize = self.dims
        err = lib.trb_sbmm_indexed_phase(ptr(xs), ptr(q), ptr(m), ptr(s), ptr(idx), ptr(y), T, N, K, D, off, groupsize,
                                         1, ptr(self.buf), self.buf.numel(), phase, dev_of(xs), stream_of(xs))
        _lib.check(err, "sbmm_indexed_phase")

    def plan(self):
        self._call(1)

    def run(self):
        self._call(2)


def sbmm_4bit_2_4_native(qweights, xs, metas, ss, indices, base_weight=None):
    if not xs.is_contiguous():
        xs = xs.contiguous()
    if base_weight is not None:
        y = base_gemm(xs, base_weight)
        return sbmm_indexed(xs, qweights, metas, ss, indices, y=y)
    return sbmm_indexed(xs, qweights, metas, ss, indices)


def sbmm_4bit_2_4_segments(qweights, xs, metas, ss, indices, base_weight=None):
    """The reference's split call sequence (torch routing prologue + `sbmm_2_4`), for callers
    that already hold grouped indices and want the legacy entry point."""
    y = _base(xs, base_weight, ss.shape[2])
    uniq, starts, counts = _segments(indices)
    if uniq.numel() == 0:
        return y
    workspace = torch.zeros(len(uniq), y.shape[1] // 8, device=xs.device, dtype=torch.int32)
    output = torch.zeros((xs.shape[0], ss.shape[2]), dtype=torch.float16, device=xs.device)
    sbmm_2_4(xs, qweights, metas, output, ss, uniq, workspace, starts, counts)
    y += output
    return y
