"""LoRA operators — same names and signatures as triteia/python/ops/matmul/lora.py
(`lora_forloop` :4, `lora_bgmv` :22, `lora_sgmv` :50)."""
import torch

from ... import _lib
from ..._lib import lib, ptr, stream_of, dev_of
from ...capi import add_lora_sgmv_cutlass
from ._base import base_or_zeros


def _base(x, base_weight, n_out):
    if base_weight is not None and not x.is_cuda:
        return torch.matmul(x, base_weight.t())        # lora_forloop also serves as a host-side check path
    return base_or_zeros(x, base_weight, n_out)


def lora_forloop(weights_A, weights_B, x, indices, base_weight=None):
    """torch comparison path: y[t] = base + (x[t] @ A[id]) @ B[id]; runs on any device."""
    y = _base(x, base_weight, weights_B.shape[2])
    for d in torch.unique(indices).tolist():
        if d != -1:
            m = indices == d
            y[m] += torch.matmul(torch.matmul(x[m], weights_A[d]), weights_B[d])
    return y


def lora_indexed(y, x, weights_A, weights_B, indices, scale=1.0):
    """In place: y[t] += scale * (x[t] @ A[id]) @ B[id] for id = indices[t] in [0, M); other ids
    leave the row alone.  A [M, H1, r], B [M, r, H2]; indices int32 or int64, any order."""
    if indices.dtype not in (torch.int32, torch.int64):
        indices = indices.to(torch.int32)
    M, H1, r = weights_A.shape
    err = lib.trb_lora_indexed(ptr(y), ptr(x), ptr(weights_A), ptr(weights_B), ptr(indices),
                               int(indices.dtype == torch.int64), x.shape[0], H1, weights_B.shape[2], r, M,
                               float(scale), _lib.dtype_tag(x.dtype), dev_of(x), stream_of(x))
    if err == _lib.ERR_KERN_SHAPE:
        raise RuntimeError(f"No suitable kernel. h_in={H1} h_out={weights_B.shape[2]} rank={r} dtype={x.dtype}")
    _lib.check(err, "lora_indexed")
    return y


def lora_bgmv(weights_A, weights_B, x, indices, base_weight=None, layer_idx=0, scale=1.0):
    """One adapter per token.  One launch on the natural layouts: no per-call transpose of the
    adapters, no gather / scatter of the rows (compare lora.py:33-47 of the reference)."""
    y = _base(x, base_weight, weights_B.shape[2])
    if not (weights_A.is_contiguous() and weights_B.is_contiguous() and x.is_contiguous()):
        weights_A, weights_B, x = weights_A.contiguous(), weights_B.contiguous(), x.contiguous()
    return lora_indexed(y, x, weights_A, weights_B, indices, scale)


def sgmv_stacked(y, x, weights, seg, accumulate=True, max_rows=0):
    """In place: y[seg[i]:seg[i+1]] (+)= x[seg[i]:seg[i+1]] @ weights[i]; weights [S, d_in, d_out]
    contiguous, seg int32 [S + 1] on the device."""
    S, d_in, d_out = weights.shape
    err = lib.trb_sgmv_stacked(ptr(y), ptr(x), ptr(weights), ptr(seg), S, x.shape[0], d_in, d_out, int(max_rows),
                               int(accumulate), _lib.dtype_tag(x.dtype), dev_of(x), stream_of(x))
    if err == _lib.ERR_KERN_SHAPE:
        raise RuntimeError(f"No suitable kernel. d_in={d_in} d_out={d_out} problems={S} dtype={x.dtype}")
    _lib.check(err, "sgmv_stacked")
    return y


def lora_sgmv(weights_A, weights_B, x, indices, base_weight=None, layer_idx=0):
    """One adapter per contiguous token segment; indices grouped by id with the -1 run first.
    The segment offsets are built on the device (the reference loops on the host with `.item()`,
    lora.py:63-78), and shrink and expand are two launches of one tensor-core kernel on the stacked
    weights as they are (no per-problem pointer arrays; the reference's two grouped GEMMs go through
    `add_lora_sgmv_cutlass`, triteia/python/capi/punica.py:4-32, which stays available in capi)."""
    y = _base(x, base_weight, weights_B.shape[2])
    M, _, rank = weights_A.shape
    ids = torch.arange(-1, M, device=x.device, dtype=indices.dtype)
    counts = (indices[:, None] == ids[None, :]).sum(0)           # [-1, 0, .., M-1]
    s = torch.cumsum(counts, 0).to(torch.int32)                   # s[i] = first row of adapter i
    if not (weights_A.is_contiguous() and weights_B.is_contiguous() and x.is_contiguous()):
        weights_A, weights_B, x = weights_A.contiguous(), weights_B.contiguous(), x.contiguous()
    if rank % 8 != 0 or x.shape[1] % 8 != 0 or y.shape[1] % 8 != 0 or M > 1024:
        wa, wb = weights_A.unsqueeze(1), weights_B.unsqueeze(1)   # shapes the tensor-core kernel does not take
        ar = torch.arange(M, device=x.device, dtype=torch.int64)
        add_lora_sgmv_cutlass(y, x, wa.data_ptr() + ar * (wa.stride(0) * wa.element_size()),
                              wb.data_ptr() + ar * (wb.stride(0) * wb.element_size()), s, layer_idx, rank)
        return y
    v = torch.empty(x.shape[0], rank, dtype=x.dtype, device=x.device)
    sgmv_stacked(v, x, weights_A, s, accumulate=False)
    sgmv_stacked(y, v, weights_B, s, accumulate=True)
    return y
