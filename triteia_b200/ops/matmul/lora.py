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


def lora_sgmv(weights_A, weights_B, x, indices, base_weight=None, layer_idx=0):
    """One adapter per contiguous token segment; indices grouped by id with the -1 run first.
    The segment pointer array is built on the device (the reference loops on the host with
    `.item()`, lora.py:63-78)."""
    y = _base(x, base_weight, weights_B.shape[2])
    M, _, rank = weights_A.shape
    ids = torch.arange(-1, M, device=x.device, dtype=indices.dtype)
    counts = (indices[:, None] == ids[None, :]).sum(0)           # [-1, 0, .., M-1]
    s = torch.cumsum(counts, 0).to(torch.int32)                   # s[i] = first row of adapter i
    wa = weights_A.unsqueeze(1)
    wb = weights_B.unsqueeze(1)
    step_a, step_b = wa.stride(0) * wa.element_size(), wb.stride(0) * wb.element_size()
    ar = torch.arange(M, device=x.device, dtype=torch.int64)
    wa_ptr = wa.data_ptr() + ar * step_a
    wb_ptr = wb.data_ptr() + ar * step_b
    add_lora_sgmv_cutlass(y, x, wa_ptr, wb_ptr, s, layer_idx, rank)
    return y
