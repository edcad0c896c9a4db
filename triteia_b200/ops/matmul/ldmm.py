"""ldmm: per token, base GEMM plus either a LoRA adapter or a packed delta, chosen by one index
vector — same signatures as triteia/python/ops/matmul/ldmm.py (`baseline_ldmm` :8, `ldmm` :51).

Index space (ldmm.py:54-59 of the reference): [0, M) = LoRA adapter, [M, M + D) = delta,
-1 = base only, with M = LwA.shape[0].
"""
import torch

from ._base import base_gemm, base_or_zeros as _base, lora_shrink_rows
from .lora import lora_forloop, lora_indexed
from .sbmm import IndexedDeltaCall, sbmm_4bit_2_4_forloop, sbmm_indexed

_side_streams = {}


def _side_stream(device):
    """One extra stream per device for the part of ldmm that can run beside the base product."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


def baseline_ldmm(indices, x, LwA, LwB, DeltaW, metas, ss, base_weight=None, debug=False):
    """Comparison path built from the per-id loops (gathers and scatters through masks)."""
    x_ = x.to(torch.float16)
    y = _base(x_, base_weight, LwB.shape[2])
    M = LwA.shape[0]
    mask_lora = (indices < M) & (indices != -1)
    mask_sbmm = (indices >= M) & (indices != -1)
    if bool(mask_lora.any()):
        y[mask_lora] += lora_forloop(LwA.to(torch.float16), LwB.to(torch.float16), x_[mask_lora], indices[mask_lora])
    if bool(mask_sbmm.any()):
        y[mask_sbmm] += sbmm_4bit_2_4_forloop(DeltaW, x_[mask_sbmm], metas, ss, indices[mask_sbmm] - M)
    return y.to(x.dtype)


def ldmm(indices, x, LwA, LwB, DeltaW, metas, ss, base_weight=None, debug=False):
    """No library GEMM, no host synchronisation, no masks.  With a base weight: the LoRA shrink
    writes every token's rank-r vector into the column block of its adapter, and ONE tensor-core
    kernel produces base + LoRA in one accumulator (the expand is extra K of the same product) and
    writes y once; the delta kernel then adds its rows.  Without a base weight the indexed LoRA
    kernel runs alone.  Both parts read the one index vector: the LoRA side skips ids outside
    [0, M), the router of the delta kernel skips ids outside [M, M + D).  Any token order."""
    x_ = x.to(torch.float16)
    if not x_.is_contiguous():
        x_ = x_.contiguous()
    M = LwA.shape[0]
    idx = indices if indices.dtype == torch.int32 else indices.to(torch.int32)
    has_delta = DeltaW is not None and DeltaW.shape[0] > 0
    if base_weight is not None and M > 0 and has_delta and x_.shape[0] > 0:
        # Router and row gather of the delta part need x and the ids only: they run on a side stream
        # while this stream does the LoRA shrink and the base + LoRA product; the grouped kernels, which
        # add into y, follow the join.  (Captured in a CUDA graph this is a fork and a join.)
        A16, B16 = LwA.to(torch.float16).contiguous(), LwB.to(torch.float16).contiguous()
        N = B16.shape[2]
        y = torch.empty(x_.shape[0], N, dtype=torch.float16, device=x_.device)
        call = IndexedDeltaCall(x_, DeltaW, metas, ss, idx, y, index_offset=M)
        cur, side = torch.cuda.current_stream(x_.device), _side_stream(x_.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            call.plan()
        v = lora_shrink_rows(x_, A16, idx)
        base_gemm(x_, base_weight.to(torch.float16), lora_v=v, lora_b=B16.view(M * B16.shape[1], N), out=y)
        cur.wait_stream(side)
        call.run()
        return y.to(x.dtype)
    if base_weight is not None and M > 0:
        A16, B16 = LwA.to(torch.float16).contiguous(), LwB.to(torch.float16).contiguous()
        v = lora_shrink_rows(x_, A16, idx)
        y = base_gemm(x_, base_weight.to(torch.float16), lora_v=v, lora_b=B16.view(M * B16.shape[1], B16.shape[2]))
    else:
        y = _base(x_, base_weight, LwB.shape[2])
        if M > 0:
            lora_indexed(y, x_, LwA.to(torch.float16).contiguous(), LwB.to(torch.float16).contiguous(), idx)
    if has_delta:
        sbmm_indexed(x_, DeltaW, metas, ss, idx, y=y, index_offset=M)
    return y.to(x.dtype)
