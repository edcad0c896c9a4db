"""The base product that opens every operator of the path: y = x @ base_weight.t().

The reference calls torch.matmul here (triteia/python/ops/matmul/sbmm.py:90-93, ldmm.py:72-76,
lora.py:5-9).  This module calls the library's own tensor-core kernel instead (trb_base_gemm), which
can also take the LoRA expand into the same accumulator, so that y is written once.
"""
import torch

from ... import _lib
from ..._lib import lib, ptr, stream_of, dev_of


def base_gemm(x, base_weight, lora_v=None, lora_b=None, out=None, accumulate=False):
    """x [T, K], base_weight [N, K] (fp16 or bf16, contiguous) -> y [T, N] = x @ base_weight.t()
    (+ lora_v [T, Kv] @ lora_b [Kv, N]).  `out` with accumulate=True adds into an existing y."""
    if not x.is_contiguous():
        x = x.contiguous()
    if not base_weight.is_contiguous():
        base_weight = base_weight.contiguous()
    if base_weight.dtype != x.dtype:
        base_weight = base_weight.to(x.dtype)
    T, K = x.shape
    N = base_weight.shape[0]
    y = out if out is not None else torch.empty(T, N, dtype=x.dtype, device=x.device)
    kv = 0 if lora_v is None else lora_v.shape[1]
    err = lib.trb_base_gemm(ptr(x), ptr(base_weight), ptr(y), T, N, K, ptr(lora_v), ptr(lora_b), kv, int(accumulate),
                            _lib.dtype_tag(x.dtype), dev_of(x), stream_of(x))
    if err in (_lib.ERR_PROB_SHAPE, _lib.ERR_KERN_SHAPE):
        raise RuntimeError(f"No suitable kernel. base product K={K} N={N} dtype={x.dtype} "
                           "(K must be a multiple of 64, N a multiple of 8)")
    _lib.check(err, "base_gemm")
    return y


def base_or_zeros(x, base_weight, n_out):
    if base_weight is not None:
        return base_gemm(x, base_weight)
    return torch.zeros(x.shape[0], n_out, dtype=x.dtype, device=x.device)


def lora_shrink_rows(x, weights_A, indices, scale=1.0):
    """V [T, M * r] fp16: row t holds scale * x[t] @ A[id] in the column block of id =
    indices[t] and zeros elsewhere (ids outside [0, M) give a zero row)."""
    M, H1, r = weights_A.shape
    cols = M * r          # exactly the rows of the stacked expand matrices: the kernel pads by TMA zero fill
    v = torch.empty(x.shape[0], cols, dtype=torch.float16, device=x.device)
    if indices.dtype not in (torch.int32, torch.int64):
        indices = indices.to(torch.int32)
    err = lib.trb_lora_shrink_rows(ptr(v), ptr(x), ptr(weights_A), ptr(indices), int(indices.dtype == torch.int64),
                                   x.shape[0], H1, r, M, cols, float(scale), dev_of(x), stream_of(x))
    if err == _lib.ERR_KERN_SHAPE:
        raise RuntimeError(f"No suitable kernel. h_in={H1} rank={r}")
    _lib.check(err, "lora_shrink_rows")
    return v
