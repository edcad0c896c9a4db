"""1:1 shims over the extension, as triteia/python/capi/marlin.py (mul_2_4 :4, bmm_2_4 :23,
sbmm_2_4 :33, sbmm_2_4_multilaunch :67)."""
from .. import triteia_cuda


def mul_2_4(A, B, meta, C, s, workspace, thread_k=-1, thread_m=-1, sms=-1, max_par=16):
    """C[T, N] = A[T, K] @ dequant(B, meta, s): fp16 x (int4 + 2:4 sparsity), fp32 accumulation.

    A: fp16 activations [T, K]; B: int32 packed weights [K/32, 2N]; meta: int16 [N, K/16];
    C: fp16 output [T, N] (overwritten); s: fp16 scales [1, N] or [K/128, N];
    workspace: int32, at least N / 128 * max_par zeros (kept for call compatibility).
    """
    triteia_cuda.mul_2_4(A, B, meta, C, s, workspace, thread_k, thread_m, sms, max_par)


def bmm_2_4(A, B, meta, C, s, workspace, thread_k=-1, thread_m=-1, sms=-1, max_par=16):
    """One packed weight per request: C[b] = A[b] @ dequant(B[b], meta[b], s[b])."""
    triteia_cuda.bmm_2_4(A, B, meta, C, s, workspace, thread_k, thread_m, sms, max_par)


def sbmm_2_4(A, B, meta, C, s, indices, workspace, starts, counts, thread_k=-1, thread_n=-1, sms=-1, max_par=16):
    """Selective batched matmul: segment r = rows starts[r] .. starts[r] + counts[r] of A use
    delta indices[r]; one launch for all segments."""
    triteia_cuda.sbmm_2_4(A, B, meta, C, s, indices, workspace, starts, counts, thread_k, thread_n, sms, max_par)


def sbmm_2_4_multilaunch(A, B, meta, C, s, indices, workspace, starts, counts, thread_k=-1, thread_n=-1, sms=-1,
                         max_par=16):
    """Same result as sbmm_2_4 with one launch per segment."""
    triteia_cuda.sbmm_forloop(A, B, meta, C, s, indices, workspace, starts, counts, thread_k, thread_n, sms, max_par)
