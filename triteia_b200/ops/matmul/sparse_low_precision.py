"""matmul_4bit_2_4 — same signature as triteia/python/ops/matmul/sparse_low_precision.py:5-24."""
import torch

from ...capi import mul_2_4


def matmul_4bit_2_4(qweight, x, meta, s):
    """fp16 activations x [..., K] times one packed (int4, 2:4 sparse) weight.

    qweight int32 [K/32, 2N], meta int16 [N, K/16], s fp16 [1, N] or [K/128, N].
    Returns fp16 [..., N].
    """
    C = torch.empty((x.shape[:-1] + (s.shape[1],)), dtype=x.dtype, device=x.device)
    workspace = torch.zeros(s.shape[1], dtype=torch.int32, device=x.device)
    mul_2_4(x.reshape(-1, x.shape[-1]), qweight, meta, C.view(-1, C.shape[-1]), s, workspace)
    return C
