"""Batched matmul with one packed weight per request — triteia/python/ops/matmul/bmm.py:6-35."""
import torch

from ...capi.marlin import bmm_2_4
from .sparse_low_precision import matmul_4bit_2_4


def bmm_4bit_2_4_forloop(qweights, xs, metas, ss):
    outputs = torch.zeros((xs.shape[0], xs.shape[1], ss.shape[2]), dtype=xs.dtype, device=xs.device)
    for i in range(xs.shape[0]):
        outputs[i] = matmul_4bit_2_4(qweights[i], xs[i], metas[i], ss[i])
    return outputs


def bmm_4bit_2_4(qweights, xs, metas, ss):
    """xs [B, 1, K], qweights [B, K/32, 2N], metas [B, N, K/16], ss [B, G, N] -> [B, 1, N]."""
    C = torch.empty((xs.shape[0], xs.shape[1], ss.shape[2]), dtype=xs.dtype, device=xs.device)
    workspace = torch.zeros(xs.shape[0] * max(ss.shape[2], ss.shape[1]), device=xs.device, dtype=torch.int32)
    bmm_2_4(xs, qweights, metas, C, ss, workspace)
    return C
