"""LoRA shims, as triteia/python/capi/punica.py (add_lora_sgmv_cutlass :4, add_lora_bgmv :34)."""
import torch

from .. import triteia_cuda


def add_lora_sgmv_cutlass(y, x, wa_ptr, wb_ptr, s, layer_idx, lora_rank):
    """y[s[i]:s[i+1]] += x[s[i]:s[i+1]] @ deref(wa_ptr[i]) @ deref(wb_ptr[i]).

    y [B, H2] (in place), x [B, H1]; wa_ptr / wb_ptr int64 [S] device pointers to
    [num_layers, H1, R] / [num_layers, R, H2]; s int32 [S + 1] with s[0] == 0, s[-1] == B.
    """
    tmp = torch.empty((triteia_cuda.sgmv_cutlass_tmp_size(wa_ptr.size(0)),), dtype=torch.uint8, device=x.device)
    v = torch.zeros((x.size(0), lora_rank), dtype=x.dtype, device=x.device)
    triteia_cuda.sgmv_cutlass(v, x, wa_ptr, s, tmp, layer_idx)
    triteia_cuda.sgmv_cutlass(y, v, wb_ptr, s, tmp, layer_idx)


def add_lora_bgmv(y, x, wa_T_all, wb_T_all, indicies, layer_idx, scale):
    """y[i] += x[i] @ wa_T_all[idx[i], layer].T @ wb_T_all[idx[i], layer].T * scale.

    wa_T_all [M, L, R, H1], wb_T_all [M, L, H2, R], indicies int64 [B].
    """
    r = wb_T_all.size(-1)
    tmp = torch.zeros((x.size(0), r), dtype=x.dtype, device=x.device)
    triteia_cuda.dispatch_bgmv(tmp, x, wa_T_all, indicies, layer_idx, 1.0)
    triteia_cuda.dispatch_bgmv(y, tmp, wb_T_all, indicies, layer_idx, scale)
