"""sparse_low_precision_linear — the module of triteia/python/nn/linear.py:18-141: buffers
`qweight`, `meta`, `scale`, `workspace`, `forward(x)` through `mul_2_4`, and `pack`."""
import torch
import torch.nn as nn

from ..capi import mul_2_4
from ..ops.utils.sparsity import pack_2_4


class sparse_low_precision_linear(nn.Module):
    def __init__(self, infeatures, outfeatures, groupsize=-1):
        super().__init__()
        assert groupsize in [-1, 128], f"Group size must be -1 or 128, got {groupsize}"
        assert infeatures % 128 == 0, f"Input features must be a multiple of 128, got {infeatures}"
        assert outfeatures % 256 == 0, f"Output features must be a multiple of 256, got {outfeatures}"
        self.infeatures = infeatures
        self.outfeatures = outfeatures
        self.groupsize = infeatures if groupsize == -1 else groupsize
        groups = infeatures // self.groupsize
        self.register_buffer("qweight", torch.empty((infeatures // 32, outfeatures * 2), dtype=torch.int32))
        self.register_buffer("meta", torch.empty((outfeatures, infeatures // 16), dtype=torch.int16))
        self.register_buffer("scale", torch.empty((groups, outfeatures), dtype=torch.float16))
        self.register_buffer("workspace", torch.zeros(outfeatures // 128 * 16, dtype=torch.int32))

    def forward(self, x):
        C = torch.empty(x.shape[:-1] + (self.outfeatures,), dtype=x.dtype, device=x.device)
        mul_2_4(x.reshape(-1, x.shape[-1]), self.qweight, self.meta, C.view(-1, C.shape[-1]), self.scale,
                self.workspace)
        return C

    def pack(self, weight, scales, trans=True):
        """weight fp16 [infeatures, outfeatures], scales fp16 [groups, outfeatures] (logical
        order).  Fills qweight / meta / scale.  Only the transposed (`trans=True`) weight
        layout of the reference is a 2:4 format; it is the only one supported."""
        if weight.dtype != torch.half:
            raise ValueError("Only `torch.half` weights are supported.")
        if not trans:
            raise ValueError("only the 2:4 (trans=True) layout is supported")
        # The torch packer, on whatever device the tensors are: where a group of four holds fewer than
        # two non-zeros its choice of the stored zero follows torch's sort, as the reference's does;
        # pack_2_4_cuda (one kernel) encodes the same weights but may pick another zero.
        q, s, meta = pack_2_4(weight, scales)
        self.qweight.copy_(q)
        self.scale.copy_(s)
        self.meta.copy_(meta)
