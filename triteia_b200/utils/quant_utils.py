"""GPTQ-style 4-bit checkpoint tensors -> dense weights, as the reference's converter needs them
(triteia/python/utils/quant_utils.py:6-44).  Vectorised: the reference unpacks row by row in a
Python loop."""
import torch


@torch.no_grad()
def unpack_4bit_to_32bit_signed(qweight, qzeros):
    """qweight int32 [in/8, out] (nibble i of a word = input row 8*word_row + i), qzeros int32
    [groups, out/8] -> (codes int8 [in, out], zero points + 1 int8 [groups, out]).
    Only symmetric checkpoints (every stored zero point == 7) are accepted, as in the reference
    (quant_utils.py:28-33)."""
    shifts = torch.arange(0, 32, 4, device=qweight.device, dtype=torch.int32)
    w = (qweight.unsqueeze(1) >> shifts.view(1, 8, 1)) & 0xF            # [in/8, 8, out]
    w = w.reshape(qweight.shape[0] * 8, qweight.shape[1]).to(torch.int8)
    z = (qzeros.unsqueeze(2) >> shifts.view(1, 1, 8)) & 0xF             # [groups, out/8, 8]
    z = z.reshape(qzeros.shape[0], qzeros.shape[1] * 8).to(torch.int8)
    if not torch.all(z == 7):
        raise ValueError(
            "Marlin kernel is compatible only with checkpoints using symmetric quantization."
            "Found non-symmetric quantization for the weight"
        )
    return w, z + 1


@torch.no_grad()
def dequantize_weight(qweight, qzeros, scales):
    """Dense weight [out, in] = ((code - zero) * scale) transposed; scales [groups, out]
    (quant_utils.py:38-44)."""
    w, z = unpack_4bit_to_32bit_signed(qweight, qzeros)
    group_size = w.shape[0] // scales.shape[0]
    s = scales.repeat_interleave(group_size, dim=0)
    z = z.repeat_interleave(group_size, dim=0)
    return ((w - z) * s).T
