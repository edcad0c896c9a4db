"""Checkpoint converter: a deltazip / GPTQ-style 4-bit state dict -> the packed 2:4 Sparse-Marlin
tensors the delta matmul path consumes, split for tensor parallelism and keyed
`{module}.{tp_rank}.{qweight,scales,meta}`.

Mirrors triteia/tools/converters/convert_deltazip.py:18-137:
  * every `X.qweight / X.qzeros / X.scales / X.g_idx` group is dequantised to fp16 [in, out];
  * q/k/v and gate/up of a layer are concatenated along the output features into
    `self_attn.qkv_proj` / `mlp.gate_up_proj` (positions from configs/models/llama.py) and split by
    output columns; `o_proj` / `down_proj` are split by input rows;
  * `embed_tokens` / `lm_head` are sliced by rows, uncompressed (`{module}.{tp_rank}.weight`);
  * any other tensor is not carried over (as in the reference).
The lossless (nvCOMP) input form of the reference is not supported here: that codec is outside
the delta matmul path.  Runs on whatever device the tensors are on; the packer is torch code.
"""
import argparse

import torch

from ..configs.models.llama import pack_modules, row_chunking_modules, uncompressed_row_chunking_modules
from ..ops.utils.generator import torch_weight_to_sparse_marlin
from ..utils.quant_utils import dequantize_weight


@torch.no_grad()
def convert_state_dict(tensors, tp_size, use_kernel=False):
    """tensors: {key: tensor} of the source checkpoint.  Returns the converted {key: tensor}.
    use_kernel: pack fp16 CUDA chunks with the packer kernel instead of the torch packer."""
    new_tensors = {}
    remaining = list(tensors.keys())
    modules = [k[: -len(".qweight")] for k in tensors if k.endswith(".qweight")]
    dense = {}
    for m in modules:
        w = dequantize_weight(tensors[m + ".qweight"], tensors[m + ".qzeros"], tensors[m + ".scales"])
        dense[m] = (w.to(torch.float16).t().contiguous(), tensors[m + ".scales"])       # [in, out], [groups, out]
        for suffix in (".qweight", ".qzeros", ".scales", ".g_idx"):
            if m + suffix in remaining:
                remaining.remove(m + suffix)

    def emit(name, qweights, scales, metas):
        for i, (q, s, meta) in enumerate(zip(qweights, scales, metas)):
            new_tensors[f"{name}.{i}.qweight"] = q
            new_tensors[f"{name}.{i}.scales"] = s
            new_tensors[f"{name}.{i}.meta"] = meta

    fused = {}
    for m in modules:
        src = next((k for k in pack_modules if m.endswith(k)), None)
        if src is not None:
            target, pos = pack_modules[src].split(":")
            fused.setdefault(m[: -len(src)] + target, []).append((int(pos), m))
        elif any(m.endswith(k) for k in row_chunking_modules):
            emit(m, *torch_weight_to_sparse_marlin(dense[m][0], dense[m][1], tp_size=tp_size, chunk_by="row", use_kernel=use_kernel))
    for name, parts in fused.items():
        parts.sort()
        weight = torch.cat([dense[m][0] for _, m in parts], dim=1)
        scales = torch.cat([dense[m][1] for _, m in parts], dim=1)
        emit(name, *torch_weight_to_sparse_marlin(weight, scales, tp_size=tp_size, chunk_by="column", use_kernel=use_kernel))
    for key in remaining:
        if any(k in key for k in uncompressed_row_chunking_modules) and key.endswith(".weight"):
            w = tensors[key]
            rows = w.shape[0]
            for i in range(tp_size):
                new_tensors[f"{key[: -len('.weight')]}.{i}.weight"] = w[i * rows // tp_size:(i + 1) * rows // tp_size, :]
    return new_tensors


def convert_model(ckpt, tp_size, save_path=None, device="cpu", lossless=False):
    """safetensors file in -> converted tensors (and a safetensors file out when save_path is given)."""
    if lossless:
        raise NotImplementedError("lossless (nvCOMP) checkpoints are not supported: decompress them first")
    from safetensors import safe_open
    from safetensors.torch import save_file

    tensors = {}
    with safe_open(ckpt, framework="pt", device=device) as f:
        for key in f.keys():
            tensors[key] = f.get_tensor(key)
    out = convert_state_dict(tensors, tp_size)
    if save_path:
        save_file({k: v.detach().cpu().clone().contiguous() for k, v in out.items()}, save_path)   # no shared storage in the file
    return out


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--tp-size", type=int, required=True)
    ap.add_argument("--save-path", required=True)
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--lossless", action="store_true")
    args = ap.parse_args()
    out = convert_model(args.ckpt, args.tp_size, args.save_path, device=args.device, lossless=args.lossless)
    print(f"wrote {len(out)} tensors to {args.save_path}")


if __name__ == "__main__":
    main()
