"""Generate the golden fixtures under tests/golden/ from the reference's own Python code.

Run once where a checkout of the reference is at hand, with TRITEIA_REFERENCE pointing at it:

    TRITEIA_REFERENCE=<path of the checkout> python tests/golden/make_golden.py

The reference's Python host code is imported on CPU.  Three things are stubbed so
that it imports without a GPU: the `triteia_cuda` extension module, `pynvml`
(initialised at import time by triteia/python/configs/gpus/specs.py:1-3) and
`torch.Tensor.cuda` (hard-coded `.cuda()` calls at triteia/python/nn/linear.py:108 and
triteia/python/ops/utils/generator.py:51).  Only torch-on-CPU reference code runs:
the packer (nn/linear.py:79-141), the 2:4 compressor (ops/utils/sparsity.py:167-290),
`mask_creator` (sparsity.py:99-118), the routing prologue (ops/matmul/sbmm.py:94-123),
`sbmm_16bit_forloop` (sbmm.py:7-23), `lora_forloop` (ops/matmul/lora.py:4-20) and the
dispatch rule of `baseline_ldmm` (ops/matmul/ldmm.py:22-46), the GPTQ dequantiser
(utils/quant_utils.py:38-44) and the tensor-parallel chunking of the packer
(ops/utils/generator.py:126-176).

The fixtures travel with the repository; nothing at test time reads the reference.
"""
import os
import sys
import types

import numpy as np
import torch

REF = os.environ.get("TRITEIA_REFERENCE")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set TRITEIA_REFERENCE to a checkout of the reference")
OUT = os.path.dirname(os.path.abspath(__file__))


def import_reference():
    sys.path.insert(0, REF)
    sys.modules["triteia_cuda"] = types.ModuleType("triteia_cuda")
    nv = types.ModuleType("pynvml")
    nv.nvmlInit = lambda: None
    nv.nvmlDeviceGetHandleByIndex = lambda i: None
    nv.nvmlDeviceGetName = lambda h: "cpu"
    sys.modules["pynvml"] = nv
    torch.Tensor.cuda = lambda self, *a, **k: self
    import triteia.python.ops as ops  # noqa
    return ops


def routing_prologue(indices):
    """Lines 96 and 112-123 of ops/matmul/sbmm.py, run on CPU tensors."""
    unique_indices, counts = torch.unique_consecutive(indices, return_counts=True)
    unique_indices = unique_indices.int()
    counts = counts.int()
    first_nonnegative = torch.where(indices != -1)[0][0]
    if first_nonnegative > 0:
        unique_indices = unique_indices[1:]
        counts = counts[1:]
    start = torch.cat(
        (
            torch.tensor([first_nonnegative]),
            (torch.cumsum(counts, dim=0) + first_nonnegative)[:-1],
        )
    ).int()
    return unique_indices, start, counts


def main():
    ops = import_reference()
    from triteia.python.ops.utils.sparsity import (
        mask_creator,
        sparse_semi_structured_from_dense_cutlass,
        sparse_semi_structured_to_dense_cutlass,
    )

    out = {}
    # ---- packed deltas from the reference packer (per-channel scales) ----
    for name, (n_out, k_in, seed) in {
        "pack_a": (256, 128, 1),
        "pack_b": (512, 256, 2),
        "pack_c": (256, 384, 3),
    }.items():
        torch.manual_seed(seed)
        unc, q, s, meta = ops.gen_sparse_quant4_NT(n_out, k_in, groupsize=-1, device="cpu")
        out[f"{name}_uncompress"] = unc.numpy()
        out[f"{name}_q"] = q.numpy()
        out[f"{name}_s"] = s.numpy()
        out[f"{name}_meta"] = meta.numpy()

    # ---- batched deltas + sbmm_16bit_forloop on CPU (fp16 matmul) ----
    torch.manual_seed(10)
    unc, qs, ss, metas = ops.gen_batched_sparse_quant4_NT(4, 256, 128, device="cpu")
    xs = torch.randn(12, 128, dtype=torch.float16)
    idx = torch.tensor([-1, -1, 0, 0, 0, 1, 3, 3, 3, 3, 3, 3], dtype=torch.int32)
    y = ops.sbmm_16bit_forloop(unc, xs, idx, base_weight=None)
    base = (torch.randn(256, 128) * 0.02).half()
    yb = ops.sbmm_16bit_forloop(unc, xs, idx, base_weight=base)
    out.update(
        sbmm_unc=unc.numpy(), sbmm_q=qs.numpy(), sbmm_s=ss.numpy(), sbmm_meta=metas.numpy(),
        sbmm_x=xs.numpy(), sbmm_idx=idx.numpy(), sbmm_y=y.numpy(), sbmm_base=base.numpy(),
        sbmm_y_base=yb.numpy(),
    )

    # ---- routing prologue ----
    cases = {
        "route_a": [-1, -1, 0, 0, 0, 1, 3, 3, 3, 3, 3, 3],
        "route_b": [2, 2, 5, 7, 7, 7, 9],
        "route_c": [-1, 4, 4, 4, 4, 4, 4, 4, 4, 6],
        "route_d": [0, 1, 2, 3, 4, 5, 6, 7],
    }
    for name, v in cases.items():
        t = torch.tensor(v, dtype=torch.int32)
        u, st, c = routing_prologue(t)
        out[f"{name}_idx"] = t.numpy()
        out[f"{name}_unique"] = u.numpy()
        out[f"{name}_start"] = st.numpy()
        out[f"{name}_count"] = c.numpy()

    # ---- mask_creator ----
    torch.manual_seed(20)
    m_in = torch.randn(16, 32, dtype=torch.float16)
    out["mask_in"] = m_in.numpy()
    out["mask_out"] = mask_creator(m_in, 2, 4).numpy()

    # ---- 2:4 compressor round trip on int codes ----
    torch.manual_seed(21)
    dense = torch.randint(1, 16, (64, 64), dtype=torch.int32)
    dense = (dense * mask_creator(torch.randn(64, 64), 2, 4).int()).contiguous()
    sp, me = sparse_semi_structured_from_dense_cutlass(dense)
    back = sparse_semi_structured_to_dense_cutlass(sp, me)
    assert torch.equal(back, dense)
    out.update(comp_dense=dense.numpy(), comp_sparse=sp.numpy(), comp_meta=me.numpy())

    # ---- LoRA loop + ldmm dispatch rule (CPU fp16) ----
    torch.manual_seed(30)
    A, B = ops.gen_batched_lora_16_bit(3, 128, 256, 16, device="cpu")
    A = (A.float() / 128 ** 0.5).half()
    B = (B.float() / 4.0).half()
    lx = torch.randn(10, 128, dtype=torch.float16)
    lidx = torch.tensor([-1, 0, 0, 1, 1, 1, 2, 2, 2, 2], dtype=torch.int32)
    ly = ops.lora_forloop(A, B, lx, lidx)
    out.update(lora_A=A.numpy(), lora_B=B.numpy(), lora_x=lx.numpy(), lora_idx=lidx.numpy(), lora_y=ly.numpy())

    # baseline_ldmm's delta branch calls the CUDA extension, so its dispatch rule is
    # evaluated here with the torch references of both branches (ldmm.py:22-46).
    M = A.shape[0]
    didx = torch.tensor([-1, 0, 2, 2, 3, 3, 3, 4, 6, 6, 1, -1], dtype=torch.int32)
    dx = torch.randn(12, 128, dtype=torch.float16)
    yd = torch.zeros(12, 256, dtype=torch.float16)
    mask_l = (didx < M) & (didx != -1)
    mask_s = (didx >= M) & (didx != -1)
    yd[mask_l] = ops.lora_forloop(A, B, dx[mask_l], didx[mask_l].long())
    yd[mask_s] = ops.sbmm_16bit_forloop(unc, dx[mask_s], didx[mask_s] - M)
    out.update(ldmm_idx=didx.numpy(), ldmm_x=dx.numpy(), ldmm_y=yd.numpy())

    # ---- index distributions (numpy global seed, generator.py:90-102) ----
    import triteia.python.ops.utils.generator as gen
    orig_tensor = torch.tensor
    gen.torch.tensor = lambda data, dtype=None, device=None: orig_tensor(np.asarray(data), dtype=dtype)
    np.random.seed(5)
    out["dist_uniform"] = ops.generate_model_distribution("uniform", 64, 8).numpy()
    np.random.seed(5)
    out["dist_zipf"] = ops.generate_model_distribution("zipf:1.5", 64, 8).numpy()
    gen.torch.tensor = orig_tensor

    # ---- GPTQ-style checkpoint tensors -> dense weight (utils/quant_utils.py:38-44) ----
    from triteia.python.utils.quant_utils import dequantize_weight
    g = torch.Generator().manual_seed(40)
    gq = torch.randint(-2 ** 31, 2 ** 31 - 1, (8, 32), generator=g, dtype=torch.int64).to(torch.int32)
    gz = torch.full((1, 4), 0x77777777, dtype=torch.int32)
    gs = (torch.rand(1, 32, generator=g) * 0.01 + 0.001).half()
    out.update(gptq_qweight=gq.numpy(), gptq_qzeros=gz.numpy(), gptq_scales=gs.numpy(),
               gptq_dense=dequantize_weight(gq, gz, gs).numpy())

    # ---- tensor-parallel chunking of the packer (ops/utils/generator.py:126-176) ----
    from triteia.python.ops.utils.generator import torch_weight_to_sparse_marlin
    torch.manual_seed(41)
    lev = torch.randint(1, 8, (256, 512)) * (torch.randint(0, 2, (256, 512)) * 2 - 1)
    keep = mask_creator(torch.randn(512, 256), 2, 4).t()            # 2 of every 4 along the input features
    tp_scale = (torch.rand(1, 512) * 0.01 + 0.001).half()
    tp_w = (lev * keep).half() * tp_scale                             # [in, out]
    out.update(tp_weight=tp_w.numpy(), tp_scale=tp_scale.numpy())
    for how in ("column", "row"):
        qs_, ss_, ms_ = torch_weight_to_sparse_marlin(tp_w.clone(), tp_scale.clone(), tp_size=2, chunk_by=how)
        for i in range(2):
            out[f"tp_{how}_{i}_q"] = qs_[i].numpy()
            out[f"tp_{how}_{i}_s"] = ss_[i].numpy()
            out[f"tp_{how}_{i}_meta"] = ms_[i].numpy()

    path = os.path.join(OUT, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
