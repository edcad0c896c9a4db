"""Synthetic inputs for the delta matmul path: quantise + prune + pack, LoRA pairs, index
distributions, tensor-parallel chunking.

Same call signatures and (for the same torch / numpy seeds on the same device) the same
results as the reference's triteia/python/ops/utils/generator.py: `gen_lora_16_bit` :7,
`gen_batched_lora_16_bit` :12, `gen_sparse_quant4_NT` :24-69, `gen_batched_sparse_quant4_NT`
:72-87, `generate_model_distribution` :90-102, `fp16_to_sparse` :105,
`torch_weight_to_sparse_marlin` :126-176.  Differences, all additive:
  * `groupsize=128` works (the reference raises for any groupsize other than -1);
  * `device` may be "cpu";
  * `generate_model_distribution` accepts `device=` and `rng=` and the extra law
    "true-zipf:a" (p proportional to rank**-a over the delta ids, no -1); the name "zipf:a"
    keeps the reference's law, which weights id j by (j + 2)**(+a) and includes -1;
  * `random_packed_deltas` draws valid packed tensors directly (benchmark-sized inputs).
"""
import numpy as np
import torch

from .sparsity import mask_creator, pack_2_4, pack_2_4_cuda


def gen_lora_16_bit(m, n, rank, device="cuda"):
    A = torch.randn((m, rank), dtype=torch.float16, device=device)
    B = torch.randn((rank, n), dtype=torch.float16, device=device)
    return A, B


def gen_batched_lora_16_bit(b, m, n, rank, device="cuda"):
    pairs = [gen_lora_16_bit(m, n, rank, device) for _ in range(b)]
    return torch.stack([p[0] for p in pairs]), torch.stack([p[1] for p in pairs])


def gen_sparse_quant4_NT(m, k, groupsize=-1, device="cuda", prune_n=2, prune_m=4):
    """m = output features, k = input features.

    Returns (uncompress fp16 [k, m], qweight int32 [k/32, 2m], scales fp16 [G, m],
    meta int16 [m, k/16]) with G = 1 (groupsize -1) or k / groupsize.
    """
    w = torch.randn((m, k), dtype=torch.half, device=device).t()  # [k, m]
    g = 1 if groupsize == -1 else k // groupsize
    rows = k // g
    s = w.reshape(g, rows, m).abs().amax(dim=1) * (2 / 15)  # [g, m]
    s_rows = s.repeat_interleave(rows, dim=0) if g > 1 else s
    codes = torch.clamp(torch.round(w / s_rows).int() + 8, 0, 15)
    ref = (codes - 8).half() * s_rows
    # The reference prunes on the magnitude of the unsigned codes (generator.py:51).
    mask = mask_creator(codes.t(), n=prune_n, m=prune_m).bool()
    uncompress = (mask * ref.t()).t()
    q, s_stored, meta = pack_2_4(uncompress, s)
    return uncompress, q, s_stored, meta


def gen_batched_sparse_quant4_NT(b, m, n, groupsize=-1, device="cuda:0"):
    items = [gen_sparse_quant4_NT(m, n, groupsize=groupsize, device=device) for _ in range(b)]
    unc, qs, ss, metas = (torch.stack([it[i] for it in items]) for i in range(4))
    return unc, qs, ss, metas


def generate_model_distribution(distribution, num_queries, num_models, device="cuda", rng=None):
    rnd = np.random if rng is None else rng
    ids = list(range(-1, num_models))
    if distribution == "uniform":
        models = rnd.choice(ids, num_queries)
    elif distribution == "distinct":
        models = ids
    elif distribution.startswith("zipf"):
        alpha = float(distribution.split(":")[1])
        assert alpha > 1, "alpha must be greater than 1"
        probs = np.array([i ** alpha for i in range(1, len(ids) + 1)], dtype=np.float64)
        models = rnd.choice(ids, num_queries, p=probs / probs.sum())
    elif distribution.startswith("true-zipf"):
        alpha = float(distribution.split(":")[1])
        probs = np.arange(1, num_models + 1, dtype=np.float64) ** (-alpha)
        models = rnd.choice(np.arange(num_models), num_queries, p=probs / probs.sum())
    else:
        raise ValueError(f"unknown distribution {distribution!r}")
    return torch.tensor(np.asarray(models), dtype=torch.int32, device=device)


def fp16_to_sparse(weights, scale, device="cuda"):
    """weights fp16 [k, m], scale fp16 [1, m] -> (weights, qweight, scales, meta)."""
    q, s, meta = pack_2_4(weights.to(device), scale.to(device))
    return weights, q, s, meta


@torch.no_grad()
def torch_weight_to_sparse_marlin(weight, scale, tp_size=1, chunk_by="column", use_kernel=False):
    """weight [in, out], scale [1, out] -> per tensor-parallel chunk lists (qweights, scales, metas).

    "column" splits the output features (each chunk keeps its slice of the scales), "row"
    splits the input features (every chunk keeps all scales).  use_kernel: pack CUDA fp16 chunks
    with the packer kernel (same weights; a group of four with fewer than two non-zeros may store a
    different one of its zeros than the torch packer does).
    """
    assert chunk_by in ["column", "row"], "chunk_by must be either 'column' or 'row'"
    assert weight.dim() == 2, "weight must be a 2D tensor"
    assert weight.size(0) % tp_size == 0, "out_features must be divisible by tp_size"
    assert weight.size(1) == scale.size(1), "out_features of weight and scale must match"
    qweights, scales, metas = [], [], []
    for i in range(tp_size):
        if chunk_by == "column":
            lo, hi = i * weight.size(1) // tp_size, (i + 1) * weight.size(1) // tp_size
            w_i, s_i = weight[:, lo:hi], scale[:, lo:hi]
        else:
            lo, hi = i * weight.size(0) // tp_size, (i + 1) * weight.size(0) // tp_size
            w_i, s_i = weight[lo:hi, :], scale
        if use_kernel and w_i.is_cuda and w_i.dtype == torch.float16 and s_i.dtype == torch.float16:
            q, s, meta = pack_2_4_cuda(w_i.contiguous(), s_i.contiguous())     # one kernel instead of ~20 torch ops
        else:
            q, s, meta = pack_2_4(w_i.contiguous(), s_i.contiguous())
        qweights.append(q.contiguous())
        scales.append(s.contiguous())
        metas.append(meta.contiguous())
    return qweights, scales, metas


def random_packed_deltas(num, k, n, groupsize=-1, device="cuda", seed=0, scale_lo=0.001, scale_hi=0.01):
    """Draw `num` valid packed deltas directly: uniform non-zero levels in [-7, 7] at two
    uniformly chosen positions of every four along K, scales ~ U(scale_lo, scale_hi).

    Returns (qweights int32 [num, k/32, 2n], metas int16 [num, n, k/16], scales fp16 [num, G, n]).
    Every delta has its own memory; nothing is aliased.
    """
    from .sparsity import compress_2_4, pack_codes, store_scales

    gen = torch.Generator(device=device).manual_seed(seed)
    g = 1 if groupsize == -1 else k // groupsize
    qs = torch.empty(num, k // 32, 2 * n, dtype=torch.int32, device=device)
    metas = torch.empty(num, n, k // 16, dtype=torch.int16, device=device)
    ss = torch.empty(num, g, n, dtype=torch.float16, device=device)
    pairs = torch.tensor([[0, 1], [0, 2], [0, 3], [1, 2], [1, 3], [2, 3]], device=device)
    for d in range(num):
        which = pairs[torch.randint(0, 6, (n, k // 4), generator=gen, device=device)]  # [n, k/4, 2]
        lev = torch.randint(1, 8, (n, k // 4, 2), generator=gen, device=device)
        sign = torch.randint(0, 2, (n, k // 4, 2), generator=gen, device=device) * 2 - 1
        codes = torch.zeros(n, k // 4, 4, dtype=torch.int32, device=device)
        codes.scatter_(2, which, (lev * sign + 8).to(torch.int32))
        comp, meta = compress_2_4(codes.reshape(n, k))
        qs[d] = pack_codes(comp)
        metas[d] = meta
        s = torch.rand(g, n, generator=gen, device=device) * (scale_hi - scale_lo) + scale_lo
        ss[d] = store_scales(s.to(torch.float16))
    return qs, metas, ss
