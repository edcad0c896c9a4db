"""2:4 pruning mask and the packed int4 + 2:4 delta format (producer side).

Mirrors the interface of the reference's triteia/python/ops/utils/sparsity.py
(`mask_creator` :99-118, the CUTLASS-style compressor :167-290 and the metadata reorder
:134-161) and of the packer triteia/python/nn/linear.py:79-141, but builds the packed
tensors with closed-form gathers instead of reshape/permute chains, so that it runs on
any torch device (the benchmarks pack on the GPU).

Wire format, for a delta with K input and N output features:
  qweight int32 [K/32, 2N]  one row per 32-K slab (16 compressed rows).  Word w of a row
                            belongs to 64-column block w // 128, lane i = (w % 128) // 4,
                            register j = w % 4; nibble p holds output column
                            64*blk + 8*(i // 4) + 4*((p % 4) // 2) + j and compressed row
                            2*(i % 4) + (p >= 4) + 8*(p % 2) of the slab.
  meta    int16 [N, K/16]   nibble q of nominal element (n, c) describes dense positions
                            16c + 4q .. +3: low 2 bits = first kept position, high 2 bits =
                            second.  Physical order: see `meta_physical_offsets`.
  scales  fp16  [1, N]      per-channel, natural order;  or [K/g, N] per group of g dense
                            K positions with each 8 columns stored as 0,4,1,5,2,6,3,7.
"""
import torch

SCALE_GROUP_ORDER = (0, 4, 1, 5, 2, 6, 3, 7)


def mask_creator(x: torch.Tensor, n: int = 2, m: int = 4):
    """0/1 mask keeping the `n` largest-magnitude entries of every `m` consecutive elements."""
    if x.numel() % m != 0:
        raise ValueError(f"Tensor of size {x.shape} can't be evenly divided into {m} groups")
    mag = x.detach().abs().reshape(x.numel() // m, m)
    drop = torch.argsort(mag, dim=1)[:, : int(m - n)]
    keep = torch.ones(mag.shape, device=mag.device)
    return keep.scatter_(dim=1, index=drop, value=0).reshape(x.shape)


def _selection_table(device):
    """For each of the 16 non-zero patterns (bit i set = element i of the group is non-zero):
    positions of the two stored elements.  Same truth table as sparsity.py:205-244."""
    rows = []
    for pat in range(16):
        m0, m1, m3 = bool(pat & 1), bool(pat & 2), bool(pat & 8)
        e0, e1, e2 = m0 and m1, (not m0) and m1, (not m0) and (not m1)
        first = int(e1) | (int(e2) << 1)
        second = int(e0 or e2 or m3) | (int(e1 or not m1) << 1)
        rows.append((first, second))
    return torch.tensor(rows, dtype=torch.int64, device=device)


def meta_physical_offsets(n_rows, n_cols, device):
    """Flat int16 offset of every nominal metadata element [n_rows, n_cols]."""
    r = torch.arange(n_rows, device=device)[:, None].expand(n_rows, n_cols)
    c = torch.arange(n_cols, device=device)[None, :].expand(n_rows, n_cols)
    dst = (r // 64) * 64 + (r % 2) * 2 + (r % 8) // 4 + ((r % 32) % 4) // 2 * 32 + ((r % 64) // 8) * 4
    tr = ((dst % 2 == 0) & (c % 2 == 1)).to(torch.int64)
    bl = ((dst % 2 == 1) & (c % 2 == 0)).to(torch.int64)
    dst = dst + tr - bl
    c = c - tr + bl
    return (c // 2) * n_rows * 2 + dst * 2 + c % 2


def compress_2_4(codes_nk: torch.Tensor):
    """codes_nk integer [N, K], zero where pruned.  Returns (compressed [N, K/2] same dtype,
    meta int16 [N, K/16] in physical order)."""
    n, k = codes_nk.shape
    if n % 32 != 0 or k % 16 != 0:
        raise RuntimeError(f"compress_2_4 needs N % 32 == 0 and K % 16 == 0, got {n}x{k}")
    dev = codes_nk.device
    g = codes_nk.reshape(n, k // 4, 4)
    nz = (g != 0).to(torch.int64)
    pat = nz[..., 0] | (nz[..., 1] << 1) | (nz[..., 2] << 2) | (nz[..., 3] << 3)
    sel = _selection_table(dev)[pat]  # [N, K/4, 2]
    comp = torch.gather(g, 2, sel).reshape(n, k // 2)
    nib = (sel[..., 0] | (sel[..., 1] << 2)).reshape(n, k // 16, 4)
    nominal = nib[..., 0] | (nib[..., 1] << 4) | (nib[..., 2] << 8) | (nib[..., 3] << 12)
    nominal = torch.where(nominal >= 32768, nominal - 65536, nominal).to(torch.int16)
    phys = torch.empty(n * (k // 16), dtype=torch.int16, device=dev)
    phys[meta_physical_offsets(n, k // 16, dev).reshape(-1)] = nominal.reshape(-1)
    return comp, phys.reshape(n, k // 16)


def pack_codes(comp_nk2: torch.Tensor):
    """compressed codes [N, K/2] (0..15) -> qweight int32 [K/32, 2N]."""
    n, kh = comp_nk2.shape
    dev = comp_nk2.device
    w = torch.arange(2 * n, device=dev)
    blk, lane, j = w // 128, (w % 128) // 4, w % 4
    src = comp_nk2.t().contiguous().to(torch.int64).reshape(kh // 16, 16, n)
    q = torch.zeros(kh // 16, 2 * n, dtype=torch.int64, device=dev)
    for p in range(8):
        col = 64 * blk + 8 * (lane // 4) + 4 * ((p % 4) // 2) + j
        crow = 2 * (lane % 4) + (1 if p >= 4 else 0) + 8 * (p % 2)
        q |= src[:, crow, col] << (4 * p)
    q = torch.where(q >= 2 ** 31, q - 2 ** 32, q)
    return q.to(torch.int32)


def store_scales(s_logical: torch.Tensor):
    """Logical scales [G, N] -> stored order (identity for G == 1)."""
    if s_logical.shape[0] == 1:
        return s_logical.contiguous()
    g, n = s_logical.shape
    order = torch.tensor(SCALE_GROUP_ORDER, device=s_logical.device)
    return s_logical.reshape(g, n // 8, 8)[:, :, order].reshape(g, n).contiguous()


def pack_2_4(weight_kn: torch.Tensor, scales: torch.Tensor):
    """fp16 weight [K, N] (already 2:4 along K or not: the two largest magnitudes of every
    four K positions are kept) and logical scales [G, N], G = 1 or K/groupsize.

    Returns (qweight int32 [K/32, 2N], stored scales fp16 [G, N], meta int16 [N, K/16]).
    """
    k, n = weight_kn.shape
    if k % 128 != 0 or n % 256 != 0:
        raise ValueError(f"pack_2_4 needs K % 128 == 0 and N % 256 == 0, got K={k}, N={n}")
    g = scales.shape[0]
    if k % g != 0:
        raise ValueError(f"K={k} is not divisible into {g} scale groups")
    mask = mask_creator(weight_kn.t(), 2, 4).bool()  # [N, K]
    s_rows = scales if g == 1 else scales.repeat_interleave(k // g, dim=0)
    codes = torch.clamp(torch.round(weight_kn / s_rows).int() + 8, 0, 15)  # [K, N]
    codes_nk = (mask * codes.t()).contiguous()
    comp, meta = compress_2_4(codes_nk)
    return pack_codes(comp), store_scales(scales.to(torch.float16)), meta


def pack_2_4_cuda(weight_kn: torch.Tensor, scales: torch.Tensor):
    """pack_2_4 as one CUDA kernel (trb_pack_2_4): fp16 weight [K, N] and logical scales fp16 [G, N]
    on a GPU -> (qweight, stored scales, meta).  Identical to pack_2_4 when every group of four K
    positions holds exactly two non-zeros of distinct or equal magnitude; with ties between a kept
    and a pruned element (fewer than two non-zeros, or more than two equal magnitudes) torch's
    argsort leaves the choice open and the kernel keeps the higher index: the packed tensors then
    decode to the same weights but need not be the same bits."""
    from ... import _lib

    if not weight_kn.is_cuda or weight_kn.dtype != torch.float16 or scales.dtype != torch.float16:
        raise RuntimeError("pack_2_4_cuda needs fp16 CUDA tensors")
    k, n = weight_kn.shape
    g = scales.shape[0]
    if g != 1 and k // g != 128:
        raise ValueError("group size must be -1 (one row of scales) or 128")
    weight_kn, scales = weight_kn.contiguous(), scales.contiguous()
    dev = weight_kn.device
    q = torch.empty(k // 32, 2 * n, dtype=torch.int32, device=dev)
    meta = torch.empty(n, k // 16, dtype=torch.int16, device=dev)
    s_out = torch.empty(g, n, dtype=torch.float16, device=dev)
    _lib.check(_lib.lib.trb_pack_2_4(_lib.ptr(weight_kn), _lib.ptr(scales), _lib.ptr(q), _lib.ptr(meta), _lib.ptr(s_out),
                                     k, n, -1 if g == 1 else 128, _lib.dev_of(weight_kn), _lib.stream_of(weight_kn)),
               "pack_2_4")
    return q, s_out, meta
