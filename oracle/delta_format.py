"""CPU oracle, part 1: decoder of the packed int4 + 2:4 delta format.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and the cpu_baseline / reference legs of bench.py may
import this package; the product (triteia_b200) never does.

This is an independent closed-form restatement of the wire format that the reference
defines in code.  It uses numpy only and shares nothing with the product's packer.

Format (reference files, relative to the reference checkout):
  * quantisation: code = clamp(round(w / s) + 8, 0, 15), triteia/python/nn/linear.py:110-112
  * 2:4 compression and metadata nibbles: triteia/python/ops/utils/sparsity.py:167-290
    (low 2 bits of a nibble = position of the first kept value inside its group of four
    consecutive K positions, high 2 bits = position of the second, sparsity.py:246-272)
  * metadata physical order: sparsity.py:134-161
  * 16x16 tiling, lane permutation and nibble interleave of the codes:
    nn/linear.py:128-138 with the permutation built at sparsity.py:35-54
  * grouped scales are stored with every 8 output columns in the order 0,4,1,5,2,6,3,7
    (sparsity.py:55-57, read back at triteia/csrc/ops/marlin.cuh:206-208,376-380);
    per-channel scales are stored in natural order (sparsity.py:58-60).

Parity pin: tests/test_oracle_golden.py checks `dequantize` bit-exactly against the fp16
`uncompress` matrices that the reference packer returned for the tensors stored in
tests/golden/reference_vectors.npz (made by tests/golden/make_golden.py).
"""
import numpy as np

SCALE_GROUP_ORDER = np.array([0, 4, 1, 5, 2, 6, 3, 7])


def unpack_codes(qweight):
    """qweight int32 [K/32, 2N] -> compressed codes uint8 [K/2, N] (values 0..15).

    Word w of slab row kt belongs to the 64-column block w // 128, lane i = (w % 128) // 4
    and register j = w % 4.  Nibble p of that word holds output column
    64*blk + 8*(i // 4) + 4*((p % 4) // 2) + j and compressed row
    16*kt + 2*(i % 4) + (p >= 4) + 8*(p % 2).
    """
    q = np.ascontiguousarray(qweight).view(np.uint32)
    kt, w2 = q.shape
    n = w2 // 2
    out = np.zeros((kt * 16, n), dtype=np.uint8)
    w = np.arange(w2)
    blk = w // 128
    lane = (w % 128) // 4
    j = w % 4
    for p in range(8):
        col = 64 * blk + 8 * (lane // 4) + 4 * ((p % 4) // 2) + j
        crow = 2 * (lane % 4) + (1 if p >= 4 else 0) + 8 * (p % 2)
        vals = ((q >> np.uint32(4 * p)) & np.uint32(0xF)).astype(np.uint8)
        rows = (16 * np.arange(kt)[:, None] + crow[None, :])
        out[rows, np.broadcast_to(col[None, :], rows.shape)] = vals
    return out


def meta_physical_offset(row, col, n_rows):
    """Flat int16 offset of nominal metadata element (row = output column, col = K // 16)."""
    r = row
    dst = (r // 64) * 64 + (r % 2) * 2 + (r % 8) // 4 + ((r % 32) % 4) // 2 * 32 + ((r % 64) // 8) * 4
    topright = ((dst % 2 == 0) & (col % 2 == 1)).astype(np.int64)
    bottomleft = ((dst % 2 == 1) & (col % 2 == 0)).astype(np.int64)
    dst = dst + topright - bottomleft
    c = col - topright + bottomleft
    return (c // 2) * n_rows * 2 + dst * 2 + c % 2


def unpack_meta(meta):
    """meta int16 [N, K/16] (physical order) -> kept positions uint8 [N, K/4, 2] (0..3)."""
    n, kc = meta.shape
    flat = np.ascontiguousarray(meta).reshape(-1).view(np.uint16)
    rows, cols = np.meshgrid(np.arange(n), np.arange(kc), indexing="ij")
    nominal = flat[meta_physical_offset(rows, cols, n)]  # [N, K/16]
    pos = np.zeros((n, kc, 4, 2), dtype=np.uint8)
    for qd in range(4):
        nib = (nominal >> np.uint16(4 * qd)) & np.uint16(0xF)
        pos[:, :, qd, 0] = nib & 3
        pos[:, :, qd, 1] = (nib >> 2) & 3
    return pos.reshape(n, kc * 4, 2)


def logical_scales(s):
    """Stored scales fp16 [G, N] -> logical fp16 [G, N] (G = 1: natural order already)."""
    s = np.asarray(s)
    if s.shape[0] == 1:
        return s
    g, n = s.shape
    out = np.empty_like(s)
    blocks = s.reshape(g, n // 8, 8)
    out.reshape(g, n // 8, 8)[:, :, SCALE_GROUP_ORDER] = blocks
    return out


def dense_levels(qweight, meta):
    """Signed levels int8 [K, N] (code - 8 at kept positions, 0 elsewhere)."""
    codes = unpack_codes(qweight)  # [K/2, N]
    pos = unpack_meta(meta)  # [N, K/4, 2]
    khalf, n = codes.shape
    k = khalf * 2
    dense = np.zeros((k, n), dtype=np.int8)
    cols = np.arange(n)
    groups = np.arange(k // 4)
    for which in range(2):
        lev = codes[which::2, :].astype(np.int16) - 8  # [K/4, N]
        krow = 4 * groups[:, None] + pos[:, :, which].T.astype(np.int64)  # [K/4, N]
        dense[krow, np.broadcast_to(cols[None, :], krow.shape)] = lev.astype(np.int8)
    return dense


def dequantize(qweight, meta, s):
    """Packed delta -> dense fp16 weight [K, N], W = fp16(level) * fp16(scale) rounded to fp16.

    The rounding matches how the reference builds its fp16 `uncompress` matrix
    (triteia/python/ops/utils/generator.py:40: `(w - 8).half() * s`).
    """
    lev = dense_levels(qweight, meta)
    k, n = lev.shape
    sl = logical_scales(s).astype(np.float16)
    g = sl.shape[0]
    per_row = np.repeat(sl, k // g, axis=0)  # [K, N]
    return (lev.astype(np.float16) * per_row).astype(np.float16)


def column_blocks(qweight, meta, s, blk0, nblk):
    """The packed tensors of output columns [64 * blk0, 64 * (blk0 + nblk)) of one delta.

    A 64-column block is self-contained in every packed tensor: 128 consecutive words of each
    qweight row, rows 64b..64b+63 of the metadata (physically [K/32][N][2] int16, reordered only
    inside 64-row groups), 64 consecutive scale columns (the stored order permutes inside 8-column
    blocks).  The result decodes with `dequantize` to the same values as columns 64*blk0.. of the
    whole delta, at 1/(N/64/nblk) of the cost: full-size parity checks use it on sampled rows.
    Takes numpy arrays or tensors (only slicing and reshape are used before the copy to numpy).
    """
    q = qweight[:, 128 * blk0:128 * (blk0 + nblk)]
    n, kc = meta.shape
    m = meta.reshape(kc // 2, n, 2)[:, 64 * blk0:64 * (blk0 + nblk), :].reshape(64 * nblk, kc)
    sc = s[:, 64 * blk0:64 * (blk0 + nblk)]
    return to_numpy(q), to_numpy(m), to_numpy(sc)


def to_numpy(a):
    """numpy view or copy of an array-like; device tensors (anything with .detach) come through the host."""
    if hasattr(a, "detach"):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a)


VALID_META_NIBBLES = np.array([0b0100, 0b1000, 0b1100, 0b1001, 0b1101, 0b1110], dtype=np.uint16)


def random_packed(k, n, groupsize=-1, seed=0, scale_lo=0.001, scale_hi=0.01):
    """A valid packed delta drawn directly in the wire format (numpy only): every code word is
    valid as it is, a metadata nibble is valid when its first position (low 2 bits) is below its
    second (high 2 bits), and the physical metadata order is a permutation, so any arrangement of
    valid nibbles decodes.  Levels come out uniform in [-8, 7].  Used by the CPU timing legs, which
    must not load the product library."""
    rng = np.random.default_rng(seed)
    q = rng.integers(0, 1 << 32, size=(k // 32, 2 * n), dtype=np.uint64).astype(np.uint32).view(np.int32)
    nib = VALID_META_NIBBLES[rng.integers(0, 6, size=(n, k // 16, 4))]
    m = (nib[..., 0] | (nib[..., 1] << 4) | (nib[..., 2] << 8) | (nib[..., 3] << 12)).astype(np.uint16).view(np.int16)
    g = 1 if groupsize == -1 else k // groupsize
    s = rng.uniform(scale_lo, scale_hi, size=(g, n)).astype(np.float16)
    return q, m, s
