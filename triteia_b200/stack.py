"""A stack of independent indexed delta linears over one routed token batch, with the delta set
sharded by id across the ranks of a process group (the "full Llama-2-7B-shaped linear stack"
scenario: per layer q/k/v/o 4096->4096, gate/up 4096->11008, down 11008->4096).

The reference has no such driver: it runs one linear at a time
(triteia/python/ops/matmul/sbmm.py:94-123) and its weights are chunked for tensor parallelism
offline (triteia/python/ops/utils/generator.py:126-176).  What is used here of its semantics: a
token's delta id selects the same delta in every linear, id -1 means "no delta" (zero output).

Protocol of one pass (one exchange each way, whatever the number of layers):
  1. every rank sends each of its tokens that has a delta ONCE, as the row [x_4096 | x_11008],
     with its local delta id, to owner(id) = id % world (NCCL all-to-all; counts first);
  2. the owner groups the received rows once, by segment size class and delta (sort + one segment
     list per class; a handful of host reads per pass), then runs every linear of every layer on
     the grouped rows with the segment-list kernel entry point, one launch per size class (no
     router and no gather per linear), and folds each output into a per-token fp32 checksum;
  3. the last linear's output rows and the checksums travel back and are scattered into token order.
The linears are independent (each reads the seeded activation of its input width), so the result
does not depend on the number of ranks.
"""
import torch
import torch.distributed as dist

from .sharded import DispatchPlan

# (name, in features, out features) of the seven linears of one Llama-2-7B decoder layer.
LLAMA_7B_LINEARS = (
    ("q", 4096, 4096), ("k", 4096, 4096), ("v", 4096, 4096), ("o", 4096, 4096),
    ("gate", 4096, 11008), ("up", 4096, 11008), ("down", 11008, 4096),
)
# The same layer as the reference's converter stores it: q/k/v fused into one packed matrix along the
# output features, gate/up likewise (triteia/python/configs/models/llama.py:8-14,
# triteia/tools/converters/convert_deltazip.py:98-123).  Four launches per layer instead of seven,
# each with up to three times the work items.
LLAMA_7B_FUSED_LINEARS = (
    ("qkv", 4096, 3 * 4096), ("o", 4096, 4096), ("gate_up", 4096, 2 * 11008), ("down", 11008, 4096),
)


class StackLinear:
    """One linear of the stack on one rank: this rank's packed deltas [D_local, ...]."""

    def __init__(self, name, k, n, qweights, metas, scales):
        self.name, self.k, self.n = name, int(k), int(n)
        self.qweights, self.metas, self.scales = qweights, metas, scales


class DeltaStackShard:
    """This rank's part of the stack: `layers` is a list (layers) of lists (linears) of StackLinear.

    __call__(x_by_width, local_ids) takes rows received from any rank (x_by_width[k] is [rows, k]
    fp16, local_ids [rows] int32, all >= 0) and returns (y_last [rows, n_last] fp16, checksum [rows]
    fp32) in the order of the rows: y_last is the output of the last linear of the last layer,
    checksum[t] the fp32 sum over every linear of the sum of its fp16 output row t.
    """

    def __init__(self, layers):
        self.layers = layers
        self.n_last = layers[-1][-1].n

    # Segments are handled in two size classes, one launch per class and linear: up to 32 rows ->
    # 8-row tiles of the mma.sp kernel, longer ones -> 256-row tiles of the tcgen05 kernel.
    CLASS_BOUNDS = (32,)
    CLASS_TILES = (8, 256)

    def _plan(self, local_ids):
        """Rows ordered by (size class, delta id) and, per class, its row range and segment list."""
        from .ops.matmul.sbmm import _segments

        dev = local_ids.device
        ids64 = local_ids.to(torch.int64)
        counts = torch.bincount(ids64)
        bounds = torch.tensor(self.CLASS_BOUNDS, device=dev)
        cls_of = torch.bucketize(counts, bounds)                      # 0: <= 8 rows ... 3: > 32 rows
        big = int(counts.numel()) + 1
        order = torch.argsort(cls_of[ids64] * big + ids64, stable=True)
        ids_sorted = local_ids[order].to(torch.int32).contiguous()
        cls_sorted = cls_of[ids64][order]
        cls_rows = torch.bincount(cls_sorted, minlength=len(self.CLASS_BOUNDS) + 1).tolist()   # host read (once per pass)
        classes, at = [], 0
        for ci, n_rows in enumerate(cls_rows):
            if n_rows:
                uniq, starts, cnts = _segments(ids_sorted[at:at + n_rows])   # sizes its outputs on the host
                classes.append((at, n_rows, uniq, starts, cnts, self.CLASS_TILES[ci]))
            at += n_rows
        return order, classes

    def _ksplit(self, dev):
        """Working memory of the grouped kernel's tail K split (zero on entry, left zero by every launch)."""
        from . import _lib

        if getattr(self, "_ksplit_buf", None) is None or self._ksplit_buf.device != dev:
            self._ksplit_buf = torch.zeros(_lib.lib.trb_sbmm_ksplit_bytes(), dtype=torch.uint8, device=dev)
        return self._ksplit_buf

    def _static_arrays(self):
        """Host arrays of the per-linear device pointers and shapes (built once)."""
        import ctypes
        from . import _lib

        if getattr(self, "_static", None) is None:
            lins = [lin for layer in self.layers for lin in layer]
            vp, ci = ctypes.c_void_p * len(lins), ctypes.c_int * len(lins)
            self._static = (lins, vp(*[_lib.ptr(l.qweights) for l in lins]), vp(*[_lib.ptr(l.metas) for l in lins]),
                            vp(*[_lib.ptr(l.scales) for l in lins]), ci(*[l.k for l in lins]), ci(*[l.n for l in lins]))
        return self._static

    def __call__(self, x_by_width, local_ids):
        import ctypes
        from . import _lib

        rows = int(local_ids.numel())
        dev = local_ids.device
        if rows == 0:
            return (torch.empty(0, self.n_last, dtype=torch.float16, device=dev),
                    torch.empty(0, dtype=torch.float32, device=dev))
        order, classes = self._plan(local_ids)
        xs = {k: x.index_select(0, order).contiguous() for k, x in x_by_width.items()}
        lins, q_arr, m_arr, s_arr, k_arr, n_arr = self._static_arrays()
        ybuf = {n: torch.empty(rows, n, dtype=torch.float16, device=dev) for n in {l.n for l in lins}}
        checksum = torch.zeros(rows, dtype=torch.float32, device=dev)
        vp_l, vp_c, ci_c = ctypes.c_void_p * len(lins), ctypes.c_void_p * len(classes), ctypes.c_int * len(classes)
        x_arr = vp_l(*[_lib.ptr(xs[l.k]) for l in lins])
        y_arr = vp_l(*[_lib.ptr(ybuf[l.n]) for l in lins])
        groupsize = 128 if lins[0].scales.shape[1] > 1 else -1
        err = _lib.lib.trb_stack_pass(
            len(lins), q_arr, m_arr, s_arr, k_arr, n_arr, x_arr, y_arr, len(classes),
            ci_c(*[c[0] for c in classes]), ci_c(*[c[1] for c in classes]),
            vp_c(*[_lib.ptr(c[2]) for c in classes]), vp_c(*[_lib.ptr(c[3]) for c in classes]),
            vp_c(*[_lib.ptr(c[4]) for c in classes]), ci_c(*[int(c[2].numel()) for c in classes]),
            ci_c(*[c[5] for c in classes]), _lib.ptr(checksum), rows, groupsize, _lib.ptr(self._ksplit(dev)),
            _lib.lib.trb_sbmm_ksplit_bytes(), _lib.dev_of(checksum), _lib.stream_of(checksum))
        _lib.check(err, "stack_pass")
        y = ybuf[self.n_last]
        y_out = torch.empty_like(y)
        y_out[order] = y
        cs_out = torch.empty_like(checksum)
        cs_out[order] = checksum
        return y_out, cs_out


def stack_sharded(x_by_width, indices, local_stack, n_last, group=None):
    """One pass of the sharded stack for this rank's tokens.

    x_by_width: {k: [T, k] fp16} this rank's activations, one per input width; indices [T] GLOBAL
    delta ids (-1 = none).  local_stack(x_by_width_rows, local_ids) -> (y_last, checksum) applies
    this rank's shard (a DeltaStackShard on GPUs; any callable in the CPU tests).
    Returns (y [T, n_last] in the activations' dtype, checksum [T] fp32); rows without a delta are 0.
    """
    world = dist.get_world_size(group)
    plan = DispatchPlan(indices, world, group)
    widths = sorted(x_by_width)
    first = x_by_width[widths[0]]
    T, dev, dt = first.shape[0], first.device, first.dtype
    row = torch.cat([x_by_width[k] for k in widths], dim=1)            # each token travels once
    row_send = row[plan.sent_rows].contiguous()
    row_recv = torch.empty(plan.n_recv, row.shape[1], dtype=dt, device=dev)
    id_recv = torch.empty(plan.n_recv, dtype=torch.int32, device=dev)
    dist.all_to_all_single(row_recv, row_send, plan.recv, plan.send, group=group)
    dist.all_to_all_single(id_recv, plan.local_ids, plan.recv, plan.send, group=group)
    parts, at = {}, 0
    for k in widths:
        parts[k] = row_recv[:, at:at + k].contiguous()
        at += k
    y_work, cs_work = local_stack(parts, id_recv)
    y_back = torch.empty(plan.n_send, n_last, dtype=dt, device=dev)
    cs_back = torch.empty(plan.n_send, dtype=torch.float32, device=dev)
    dist.all_to_all_single(y_back, y_work.to(dt).contiguous(), plan.send, plan.recv, group=group)
    dist.all_to_all_single(cs_back, cs_work.float().contiguous(), plan.send, plan.recv, group=group)
    y = torch.zeros(T, n_last, dtype=dt, device=dev)
    cs = torch.zeros(T, dtype=torch.float32, device=dev)
    y[plan.sent_rows] = y_back
    cs[plan.sent_rows] = cs_back
    return y, cs


def random_stack_shard(num_deltas, rank, world, num_layers, linears=LLAMA_7B_FUSED_LINEARS, groupsize=128, device="cuda",
                       seed=0):
    """Seeded synthetic shard: for every layer and linear the packed deltas with global ids
    rank, rank + world, ... (local-id order).  Every (layer, linear, global id) has its own seed, so
    the whole stack is the same set of deltas for every world size."""
    from .ops.utils.generator import random_packed_deltas

    mine = list(range(rank, num_deltas, world))
    layers = []
    for li in range(num_layers):
        layer = []
        for ji, (name, k, n) in enumerate(linears):
            qs, ms, ss = [], [], []
            for d in mine:
                q, m, s = random_packed_deltas(1, k, n, groupsize=groupsize, device=device,
                                               seed=seed + ((li * 16 + ji) * 100003 + d) * 7 + 1)
                qs.append(q[0]); ms.append(m[0]); ss.append(s[0])
            layer.append(StackLinear(name, k, n, torch.stack(qs), torch.stack(ms), torch.stack(ss)))
        layers.append(layer)
    return layers
