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
  2. the owner routes the received rows once on the device (router + one gather per input width: a
     row's delta is the same in every linear), then runs every linear of every layer on the routed
     rows from one C call with no host read (tcgen05 launch for long segments, mma.sp launch for
     the rest, no router and no gather per linear), and folds each output into a per-token fp32
     checksum;
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
        """One C call, no host read: the rows are routed once on the device (every linear uses the same
        delta per row), gathered once per input width, and every linear runs on the routed rows."""
        import ctypes
        from . import _lib

        rows = int(local_ids.numel())
        dev = local_ids.device
        if rows == 0:
            return (torch.empty(0, self.n_last, dtype=torch.float16, device=dev),
                    torch.empty(0, dtype=torch.float32, device=dev))
        lins, q_arr, m_arr, s_arr, k_arr, n_arr = self._static_arrays()
        if local_ids.dtype != torch.int32:
            local_ids = local_ids.to(torch.int32)
        widths = sorted(x_by_width)
        xs = [x_by_width[k].contiguous() for k in widths]
        xs_sorted = [torch.empty_like(x) for x in xs]
        ybuf = {n: torch.empty(rows, n, dtype=torch.float16, device=dev) for n in {l.n for l in lins}}
        y_last = torch.empty(rows, self.n_last, dtype=torch.float16, device=dev)
        checksum = torch.zeros(rows, dtype=torch.float32, device=dev)
        num_deltas = int(lins[0].qweights.shape[0])
        nbytes = _lib.lib.trb_stack_scratch_bytes(rows, num_deltas)
        if getattr(self, "_scratch", None) is None or self._scratch.numel() < nbytes or self._scratch.device != dev:
            self._scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        vp_l, vp_w, ci_w = ctypes.c_void_p * len(lins), ctypes.c_void_p * len(widths), ctypes.c_int * len(widths)
        groupsize = 128 if lins[0].scales.shape[1] > 1 else -1
        err = _lib.lib.trb_stack_pass(
            len(lins), q_arr, m_arr, s_arr, k_arr, n_arr, len(widths), ci_w(*widths),
            vp_w(*[_lib.ptr(x) for x in xs]), vp_w(*[_lib.ptr(x) for x in xs_sorted]),
            vp_l(*[_lib.ptr(ybuf[l.n]) for l in lins]), _lib.ptr(y_last), _lib.ptr(local_ids), rows, num_deltas,
            _lib.ptr(checksum), groupsize, _lib.ptr(self._scratch), self._scratch.numel(), _lib.dev_of(checksum),
            _lib.stream_of(checksum))
        _lib.check(err, "stack_pass")
        return y_last, checksum


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


class FixedStackExchange:
    """`stack_sharded` for CUDA ranks without counts on the host: fixed-capacity exchange buffers (as
    sharded.FixedCapacityExchange: `world` chunks of T + 1 rows, the last row of a chunk carries the
    rows' local ids and their number), packed by the library's pack kernel, two equal-split NCCL
    all-to-alls per pass (rows + ids out; last output + checksums back, the checksums in the spare
    row of every chunk), no host synchronisation.  The owner runs its stack over all world * T slots;
    unused slots carry id -1 and cost nothing.  Buffers are allocated once per (T, widths, n_last)."""

    def __init__(self, num_tokens, widths, n_last, device, group=None):
        self.T, self.widths, self.n_last = int(num_tokens), sorted(int(w) for w in widths), int(n_last)
        self.W = sum(self.widths)
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        if self.T * 4 + 4 > self.W * 2 or self.T * 4 > self.n_last * 2:
            raise ValueError("a row must hold num_tokens + 1 int32 ids, an output row num_tokens fp32 checksums")
        rows = self.world * (self.T + 1)
        z = lambda cols: torch.zeros(rows, cols, dtype=torch.float16, device=device)
        self.send, self.recv, self.y_work, self.y_back = z(self.W), z(self.W), z(self.n_last), z(self.n_last)
        self.slot_of = torch.zeros(max(self.T, 1), dtype=torch.int32, device=device)
        self.plan = torch.zeros(8 + self.world, dtype=torch.int32, device=device)
        self.col = torch.arange(self.T, device=device)

    def __call__(self, x_by_width, indices, local_stack):
        from . import _lib
        from ._lib import lib, ptr, stream_of, dev_of

        w, T = self.world, self.T
        row = torch.cat([x_by_width[k] for k in self.widths], dim=1)          # each token travels once
        if indices.dtype != torch.int32:
            indices = indices.to(torch.int32)
        dev, st = dev_of(row), stream_of(row)
        _lib.check(lib.trb_shard_dispatch(ptr(row), ptr(indices), T, self.W, w, ptr(self.send), None, self.rank, None,
                                          self.n_last, ptr(self.slot_of), ptr(self.plan), dev, st), "shard_dispatch")
        dist.all_to_all_single(self.recv, self.send, group=self.group)
        recv3 = self.recv.view(w, T + 1, self.W)
        idrow = recv3[:, T, :].view(torch.int32)
        local_ids = torch.where(self.col[None, :] < idrow[:, T:T + 1], idrow[:, :T],
                                torch.full_like(idrow[:, :T], -1)).reshape(-1).contiguous()
        parts, at = {}, 0
        for k in self.widths:
            parts[k] = recv3[:, :T, at:at + k].reshape(w * T, k)
            at += k
        y_w, cs_w = local_stack(parts, local_ids)
        work3 = self.y_work.view(w, T + 1, self.n_last)
        work3[:, :T] = y_w.view(w, T, self.n_last)
        work3[:, T, :].view(torch.float32)[:, :T] = cs_w.view(w, T)
        dist.all_to_all_single(self.y_back, self.y_work, group=self.group)
        y = torch.empty(T, self.n_last, dtype=torch.float16, device=row.device)
        _lib.check(lib.trb_shard_combine(ptr(self.y_back), ptr(self.slot_of), ptr(y), T, self.n_last, w, 0, dev, st),
                   "shard_combine")
        cs_all = self.y_back.view(w, T + 1, self.n_last)[:, T, :].view(torch.float32)[:, :T].reshape(-1)
        slot = self.slot_of[:T].long()
        cs = torch.where(slot >= 0, cs_all[slot.clamp(min=0)], torch.zeros((), device=row.device))
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
