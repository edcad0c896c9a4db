"""Multi-GPU form of the indexed delta matmul: the delta set is sharded by id across the ranks
of a torch.distributed process group, tokens travel to the rank that owns their delta and the
results travel back (all-to-all over NCCL / NVLink on GPUs, gloo in the CPU tests).

The reference has no distributed layer; its "tensor parallel" code only chunks weights offline
(triteia/python/ops/utils/generator.py:126-176).  Ownership rule: owner(d) = d % world_size,
local id = d // world_size, so popular low ids spread over the ranks.  Tokens with index -1
never leave their rank.  One exchange each way per call: counts, then rows + local ids out,
then result rows back.
"""
import torch
import torch.distributed as dist


def owner_of(delta_ids, world_size):
    return delta_ids % world_size


def local_id_of(delta_ids, world_size):
    return torch.div(delta_ids, world_size, rounding_mode="floor")


def shard_ids(num_deltas, rank, world_size):
    """Global delta ids held by `rank`, in local-id order."""
    return list(range(rank, num_deltas, world_size))


class DispatchPlan:
    """Routing of one batch: who sends how many rows to whom (host integers) plus the device
    permutation that groups the local rows by destination rank."""

    def __init__(self, indices, world_size, group=None):
        self.world = world_size
        idx = indices.to(torch.int64)
        has_delta = idx >= 0
        dest = torch.where(has_delta, owner_of(idx, world_size), torch.full_like(idx, world_size))
        self.order = torch.argsort(dest, stable=True)               # rows grouped by destination
        send_counts = torch.bincount(dest, minlength=world_size + 1)[:world_size]
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        self.send = send_counts.tolist()                             # the one host sync of the call
        self.recv = recv_counts.tolist()
        self.n_send = sum(self.send)
        self.n_recv = sum(self.recv)
        self.sent_rows = self.order[: self.n_send]
        self.local_ids = local_id_of(idx[self.sent_rows], world_size).to(torch.int32)


def sbmm_sharded(x, indices, local_compute, n_out, group=None, base_out=None):
    """y[t] = base_out[t] + x[t] @ delta[indices[t]] with the deltas spread over the group.

    x [T, K] fp16 and indices [T] (GLOBAL delta ids, -1 = none) are this rank's tokens.
    local_compute(x_rows, local_ids) -> [rows, n_out] applies this rank's shard to rows
    received from any rank.  Returns y [T, n_out] in x.dtype.
    """
    world = dist.get_world_size(group)
    plan = DispatchPlan(indices, world, group)
    k = x.shape[1]
    x_send = x[plan.sent_rows].contiguous()
    x_recv = torch.empty(plan.n_recv, k, dtype=x.dtype, device=x.device)
    id_recv = torch.empty(plan.n_recv, dtype=torch.int32, device=x.device)
    dist.all_to_all_single(x_recv, x_send, plan.recv, plan.send, group=group)
    dist.all_to_all_single(id_recv, plan.local_ids, plan.recv, plan.send, group=group)
    y_work = local_compute(x_recv, id_recv) if plan.n_recv > 0 else torch.empty(0, n_out, dtype=x.dtype, device=x.device)
    y_back = torch.empty(plan.n_send, n_out, dtype=x.dtype, device=x.device)
    dist.all_to_all_single(y_back, y_work.contiguous(), plan.send, plan.recv, group=group)
    y = base_out if base_out is not None else torch.zeros(x.shape[0], n_out, dtype=x.dtype, device=x.device)
    y[plan.sent_rows] += y_back
    return y


def make_local_sbmm(qweights, metas, scales):
    """local_compute built on the fused CUDA entry point for this rank's packed shard."""
    from .ops.matmul.sbmm import sbmm_indexed

    def run(x_rows, local_ids):
        return sbmm_indexed(x_rows.contiguous(), qweights, metas, scales, local_ids)

    return run


# --------------------------------------------------------------------------------------------
# Fixed-capacity exchange: no counts on the host, no host synchronisation, two collectives.
# --------------------------------------------------------------------------------------------
class FixedCapacityExchange:
    """One sbmm call over a sharded delta set with equal-split all-to-alls.

    Every rank sends `world` chunks of T + 1 rows (T = its token count, the same on all ranks):
    chunk r holds the rows whose delta lives on rank r, then one row with their local ids (int32)
    and the number of rows in use.  The owner computes on the received buffer in place and returns
    result rows in the same slots.  Buffers are allocated once per (T, K, N).

    backend "cuda": the three steps are the C-ABI calls trb_shard_dispatch / trb_shard_compute /
    trb_shard_combine with an NCCL all-to-all (equal splits) after the first two.
    backend "p2p": no collective; the receive and return buffers are CUDA symmetric memory
    (torch.distributed._symmetric_memory), the pack kernel and the grouped kernel's epilogue store
    rows straight into the owner's receive buffer / the source's output tensor over NVLink, and a
    cross-GPU barrier follows each of the two steps.  The returned tensor is this object's output
    buffer: the next call overwrites it.  backend "torch": the same buffer layout written with torch ops and a
    caller-supplied local_compute(x_rows, local_ids) -> rows; it exists so that the layout and the
    collectives can be tested on CPU ranks (gloo).
    """

    def __init__(self, num_tokens, k, n_out, device, group=None, backend="cuda", qweights=None, metas=None,
                 scales=None, local_compute=None, dtype=torch.float16):
        self.T, self.K, self.N = num_tokens, k, n_out
        self.group = group
        self.world = dist.get_world_size(group)
        self.backend = backend
        self.device = device
        rows = self.world * (self.T + 1)
        if self.T * 4 + 4 > k * dtype.itemsize:
            raise ValueError("the id row of a chunk must hold num_tokens + 1 int32 values")
        self.rank = dist.get_rank(group)
        if backend == "p2p":
            import torch.distributed._symmetric_memory as symm_mem

            grp = group if group is not None else dist.group.WORLD
            self.recv = symm_mem.empty(rows, k, dtype=dtype, device=device)
            self.y_out = symm_mem.empty(max(num_tokens, 1), n_out, dtype=dtype, device=device)
            self.recv.zero_()
            self.y_out.zero_()
            self.h_recv = symm_mem.rendezvous(self.recv, grp)
            self.h_out = symm_mem.rendezvous(self.y_out, grp)
            self.send = self.y_work = self.y_back = None
        else:
            self.send = torch.zeros(rows, k, dtype=dtype, device=device)
            self.recv = torch.zeros(rows, k, dtype=dtype, device=device)
            self.y_work = torch.zeros(rows, n_out, dtype=dtype, device=device)
            self.y_back = torch.zeros(rows, n_out, dtype=dtype, device=device)
        self.slot_of = torch.zeros(max(self.T, 1), dtype=torch.int32, device=device)
        self.plan = torch.zeros(8 + self.world, dtype=torch.int32, device=device)
        self.q, self.m, self.s = qweights, metas, scales
        self.local_compute = local_compute
        if backend in ("cuda", "p2p"):
            from ._lib import lib
            d_local, g, _ = scales.shape
            self.groupsize = -1 if g == 1 else k // g
            self.d_local = d_local
            nbytes = lib.trb_sbmm_indexed_scratch_bytes(rows, k, d_local)
            self.scratch = torch.empty(nbytes, dtype=torch.uint8, device=device)

    # ---- torch statement of the layout (CPU-capable) ----
    def _id_rows(self, buf):
        """int32 view [world, row_ints] of the id rows of an exchange buffer."""
        return buf.view(self.world, self.T + 1, -1)[:, self.T, :].view(torch.int32)

    def _dispatch_torch(self, x, idx):
        w, T = self.world, self.T
        idx64 = idx.to(torch.int64)
        has = idx64 >= 0
        dest = torch.where(has, idx64 % w, torch.full_like(idx64, w))
        onehot = (dest[:, None] == torch.arange(w, device=x.device)[None, :]).to(torch.int64)
        rank_in_dest = (torch.cumsum(onehot, 0) - onehot).gather(1, dest.clamp(max=w - 1)[:, None])[:, 0]
        slot = torch.where(has, dest * T + rank_in_dest, torch.full_like(dest, -1))
        self.slot_of.copy_(slot.to(torch.int32))
        send3 = self.send.view(w, T + 1, -1)
        rows = torch.nonzero(has)[:, 0]
        send3[dest[rows], rank_in_dest[rows]] = x[rows]
        ids = torch.zeros(w, self.send.shape[1] * self.send.element_size() // 4, dtype=torch.int32, device=x.device)
        ids[dest[rows], rank_in_dest[rows]] = torch.div(idx64[rows], w, rounding_mode="floor").to(torch.int32)
        ids[:, T] = onehot.sum(0).to(torch.int32)
        send3[:, T, :] = ids.view(self.send.dtype)

    def _compute_torch(self):
        w, T = self.world, self.T
        ids = self._id_rows(self.recv)
        recv3 = self.recv.view(w, T + 1, -1)
        work3 = self.y_work.view(w, T + 1, -1)
        for r in range(w):
            n = int(ids[r, T])
            if n > 0:
                work3[r, :n] = self.local_compute(recv3[r, :n].contiguous(), ids[r, :n].contiguous())

    def _combine_torch(self, y):
        slot = self.slot_of[: self.T].to(torch.int64)
        has = slot >= 0
        r, q = torch.div(slot, self.T, rounding_mode="floor"), slot % self.T
        back3 = self.y_back.view(self.world, self.T + 1, -1)
        rows = torch.nonzero(has)[:, 0]
        y[rows] += back3[r[rows], q[rows]]
        return y

    # ---- one call ----
    def __call__(self, x, indices, base_out=None):
        """x [T, K], indices int32 [T] (global ids, -1 = none) -> y [T, N] (= base_out + delta part)."""
        assert x.shape[0] == self.T and x.shape[1] == self.K
        if self.backend in ("cuda", "p2p"):
            from . import _lib
            from ._lib import lib, ptr, stream_of, dev_of
            dev, st = dev_of(x), stream_of(x)
            if indices.dtype != torch.int32:
                indices = indices.to(torch.int32)
            p2p = self.backend == "p2p"
            _lib.check(lib.trb_shard_dispatch(ptr(x), ptr(indices), self.T, self.K, self.world, ptr(self.send),
                                              self.h_recv.buffer_ptrs_dev if p2p else None, self.rank,
                                              ptr(self.y_out) if p2p else None, self.N,
                                              ptr(self.slot_of), ptr(self.plan), dev, st), "shard_dispatch")
            if p2p:
                self.h_recv.barrier(channel=0)
            else:
                dist.all_to_all_single(self.recv, self.send, group=self.group)
            _lib.check(lib.trb_shard_compute(ptr(self.recv), ptr(self.q), ptr(self.m), ptr(self.s),
                                             None if p2p else ptr(self.y_work), self.world, self.T, self.N,
                                             self.K, self.d_local, self.groupsize,
                                             self.h_out.buffer_ptrs_dev if p2p else None, self.rank,
                                             ptr(self.scratch), self.scratch.numel(), dev, st), "shard_compute")
            if p2p:
                self.h_out.barrier(channel=0)
                if base_out is not None:
                    base_out += self.y_out[: self.T]
                    return base_out
                return self.y_out[: self.T]
            dist.all_to_all_single(self.y_back, self.y_work, group=self.group)
            y = base_out if base_out is not None else torch.empty(self.T, self.N, dtype=x.dtype, device=x.device)
            _lib.check(lib.trb_shard_combine(ptr(self.y_back), ptr(self.slot_of), ptr(y), self.T, self.N, self.world,
                                             int(base_out is not None), dev, st), "shard_combine")
            return y
        self._dispatch_torch(x, indices)
        dist.all_to_all_single(self.recv, self.send, group=self.group)
        self._compute_torch()
        dist.all_to_all_single(self.y_back, self.y_work, group=self.group)
        y = base_out if base_out is not None else torch.zeros(self.T, self.N, dtype=x.dtype, device=x.device)
        return self._combine_torch(y)
