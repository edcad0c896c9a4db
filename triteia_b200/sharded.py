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
