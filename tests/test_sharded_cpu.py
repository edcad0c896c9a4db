"""CPU, world_size 2 over gloo: the delta-sharding / token dispatch logic of triteia_b200.sharded
(ownership rule, split sizes, permutations, combine) against an unsharded computation."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, case, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from triteia_b200 import sharded
        from triteia_b200.ops.matmul.sbmm import sbmm_16bit_forloop

        D, K, N, T = 6, 64, 16, 20
        g = torch.Generator().manual_seed(0)
        weights = torch.randn(D, K, N, generator=g)                       # every rank builds all, keeps its shard
        mine = sharded.shard_ids(D, rank, world)
        w_local = weights[mine]
        gr = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(T, K, generator=gr)
        if case == "mixed":
            idx = torch.randint(-1, D, (T,), generator=gr, dtype=torch.int32)
        elif case == "all_base":
            idx = torch.full((T,), -1, dtype=torch.int32)
        elif case == "one_owner":
            idx = torch.full((T,), 1, dtype=torch.int32)                   # everything goes to rank 1
        else:
            idx = torch.randint(0, D, (T,), generator=gr, dtype=torch.int32)

        def local_compute(rows, local_ids):
            return sbmm_16bit_forloop(w_local, rows, local_ids)

        y = sharded.sbmm_sharded(x, idx, local_compute, N)
        ref = sbmm_16bit_forloop(weights, x, idx)
        ok = torch.allclose(y, ref, rtol=1e-5, atol=1e-5)
        # fixed-capacity, sync-free exchange (torch statement of the CUDA buffer layout), twice on the
        # same buffers with different batches
        ex = sharded.FixedCapacityExchange(T, K, N, torch.device("cpu"), backend="torch", local_compute=local_compute,
                                           dtype=torch.float32)
        y2 = ex(x, idx)
        ok = ok and torch.allclose(y2, ref, rtol=1e-5, atol=1e-5)
        idx_b = torch.roll(idx, 3)
        y3 = ex(x, idx_b)
        ok = ok and torch.allclose(y3, sbmm_16bit_forloop(weights, x, idx_b), rtol=1e-5, atol=1e-5)
        plan = sharded.DispatchPlan(idx, world)
        ok = ok and plan.n_send == int((idx >= 0).sum())
        torch.save({"ok": bool(ok), "max_err": float((y - ref).abs().max())}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["mixed", "all_base", "one_owner", "no_base"])
def test_sharded_dispatch_world2(tmp_path, case):
    world = 2
    mp.start_processes(_worker, args=(world, _free_port(), case, str(tmp_path)), nprocs=world, join=True,
                       start_method="spawn")
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), f"r{r}.pt"))
        assert res["ok"], res


def test_ownership_rule():
    from triteia_b200 import sharded

    ids = torch.arange(10)
    assert sharded.owner_of(ids, 4).tolist() == [0, 1, 2, 3, 0, 1, 2, 3, 0, 1]
    assert sharded.local_id_of(ids, 4).tolist() == [0, 0, 0, 0, 1, 1, 1, 1, 2, 2]
    assert sharded.shard_ids(10, 1, 4) == [1, 5, 9]
    for r in range(4):
        for local, d in enumerate(sharded.shard_ids(10, r, 4)):
            assert int(sharded.owner_of(torch.tensor(d), 4)) == r and int(sharded.local_id_of(torch.tensor(d), 4)) == local


def _stack_worker(rank, world, port, case, out_dir):
    """The sharded linear stack's exchange (one dispatch, one combine for all layers) with a torch
    statement of the local stack, against the unsharded stack."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from triteia_b200 import sharded, stack
        from triteia_b200.ops.matmul.sbmm import sbmm_16bit_forloop

        D, T, L = 6, 24, 2
        linears = (("a", 32, 32), ("b", 32, 48), ("c", 48, 32))
        g = torch.Generator().manual_seed(1)
        weights = [[torch.randn(D, k, n, generator=g) for (_, k, n) in linears] for _ in range(L)]
        mine = sharded.shard_ids(D, rank, world)
        gr = torch.Generator().manual_seed(200 + rank)
        xs = {32: torch.randn(T, 32, generator=gr), 48: torch.randn(T, 48, generator=gr)}
        idx = torch.randint(-1, D, (T,), generator=gr, dtype=torch.int32)
        if case == "one_owner":
            idx[:] = 3
        elif case == "all_base":
            idx[:] = -1

        def run_stack(ws, x_by_width, ids):
            cs = torch.zeros(ids.numel())
            y = torch.zeros(ids.numel(), linears[-1][2])
            for layer in ws:
                for (_, k, n), w in zip(linears, layer):
                    y = sbmm_16bit_forloop(w, x_by_width[k], ids)
                    cs = cs + y.sum(dim=1)
            return y, cs

        def local_stack(x_by_width, local_ids):
            return run_stack([[w[mine] for w in layer] for layer in weights], x_by_width, local_ids)

        y, cs = stack.stack_sharded(xs, idx, local_stack, linears[-1][2])
        y_ref, cs_ref = run_stack(weights, xs, idx)
        ok = torch.allclose(y, y_ref, rtol=1e-5, atol=1e-5) and torch.allclose(cs, cs_ref, rtol=1e-4, atol=1e-4)
        ok = ok and bool(torch.all(y[idx == -1] == 0)) and bool(torch.all(cs[idx == -1] == 0))
        torch.save({"ok": bool(ok), "max_err": float((y - y_ref).abs().max())}, os.path.join(out_dir, f"s{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["mixed", "one_owner", "all_base"])
def test_sharded_stack_world2(tmp_path, case):
    world = 2
    mp.start_processes(_stack_worker, args=(world, _free_port(), case, str(tmp_path)), nprocs=world, join=True,
                       start_method="spawn")
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), f"s{r}.pt"))
        assert res["ok"], res
