"""GPU: the sharded sbmm path (C-ABI shard entry points + NCCL equal-split all-to-all) against the
CPU oracle over the whole delta set.  Runs as child processes: world 1 always, world 2 when the box
has two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir, backend):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import triteia_b200.ops as ops
        from triteia_b200 import sharded, _lib
        from oracle import ops as oracle

        D, K, N, T, g = 6 * world, 256, 256, 40, 128
        qs, metas, ss = ops.random_packed_deltas(D, K, N, groupsize=g, device="cpu", seed=5, scale_lo=0.005, scale_hi=0.02)
        mine = sharded.shard_ids(D, rank, world)
        q_l, m_l, s_l = qs[mine].to(dev), metas[mine].to(dev), ss[mine].to(dev)
        ex = sharded.FixedCapacityExchange(T, K, N, dev, backend=backend, qweights=q_l, metas=m_l, scales=s_l)
        worst = 0.0
        for call in range(2):
            gen = torch.Generator().manual_seed(10 * rank + call)
            x = torch.randn(T, K, generator=gen).half().to(dev)
            idx = torch.randint(-1, D, (T,), generator=gen, dtype=torch.int32).to(dev)
            if call == 1:
                idx[: T // 2] = 1 % D            # a hot delta: most rows go to one rank
            y = ex(x, idx)
            torch.cuda.synchronize()
            ref = oracle.sbmm(qs.numpy(), x.cpu().numpy(), metas.numpy(), ss.numpy(), idx.cpu().numpy())
            err = float(oracle.row_rel_err(y.float().cpu().numpy(), ref).max())
            worst = max(worst, err)
            assert torch.all(y[idx == -1] == 0)
            base = torch.randn(T, N, generator=gen).half().to(dev)
            yb = ex(x, idx, base_out=base.clone())
            torch.cuda.synchronize()
            errb = float(oracle.row_rel_err(yb.float().cpu().numpy(), ref + base.float().cpu().numpy()).max())
            worst = max(worst, errb)
        status = _lib.device_status(rank)
        torch.save({"err": worst, "status": status}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("backend", ["cuda", "p2p"])
@pytest.mark.parametrize("world", [1, 2])
def test_sharded_exchange_cuda(cuda, tmp_path, world, backend):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.start_processes(_worker, args=(world, _free_port(), str(tmp_path), backend), nprocs=world, join=True, start_method="spawn")
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), f"r{r}.pt"))
        assert res["status"] == 0
        assert res["err"] <= 1e-2, res


def _stack_worker(rank, world, port, out_dir):
    """Sharded stack of independent delta linears (one dispatch and one combine for all layers) on
    the CUDA segment-list entry point + row checksum kernel, against the CPU oracle over the whole
    delta set."""
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from triteia_b200 import stack, _lib
        from oracle import ops as oracle

        D, T, L = 8, 48, 2
        linears = (("a", 256, 256), ("b", 256, 384), ("c", 384, 256))
        shard = stack.random_stack_shard(D, rank, world, L, linears=linears, groupsize=128, device=dev, seed=11)
        # the whole set, drawn on the same device type (a CUDA generator's stream differs from a CPU one),
        # then moved to the host for the oracle; the shard is the matching rows of it
        full = stack.random_stack_shard(D, 0, 1, L, linears=linears, groupsize=128, device=dev, seed=11)
        mine = list(range(rank, D, world))
        same = all(torch.equal(shard[l][j].qweights, full[l][j].qweights[mine]) and
                   torch.equal(shard[l][j].scales, full[l][j].scales[mine]) for l in range(L) for j in range(3))
        for layer in full:
            for lin in layer:
                lin.qweights, lin.metas, lin.scales = lin.qweights.cpu(), lin.metas.cpu(), lin.scales.cpu()
        local = stack.DeltaStackShard(shard)
        worst_y, worst_cs = 0.0, 0.0
        for call in range(2):
            gen = torch.Generator().manual_seed(31 * rank + call)
            xs = {256: torch.randn(T, 256, generator=gen).half().to(dev), 384: torch.randn(T, 384, generator=gen).half().to(dev)}
            idx = torch.randint(-1, D, (T,), generator=gen, dtype=torch.int32).to(dev)
            if call == 1:
                idx[: T // 2] = 3            # a hot delta
            y, cs = stack.stack_sharded(xs, idx, local, linears[-1][2])
            y2, cs2 = stack.FixedStackExchange(T, [k for k in xs], linears[-1][2], dev)(xs, idx, local)
            assert torch.equal(y2, y) and torch.allclose(cs2, cs, rtol=1e-6, atol=1e-6)
            torch.cuda.synchronize()
            idx_np = idx.cpu().numpy()
            cs_ref = np.zeros(T, dtype=np.float64)
            l1 = np.zeros(T, dtype=np.float64)
            ref = None
            for l in range(L):
                for j, (_, k, n) in enumerate(linears):
                    lin = full[l][j]
                    ref = oracle.sbmm(lin.qweights.numpy(), xs[k].cpu().numpy(), lin.metas.numpy(), lin.scales.numpy(), idx_np)
                    cs_ref += ref.astype(np.float64).sum(axis=1)
                    l1 += np.abs(ref).astype(np.float64).sum(axis=1)
            worst_y = max(worst_y, float(oracle.row_rel_err(y.float().cpu().numpy(), ref).max()))
            # every output element is within 1e-2 of its row's scale, so the sum of sums is within 1e-2 of the L1 mass
            worst_cs = max(worst_cs, float((np.abs(cs.cpu().numpy() - cs_ref) / np.maximum(l1, 1e-6)).max()))
            assert torch.all(y[idx == -1] == 0) and torch.all(cs[idx == -1] == 0)
        torch.save({"err_y": worst_y, "err_cs": worst_cs, "same": bool(same), "status": _lib.device_status(rank)},
                   os.path.join(out_dir, f"s{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
def test_sharded_stack_cuda(cuda, tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.start_processes(_stack_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True, start_method="spawn")
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), f"s{r}.pt"))
        assert res["status"] == 0 and res["same"]
        assert res["err_y"] <= 1e-2 and res["err_cs"] <= 1e-2, res
