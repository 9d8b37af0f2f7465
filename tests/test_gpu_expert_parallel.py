"""Expert-parallel layer on the GPU with this package's kernels (row gather, combine, routing sort, fused experts).
One rank over NCCL, with the row exchange done either by NCCL all-to-all or by this package's peer-memory kernels
(symmetric memory; the peer table then holds the rank's own buffer): every exchange is a self-exchange, so the whole data path (pack, all-to-all calls, local expert
ids, un-sort, gate-weighted combine, and the backward of each) runs on the device and is compared with the
single-GPU layer holding the same weights.  Multi-rank exchange logic is covered by the gloo tests on CPU, and by the two-rank test at the end of this file where
two GPUs are visible (the benchmark runs the same self check at every N > 1)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import _lib
from kernel_hyperdrive_b200.expert_parallel import MoE_B200_EP

from helpers import rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def single_rank_group():
    if dist.is_initialized():
        yield dist.group.WORLD
        return
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(0)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    yield dist.group.WORLD
    dist.destroy_process_group()


@pytest.mark.parametrize("world,rank,E", [(1, 0, 8), (2, 1, 8), (4, 2, 64), (8, 0, 256), (8, 7, 128), (16, 5, 256)])
def test_plan_kernel_matches_the_tensor_formulas(world, rank, E):
    """`b200moe_ep_plan` (one launch) against the same tables written as tensor operations: counts of several ranks with
    empty experts, bit-exact."""
    from kernel_hyperdrive_b200.expert_parallel import CudaRowOps

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(world * 1000 + rank * 10 + E)
    counts_all = torch.randint(0, 300, (world, E), generator=g, dtype=torch.int32)
    counts_all[torch.rand(world, E, generator=g) < 0.2] = 0  # empty experts
    counts_all[:, E // 2] = 0
    M = int(counts_all[rank].sum())
    ss = torch.randperm(M, generator=g)
    counts_all, ss = counts_all.to(dev), ss.to(dev)
    start, base, dest_pos, local_offsets, summary, inv = CudaRowOps.plan_tables(counts_all.reshape(-1).contiguous(), ss, world, rank, E)
    _lib.check_status(dev)

    e_local = E // world
    ca = counts_all.long()
    to_rank = ca.view(world, world, e_local).sum(-1)
    assert torch.equal(start.long(), torch.cat([torch.zeros(1, dtype=torch.long, device=dev), to_rank[rank].cumsum(0)]))
    assert torch.equal(base.long(), (to_rank.cumsum(0) - to_rank)[rank])
    total = ca.sum(0)
    pv = ((total + 127) // 128 * 128).view(world, e_local)
    pad_start = (pv.cumsum(1) - pv).reshape(-1)
    before = (ca.cumsum(0) - ca)[rank]
    own = ca[rank]
    excl = own.cumsum(0) - own
    se = torch.repeat_interleave(torch.arange(E, device=dev), own, output_size=M)
    assert torch.equal(dest_pos.long(), pad_start[se] + before[se] + (torch.arange(M, device=dev) - excl[se]))
    assert torch.equal(local_offsets, total[rank * e_local : (rank + 1) * e_local].cumsum(0))
    assert summary.tolist() == [int(to_rank.sum(0)[rank]), int(pv.sum(1).max())]
    ref_inv = torch.empty_like(ss)
    ref_inv[ss] = torch.arange(M, device=dev)
    assert torch.equal(inv, ref_inv)


@pytest.mark.parametrize("exchange", ["nccl", "p2p", "p2p_received_order", "p2p_no_host_read", "p2p_pipelined"])
@pytest.mark.parametrize("dtype,E,k,H,I,T", [(torch.float32, 8, 2, 128, 256, 300), (torch.bfloat16, 8, 2, 512, 1024, 1000), (torch.bfloat16, 16, 4, 256, 384, 777)])
def test_single_rank_expert_parallel_matches_single_gpu_layer(single_rank_group, exchange, dtype, E, k, H, I, T):
    dev = torch.device("cuda", 0)
    ep = MoE_B200_EP(E, k, H, I, kh.swiglu_unchunked_torch, True, False, 0.05, group=single_rank_group, device=dev, dtype=dtype, seed=2,
                     exchange=exchange.split("_")[0], exchange_rows=(T * k + 127) // 128 * 128 + 256, sync_free=exchange == "p2p_no_host_read",
                     micro_batches=2 if exchange == "p2p_pipelined" else 1, direct=exchange in ("p2p", "p2p_pipelined"))
    ref = kh.MoE_B200(E, k, H, I, kh.swiglu_unchunked_torch, True, False, 0.05).to(dev).to(dtype)
    ref.load_state_dict(ep.full_state_dict())
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, H, generator=g).to(dev, dtype)
    gy = torch.randn(T, H, generator=g).to(dev, dtype)
    outs = []
    for layer in (ref, ep):
        xr = x.clone().requires_grad_(True)
        y, logits = layer(xr)
        y.backward(gy)
        if layer is ref:
            grads = (ref.c_fc.weight.grad, ref.c_proj.weight.grad, ref.gate.weight.grad)
        else:
            grads = (ep.c_fc_weight.grad, ep.c_proj_weight.grad, ep.gate.weight.grad)
        outs.append((y.detach(), xr.grad) + grads)
    _lib.check_status(dev)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for a, b, name in zip(outs[1], outs[0], ("y", "dx", "d_w_fc", "d_w_proj", "d_gate")):
        assert rel_l2(a, b) < (tol if name != "d_gate" else 20 * tol), (name, rel_l2(a, b))


def _two_rank_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from kernel_hyperdrive_b200.expert_parallel import parity_selfcheck

        q.put((rank, parity_selfcheck(dist.group.WORLD, dev)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_exchange_matches_single_gpu_layer():
    """Two ranks, one GPU each: rows really cross between GPUs (peer stores / loads and the bounded barrier kernel, and
    the NCCL all-to-all), uneven token counts, contiguous and strided placement; compared with the single-GPU layer."""
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_two_rank_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, rep in results:
        assert rep["ok"], (rank, rep)
        assert len(rep["cases"]) == 9
