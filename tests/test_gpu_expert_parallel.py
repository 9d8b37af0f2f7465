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
