"""Expert-parallel exchange logic over gloo on CPU (world size 2 and 4): counts exchange, split sizes, row
order, autograd through both all-to-alls, shard/gather of the state dict.  The CUDA row kernels and the
fused expert kernels are replaced by torch-indexing doubles here (there is no GPU in this run); the GPU
test-suite runs the real kernels on one rank."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import expert_parallel as ep


class TorchRowOps:
    @staticmethod
    def route(flat_ids, num_experts, k):
        _, ss = flat_ids.sort(stable=True)
        return ss, flat_ids.bincount(minlength=num_experts).int()

    @staticmethod
    def gather(x, idx, fan_out, coeff=None):
        out = x[idx // fan_out]
        return out if coeff is None else out * coeff[idx].unsqueeze(-1)

    @staticmethod
    def combine(expanded, gates, k):
        e3 = expanded.view(-1, k, expanded.size(1))
        return e3.sum(1) if gates is None else (e3 * gates.view(-1, k, 1)).sum(1)


def eager_local_experts(rows, local_ids, w_fc, w_proj):
    out = torch.zeros(rows.size(0), w_proj.size(1), dtype=rows.dtype)
    for e in range(w_fc.size(0)):
        sel = (local_ids == e).nonzero().flatten()
        if sel.numel():
            out = out.index_add(0, sel, F.linear(kh.swiglu_unchunked_torch(F.linear(rows[sel], w_fc[e])), w_proj[e]))
    return out


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, E, k, H, I, T, result_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        layer = ep.MoE_B200_EP(E, k, H, I, kh.swiglu_unchunked_torch, True, False, 0.05, ops=TorchRowOps, local_experts_fn=eager_local_experts, seed=3)
        full = kh.MoE_Torch(E, k, H, I, kh.swiglu_unchunked_torch, True, False, 0.05)
        full.load_state_dict(layer.full_state_dict())
        # every rank draws all ranks' tokens so that it can evaluate the single-process layer on the union
        gen = torch.Generator().manual_seed(11)
        xs = [torch.randn(T + 3 * r, H, generator=gen) for r in range(world)]  # uneven token counts per rank
        gs = [torch.randn(T + 3 * r, H, generator=gen) for r in range(world)]
        x = xs[rank].clone().requires_grad_(True)
        y, logits = layer(x)
        y.backward(gs[rank])
        layer.allreduce_replicated_grads()

        x_all = torch.cat(xs).requires_grad_(True)
        y_all, _ = full(x_all)
        y_all.backward(torch.cat(gs))
        lo = sum(t.size(0) for t in xs[:rank])
        hi = lo + xs[rank].size(0)
        e0, e1 = rank * layer.e_local, (rank + 1) * layer.e_local
        errs = dict(
            y=(y - y_all[lo:hi]).abs().max().item(),
            dx=(x.grad - x_all.grad[lo:hi]).abs().max().item(),
            d_fc=(layer.c_fc_weight.grad - full.c_fc.weight.grad[e0:e1]).abs().max().item(),
            d_proj=(layer.c_proj_weight.grad - full.c_proj.weight.grad[e0:e1]).abs().max().item(),
            d_gate=(layer.gate.weight.grad - full.gate.weight.grad).abs().max().item(),
        )
        # state dict round trip
        sd = layer.full_state_dict()
        layer.load_full_state_dict(sd)
        sd2 = layer.full_state_dict()
        errs["sd"] = max((sd[n] - sd2[n]).abs().max().item() for n in sd)
        result_queue.put((rank, errs))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,E,k", [(2, 8, 2), (4, 8, 3), (2, 6, 1)])
def test_expert_parallel_matches_single_process_layer(world, E, k):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, E, k, 32, 48, 40, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in results:
        for name, v in errs.items():
            assert v < 2e-5, (rank, name, v)


def mismatched_worker(rank, world, port, q):
    """A rank whose split sizes disagree with its peer must fail on the host, not hang: gloo raises."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        rows = torch.ones(4, 8)
        send = [2, 2]
        recv = [2, 2] if rank == 0 else [3, 1]  # rank 1 expects more rows from rank 0 than are sent
        try:
            ep._AllToAllRows.apply(rows, send, recv, dist.group.WORLD)
            q.put((rank, "no error"))
        except Exception as exc:  # noqa: BLE001
            q.put((rank, type(exc).__name__))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def test_mismatched_split_sizes_fail_on_the_host():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=mismatched_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert any(v != "no error" for v in results.values()), results
