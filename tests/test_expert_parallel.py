"""Expert-parallel exchange logic over gloo on CPU (world size 2 and 4): counts exchange, split sizes, row
order, autograd through both exchanges, shard/gather of the state dict, expert placement.  The CUDA row kernels and
the fused expert kernels are replaced by torch-indexing doubles here (there is no GPU in this run).  Both exchanges
are covered: the all-to-all one, and the peer-memory one, whose push / pull kernels are replaced by doubles that move
rows between per-rank shared host tensors with the same placement arithmetic as the kernels
(destination = the range of `start` a row falls in, position = base[d] + n - start[d]).  The GPU test-suite runs the
real kernels on one rank, and on two ranks where two GPUs are visible."""

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


class TorchPeerExchange:
    """Stand-in for `PeerExchange` on CPU: every rank's buffers are shared host tensors visible to all ranks, `push`
    and `pull` follow the kernels of csrc/ep.cu row by row, `barrier` is the process-group barrier."""

    def __init__(self, group, shared, cap_rows):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        self.shared, self.cap_rows = shared, cap_rows
        self.bufs = {name: shared[name][self.rank] for name in shared}
        self.backward_reads_pending = False
        self.direct = False
        self.barriers = 0
        self.skipped = 0

    def barrier(self):
        self.barriers += 1
        dist.barrier(self.group)

    def _dest(self, plan, n):
        d = torch.searchsorted(plan.start[1 : self.world].long().contiguous(), n, right=True)
        if plan.dest_pos is not None:  # rows go to their place in the receiver's padded grouped order
            return d, plan.dest_pos.long()[n]
        return d, plan.base.long()[d] + n - plan.start.long()[d]

    def zero_fillers(self, name, plan):
        counts = torch.diff(plan.local_offsets, prepend=plan.local_offsets.new_zeros(1))
        seg = 0
        for c in counts.tolist():
            pad = (c + 127) // 128 * 128
            self.bufs[name][seg + c : seg + pad] = 0
            seg += pad

    def push(self, name, src, idx, fan_out, coeff, plan):
        n = torch.arange(plan.ss.numel())
        d, pos = self._dest(plan, n)
        s_ = idx if idx is not None else n
        rows = src[s_ // fan_out]
        if coeff is not None:
            rows = rows * coeff[s_].unsqueeze(-1)
        for dest in range(self.world):
            sel = (d == dest) & (pos < self.cap_rows)
            self.skipped += int(((d == dest) & (pos >= self.cap_rows)).sum())
            self.shared[name][dest][pos[sel]] = rows[sel].detach()

    def pull(self, name, gates, out, expanded, plan):
        T, k = out.size(0), plan.k
        d, pos = self._dest(plan, plan.inv)
        zero = out.new_zeros(out.size(1))  # a row that did not fit into the owner's buffer was never stored
        rows = torch.stack([self.shared[name][int(di)][int(pi)] if pi < self.cap_rows else zero for di, pi in zip(d.tolist(), pos.tolist())]) if d.numel() else out.new_zeros(0, out.size(1))
        if expanded is not None:
            expanded.copy_(rows)
        r3 = rows.view(T, k, -1)
        out.copy_(r3.sum(1) if gates is None else (r3 * gates.view(T, k, 1)).sum(1))


def eager_grouped_experts(x_rows, offsets, w_fc, w_proj):
    """Local experts on rows in the padded grouped order (segments start at multiples of 128 rows)."""
    counts = torch.diff(offsets, prepend=offsets.new_zeros(1)).tolist()
    out = torch.zeros(x_rows.size(0), w_proj.size(1), dtype=x_rows.dtype)
    seg = 0
    for e, c in enumerate(counts):
        sel = torch.arange(min(seg, x_rows.size(0)), min(seg + c, x_rows.size(0)))  # clipped where the buffer ends (an overflowing pass is refused later)
        if sel.numel():
            out = out.index_add(0, sel, F.linear(kh.swiglu_unchunked_torch(F.linear(x_rows[sel], w_fc[e])), w_proj[e]))
        seg += (c + 127) // 128 * 128
    return out


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


def worker(rank, world, port, E, k, H, I, T, result_queue, shared=None, cap_rows=0, placement=None, direct=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        load = [1.0 / (e + 1) for e in range(E)] if placement == "balanced" else None
        layer = ep.MoE_B200_EP(E, k, H, I, kh.swiglu_unchunked_torch, True, False, 0.05, ops=TorchRowOps, seed=3,
                               local_experts_fn=eager_grouped_experts if direct else eager_local_experts, placement=placement, expected_load=load)
        if shared is not None:
            layer.exchange = TorchPeerExchange(dist.group.WORLD, shared, cap_rows)
            layer.exchange.direct = direct
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
        d_fc, d_proj, mine = layer.expert_grads_in_expert_order()
        errs = dict(
            y=(y - y_all[lo:hi]).abs().max().item(),
            dx=(x.grad - x_all.grad[lo:hi]).abs().max().item(),
            d_fc=(d_fc - full.c_fc.weight.grad[mine]).abs().max().item(),
            d_proj=(d_proj - full.c_proj.weight.grad[mine]).abs().max().item(),
            d_gate=(layer.gate.weight.grad - full.gate.weight.grad).abs().max().item(),
        )
        if shared is not None:
            errs["skipped_rows"] = float(layer.exchange.skipped)
            errs["barriers_not_4"] = float(layer.exchange.barriers != 4)  # rows landed, y written, dy landed, dx written
        # state dict round trip
        sd = layer.full_state_dict()
        layer.load_full_state_dict(sd)
        sd2 = layer.full_state_dict()
        errs["sd"] = max((sd[n] - sd2[n]).abs().max().item() for n in sd)
        result_queue.put((rank, errs))
    finally:
        dist.destroy_process_group()


def shared_exchange_buffers(world, cap_rows, H):
    return {name: [torch.zeros(cap_rows, H).share_memory_() for _ in range(world)] for name in ("x", "y", "dy", "dx")}


CASES = (
    [(w, E, k, pl, "peer_direct") for (w, E, k, pl) in [(2, 8, 2, None), (4, 8, 3, None), (2, 6, 1, None), (4, 8, 2, "strided"), (2, 8, 3, "balanced")]]
    + [(w, E, k, pl, "all_to_all") for (w, E, k, pl) in [(2, 8, 2, None), (4, 8, 3, None), (2, 6, 1, "strided")]]
    + [(w, E, k, pl, "peer") for (w, E, k, pl) in [(2, 8, 2, None), (4, 8, 2, "balanced")]]
)


@pytest.mark.parametrize("world,E,k,placement,exchange", CASES)
def test_expert_parallel_matches_single_process_layer(world, E, k, placement, exchange):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    T, H = 40, 32
    cap_rows = (T + 3 * world) * k * world + 128 * (E // world)  # every row of every rank could land on one rank, plus filler rows
    shared = shared_exchange_buffers(world, cap_rows, H) if exchange != "all_to_all" else None
    procs = [ctx.Process(target=worker, args=(r, world, port, E, k, H, 48, T, q, shared, cap_rows, placement, exchange == "peer_direct")) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in results:
        for name, v in errs.items():
            assert v < 2e-5, (rank, name, v)


def overflow_worker(rank, world, port, q, shared, cap_rows, direct=False):
    """Exchange buffers too small for the busiest rank: every rank must refuse the pass (no rank may go on to a
    barrier the others never reach), and the rows that did not fit must have been skipped, not written."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    try:
        E, k, H, I, T = 4, 2, 16, 24, 24
        layer = ep.MoE_B200_EP(E, k, H, I, kh.swiglu_unchunked_torch, True, False, 0.05, ops=TorchRowOps, seed=1,
                               local_experts_fn=eager_grouped_experts if direct else eager_local_experts)
        layer.exchange = TorchPeerExchange(dist.group.WORLD, shared, cap_rows)
        layer.exchange.direct = direct
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(rank))
        # every token of every rank picks experts 0 and 1: rank 0 receives all 2 * T * world rows
        sel = torch.tensor([[0, 1]]).expand(T, 2).contiguous()
        rw = torch.full((T, 2), 0.5)
        try:
            layer._compute_experts(x, rw, sel)
            q.put((rank, "no error", layer.exchange.barriers))
        except RuntimeError as exc:
            q.put((rank, "refused" if "exchange buffer too small" in str(exc) else repr(exc), layer.exchange.barriers))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("direct", [False, True])
def test_exchange_overflow_is_refused_by_every_rank_together(direct):
    world, cap_rows = 2, 40  # rank 0 would receive 2 * 24 * 2 = 96 rows
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    shared = shared_exchange_buffers(world, cap_rows, 16)
    procs = [ctx.Process(target=overflow_worker, args=(r, world, port, q, shared, cap_rows, direct)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(r[1] == "refused" for r in results), results
    assert len({r[2] for r in results}) == 1, results  # the ranks passed the same number of barriers


def test_placement_helpers():
    assert ep.make_placement(None, 8, 2) is None
    strided = ep.make_placement("strided", 8, 4)
    assert (strided // 2).tolist() == [0, 1, 2, 3, 0, 1, 2, 3]  # expert e on rank e % 4
    load = [100.0] + [1.0] * 15
    bal = ep.make_placement("balanced", 16, 4, load)
    assert sorted(bal.tolist()) == list(range(16))
    per_rank = [sum(load[e] for e in range(16) if bal[e] // 4 == r) for r in range(4)]
    assert max(per_rank) == 103.0 and min(per_rank) == 4.0  # the heavy expert sits with three light ones
    with pytest.raises(AssertionError):
        ep.make_placement([0, 0, 1, 2], 4, 2)


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
