"""Routing integers on the GPU: bit-exact against torch.sort(stable=True) / bincount / cumsum, against
the CPU oracle and against the golden fixtures."""

import os

import numpy as np
import pytest
import torch

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import _lib
from oracle import moe_oracle as orc

from conftest import GOLDEN
from helpers import segments_equal_as_sets

pytestmark = pytest.mark.gpu


def sizes_1d():
    # the sweep of the reference's own histogram test: powers of two, their neighbours and odd sizes
    out = set()
    for p in range(0, 17, 2):
        for d in (-1, 0, 1):
            if 2**p + d > 0:
                out.add(2**p + d)
    out.update([7, 100, 1000, 4097, 12345, 70001])
    return sorted(out)


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32])
def test_contiguous_count_exact(dtype):
    g = torch.Generator().manual_seed(42)
    for n in sizes_1d():
        x = torch.randint(0, 72, (n,), generator=g, dtype=dtype)
        got = kh.contiguous_count_cute(x.cuda(), 72)
        assert got.dtype == torch.int32 and got.shape == (72,)
        assert torch.equal(got.cpu(), x.long().bincount(minlength=72).int()), n
    _lib.check_status(torch.device("cuda"))


def test_contiguous_count_empty_and_wide():
    assert kh.contiguous_count_cute(torch.zeros(0, dtype=torch.long, device="cuda"), 5).sum().item() == 0
    x = torch.randint(0, 20000, (50000,))
    assert torch.equal(kh.contiguous_count_cute(x.cuda(), 20000).cpu(), x.bincount(minlength=20000).int())


@pytest.mark.parametrize("E,k,T", [(1, 1, 1), (4, 2, 48), (8, 2, 256), (6, 1, 19), (64, 6, 777), (128, 8, 4096), (256, 8, 8192), (512, 4, 3000), (8, 2, 16384)])
def test_route_bit_exact(E, k, T):
    g = torch.Generator().manual_seed(E * 1000 + T)
    if E >= k:
        ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(min(T, 512))])
        ids = ids.repeat((T + ids.size(0) - 1) // ids.size(0), 1)[:T]
    else:
        ids = torch.randint(0, E, (T, k), generator=g)
    flat = ids.flatten()
    se, ss, off, cnt, row_token, row_slot = kh.route(flat.cuda(), E, k, True, True)
    ref_se, ref_ss = flat.sort(stable=True)
    assert torch.equal(se.cpu(), ref_se) and torch.equal(ss.cpu(), ref_ss)
    assert off.dtype == torch.int64 and torch.equal(off.cpu(), flat.bincount(minlength=E).cumsum(-1))
    assert cnt.dtype == torch.int32 and torch.equal(cnt.cpu(), flat.bincount(minlength=E).int())
    o_se, o_ss, o_off, o_cnt = orc.route(ids.numpy(), E)
    assert np.array_equal(se.cpu().numpy(), o_se) and np.array_equal(ss.cpu().numpy(), o_ss) and np.array_equal(off.cpu().numpy(), o_off)
    # an unstable sort (what the reference calls) agrees segment by segment
    u_se, u_ss = flat.sort()
    assert segments_equal_as_sets(u_se.numpy(), u_ss.numpy(), ss.cpu().numpy())
    # row maps of the padded grouped order
    pad = orc.padded_layout(o_cnt)
    rt, rs = row_token.cpu().numpy(), row_slot.cpu().numpy()
    assert rt.shape[0] == kh.scattermoe.padded_rows_cap(T * k, E) >= pad[-1]
    expect_slot = np.full_like(rs, -1)
    start = 0
    for e in range(E):
        expect_slot[pad[e] : pad[e] + o_cnt[e]] = o_ss[start : start + o_cnt[e]]
        start += o_cnt[e]
    assert np.array_equal(rs, expect_slot)
    assert np.array_equal(rt, np.where(expect_slot >= 0, expect_slot // k, -1))
    _lib.check_status(torch.device("cuda"))


def test_route_skewed_with_empty_experts():
    E, k, T = 128, 8, 8192
    p = torch.arange(1, E + 1, dtype=torch.float64).pow(-1.2)
    ids = torch.multinomial((p / p.sum()).expand(T, E), k, replacement=False, generator=torch.Generator().manual_seed(0))
    ids[ids >= 100] = 3  # leave experts 100.. without rows
    flat = ids.flatten()
    se, ss, off, cnt, _, _ = kh.route(flat.cuda(), E, k, True, False)
    ref_se, ref_ss = flat.sort(stable=True)
    assert torch.equal(se.cpu(), ref_se) and torch.equal(ss.cpu(), ref_ss)
    assert (cnt.cpu()[100:] == 0).all() and off.cpu()[-1].item() == T * k


@pytest.mark.parametrize("name", ["tiny", "c1", "ragged"])
def test_route_matches_golden(name):
    gold = dict(np.load(os.path.join(GOLDEN, f"{name}.npz")))
    sel = torch.from_numpy(gold["selected_experts"])
    E = len(gold["expert_offsets"])
    se, ss, off, _, _, _ = kh.route(sel.flatten().cuda(), E, sel.size(1), True, False)
    assert np.array_equal(se.cpu().numpy(), gold["sorted_expert_idxs"])
    assert np.array_equal(ss.cpu().numpy(), gold["sorted_scattered_idxs"])
    assert np.array_equal(off.cpu().numpy(), gold["expert_offsets"])


def test_route_full_size_properties():
    """Largest benchmark configuration (256 experts, top-8, 131072 tokens): sortedness, permutation, counts."""
    E, k, T = 256, 8, 131072
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(1))
    flat = logits.topk(k, dim=-1).indices.flatten().cuda()
    se, ss, off, cnt, row_token, row_slot = kh.route(flat, E, k, True, True)
    assert (se[1:] >= se[:-1]).all()
    assert torch.equal(ss.sort().values, torch.arange(T * k, device="cuda"))
    assert torch.equal(flat[ss], se)
    same = se[1:] == se[:-1]
    assert (ss[1:][same] > ss[:-1][same]).all()  # stable
    assert torch.equal(off, torch.bincount(flat, minlength=E).cumsum(-1)) and off[-1].item() == T * k
    valid = row_slot >= 0
    assert valid.sum().item() == T * k and torch.equal(row_slot[valid].long(), ss)
    assert torch.equal(row_token[valid], row_slot[valid] // k)
