"""The routing entry point for callers that cannot allocate device memory (b200moe_route_static).

A host that owns all device memory through its own arena cannot give the library a workspace from
cudaMalloc, so this variant of the routing call keeps its scratch in a fixed array inside the library.
The test drives it through the C ABI exactly as such a host would (raw pointers, no Python wrapper) and
checks, on two calls in a row that share the array, that every output equals what the ordinary entry
point (caller-owned workspace) produces for the same ids.  Integer outputs: bit-exact.
The file name sorts last so that a run stopping at the first failure has already run everything else.
"""

import pytest
import torch

from kernel_hyperdrive_b200 import _lib
from kernel_hyperdrive_b200._lib import lib, ptr, status_word, stream_ptr

pytestmark = pytest.mark.gpu


def _outputs(M, E, cap, dev):
    return dict(
        se=torch.full((M,), -7, dtype=torch.int64, device=dev),
        ss=torch.full((M,), -7, dtype=torch.int64, device=dev),
        off=torch.full((E,), -7, dtype=torch.int64, device=dev),
        cnt=torch.full((E,), -7, dtype=torch.int32, device=dev),
        row_token=torch.full((cap,), -7, dtype=torch.int32, device=dev),
        row_slot=torch.full((cap,), -7, dtype=torch.int32, device=dev),
    )


def _route_with_workspace(ids, E, k):
    L, dev, M = lib(), ids.device, ids.numel()
    cap = L.b200moe_padded_rows_cap(M, E)
    o = _outputs(M, E, cap, dev)
    ws = torch.empty(L.b200moe_route_workspace_bytes(M, E), dtype=torch.uint8, device=dev)
    rc = L.b200moe_route(ptr(ids), M, E, k, ptr(o["se"]), ptr(o["ss"]), ptr(o["off"]), ptr(o["cnt"]), ptr(o["row_token"]), ptr(o["row_slot"]), cap, ptr(ws), ws.numel(), ptr(status_word(dev)), stream_ptr(dev))
    assert rc == 0, L.b200moe_last_error_detail()
    return o


def _route_static(ids, E, k):
    L, dev, M = lib(), ids.device, ids.numel()
    cap = L.b200moe_padded_rows_cap(M, E)
    o = _outputs(M, E, cap, dev)  # the caller's output buffers exist before the call; the call itself allocates nothing
    rc = L.b200moe_route_static(ptr(ids), M, E, k, ptr(o["se"]), ptr(o["ss"]), ptr(o["off"]), ptr(o["cnt"]), ptr(o["row_token"]), ptr(o["row_slot"]), cap, ptr(status_word(dev)), stream_ptr(dev))
    assert rc == 0, L.b200moe_last_error_detail()
    return o


def test_route_static_matches_route_on_two_consecutive_calls():
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(5)
    cases = [(64, 6, 5000), (8, 2, 16384)]  # different E and M back to back: the second call finds the first one's scratch
    ids = [torch.randint(0, E, (T * k,), generator=g).to(dev) for E, k, T in cases]
    want = [_route_with_workspace(i, E, k) for i, (E, k, T) in zip(ids, cases)]
    got = [_route_static(i, E, k) for i, (E, k, T) in zip(ids, cases)]  # two calls in a row, nothing in between
    torch.cuda.synchronize()
    for w, g_, i, (E, k, T) in zip(want, got, ids, cases):
        for name in w:
            assert torch.equal(w[name], g_[name]), (name, E, k, T)
        ref_se, ref_ss = i.cpu().sort(stable=True)
        assert torch.equal(g_["se"].cpu(), ref_se) and torch.equal(g_["ss"].cpu(), ref_ss)
    _lib.check_status(dev)


def test_route_static_refuses_sizes_beyond_its_array():
    L, dev = lib(), torch.device("cuda")
    limit = L.b200moe_route_static_scratch_bytes()
    assert limit == 256 * 1024
    E, M = 512, 1 << 20
    assert L.b200moe_route_workspace_bytes(M, E) > limit
    ids = torch.zeros(8, dtype=torch.int64, device=dev)  # never read: the size check comes first
    before = L.b200moe_launch_count()
    rc = L.b200moe_route_static(ptr(ids), M, E, 8, None, None, None, None, None, None, 0, None, stream_ptr(dev))
    assert rc == -6
    msg = L.b200moe_last_error_detail().decode()
    assert "262144" in msg and "b200moe_route" in msg
    assert L.b200moe_launch_count() == before
