"""Failure detection without a GPU fault: a bounded wait that runs out (a barrier nothing arrives on) must end the
kernel normally, leave a code in the status word, surface as an error on the host and leave the context usable."""

import pytest
import torch

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import _lib
from kernel_hyperdrive_b200._lib import lib, ptr, status_word, stream_ptr

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reports():
    dev = torch.device("cuda")
    status = status_word(dev)
    _lib.check_status(dev)  # clean start
    finished = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib().b200moe_selftest_bounded_wait(ptr(status), 100_000_000, ptr(finished), stream_ptr(dev))  # about 50 ms
    assert rc == 0
    with pytest.raises(_lib.B200MoEError, match="299"):
        _lib.check_status(dev)
    assert finished.item() == 1  # the waiting thread gave up and the kernel ran to its end
    _lib.check_status(dev)  # the word was cleared; nothing is pending
    # the context is intact: a normal operator still runs and is exact
    x = torch.randint(0, 9, (1000,), device=dev)
    assert torch.equal(kh.contiguous_count_cute(x, 9).cpu(), x.cpu().bincount(minlength=9).int())


def test_status_word_flags_out_of_range_expert_ids():
    dev = torch.device("cuda")
    ids = torch.tensor([0, 1, 7, 2], dtype=torch.int64, device=dev)  # 7 is not an expert of a 4-expert layer
    kh.route(ids, 4, 1, True, False)
    with pytest.raises(_lib.B200MoEError, match="101"):
        _lib.check_status(dev)
    _lib.check_status(dev)
