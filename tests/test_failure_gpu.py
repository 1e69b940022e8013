"""Bounded device-side waits report through the status word instead of hanging or trapping."""
import time

import pytest
import torch

from burn_dragon_b200.ops import native
from burn_dragon_b200.parallel import watchdog

pytestmark = pytest.mark.gpu


def test_wait_on_flag_nobody_sets_times_out_and_context_survives():
    native.load()
    native.clear_status()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.time()
    native.ops.wait_timeout_probe(flag, 1, 50_000_000)          # wait at most 50 ms for a value that never comes
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert native.status_code() == 5                            # peer flag wait timed out
    with pytest.raises(watchdog.KernelTimeout):
        watchdog.device_status()
    assert native.status_code() == 0                            # cleared by the exception path
    # the context is still usable
    a = torch.ones(1024, device="cuda")
    assert float((a * 2).sum()) == 2048.0
    # a flag that is already set returns at once with a clean status
    flag.fill_(3)
    native.ops.wait_timeout_probe(flag, 1, 50_000_000)
    torch.cuda.synchronize()
    assert native.status_code() == 0
