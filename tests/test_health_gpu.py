"""Device-side failure detection: a wait on a peer's flag that nothing ever sets runs out of its budget, the kernel returns
normally with the reason in the status word, and the CUDA context stays usable."""
import time

import pytest
import torch

from gemm_b200 import _native
from gemm_b200.ops import moe
from gemm_b200.parallel.health import DeviceWaitTimeout, check_device

pytestmark = pytest.mark.gpu


def test_expired_flag_wait_reports_and_returns():
    torch.manual_seed(0)
    t, k, hidden = 4, 2, 256
    y = torch.randn(t * k, hidden, device="cuda").bfloat16()
    pair_row = torch.arange(t * k, device="cuda", dtype=torch.int32)
    w = torch.full((t, k), 0.5, device="cuda")
    flag = torch.zeros(8, dtype=torch.int32, device="cuda")           # the "peer" never raises it
    epoch = torch.ones(1, dtype=torch.int32, device="cuda")           # the wait wants flag >= 1
    _native.read_status()                                             # start from a clean status word
    t0 = time.time()
    moe.combine(y, pair_row, w, t, k, wait_flags=flag.data_ptr(), wait_n=1, epoch_ptr=epoch.data_ptr())
    with pytest.raises(DeviceWaitTimeout) as ei:
        check_device()
    dt = time.time() - t0
    st = ei.value.status
    assert st["code"] == 2 and "flag" in st["what"]
    assert st["where"] == 800 and st["aux"][1] == 1 and st["aux"][2] == 0      # site, wanted epoch, seen value
    assert 0.5 < dt < 30.0
    # the context is still usable and the status word is clean again
    out = moe.combine(y, pair_row, w, t, k)
    ref = (y.float().reshape(t, k, hidden) * 0.5).sum(1)
    assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2
    check_device()
