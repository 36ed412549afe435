"""The bounded device wait: it gives up on time, reports through the status word, and the context stays usable."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_expires_reports_and_returns():
    from vexact_b200 import _lib

    lib = _lib.load()
    assert _lib.read_status()[0] == 0
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    _lib.check(lib.b200_selftest_wait_expiry(5000, flag.data_ptr(), _lib.current_stream()), "b200_selftest_wait_expiry")
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert flag.item() == 1                       # the wait returned "expired", the kernel ran to its end
    assert elapsed < 1.0                          # 5 ms limit: nowhere near the 2 s production limit
    code, detail, block, _ = _lib.read_status()   # reading clears the word
    assert (code, detail, block) == (1, 999, 0)
    assert _lib.read_status()[0] == 0
    # the context is intact: a real kernel still runs and is right
    import vexact_b200 as vb
    x = torch.randn(8, 2048, device="cuda").bfloat16()
    w = torch.randn(64, 2048, device="cuda").bfloat16()
    torch.testing.assert_close(vb.linear(x, w).float(), x.float() @ w.float().t(), rtol=2e-2, atol=0.5)
    with pytest.raises(_lib.B200Error):
        _lib.check(lib.b200_selftest_wait_expiry(0, flag.data_ptr(), _lib.current_stream()), "b200_selftest_wait_expiry")
