"""The failure path on a live GPU, without faulting it: a bounded device-side wait expires, the kernel reports it in the
status word and returns, the host reads MIMK_E_DEVICE_WAIT, and the context keeps working."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_expires_and_is_reported():
    from mimir_b200 import MimkError, _lib
    from mimir_b200 import tensor as T
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    assert L.mimk_device_status(stream) == 0
    # ~1 ms of SM clocks: nothing ever arrives on the barrier, so the wait must give up
    assert L.mimk_selftest_wait_expiry(2_000_000, stream) == 0
    assert L.mimk_device_status(stream) == _lib.E_DEVICE_WAIT
    assert L.mimk_device_status(stream) == 0                      # the flag is cleared by the read
    with pytest.raises(MimkError) as e:
        L.mimk_selftest_wait_expiry(2_000_000, stream)
        T.device_status()
    assert e.value.status == _lib.E_DEVICE_WAIT
    # the context is intact: a real kernel runs and gives the right answer afterwards
    a = torch.eye(128, dtype=torch.bfloat16, device="cuda")
    b = torch.randn(128, 256, device="cuda").to(torch.bfloat16)
    assert torch.equal(T.product_2d(a, b), b)
    T.device_status()
    assert L.mimk_selftest_wait_expiry(-1, stream) == 1
