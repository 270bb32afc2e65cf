"""Device-side failure detection: a wait that cannot complete expires after its budget, the
kernel exits normally, and the host reads a status code; the context stays usable."""
import time

import pytest
import torch

from ffn_kernel_b200 import MaskedLinear, check_status
from ffn_kernel_b200._lib import FfnkError, lib
from ffn_kernel_b200.route import status_word, stream_ptr
from ffn_kernel_b200.synth import linear_case

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_and_context_survives(dev):
    check_status()
    L = lib()
    t0 = time.time()
    assert L.ffnk_selftest_bounded_wait(status_word(dev).data_ptr(), 20000, stream_ptr(dev)) == 0   # 20 ms budget
    with pytest.raises(FfnkError) as e:
        check_status()
    assert e.value.code == 6 and time.time() - t0 < 5.0
    check_status()                     # the word was cleared by the read
    c = linear_case(256, 64, 64, seed=0).to(dev)
    y = MaskedLinear.apply(c.x, c.wv.T, c.wt.T, c.mask)
    check_status()
    assert bool(torch.isfinite(y.float()).all())


def test_selftest_rejects_bad_budget(dev):
    assert lib().ffnk_selftest_bounded_wait(status_word(dev).data_ptr(), 0, stream_ptr(dev)) == -2
    assert lib().ffnk_selftest_bounded_wait(None, 10, stream_ptr(dev)) == -1
