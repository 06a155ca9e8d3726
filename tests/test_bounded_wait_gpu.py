"""The bounded device-side wait reports instead of hanging: a wait that nothing completes runs out, leaves its code in
the status word, and the context stays usable (no fault, trap or endless loop is involved)."""
import time

import pytest
import torch

from turbodeberta_b200 import _cabi as cabi
from turbodeberta_b200.ops import flash_attention as fa

pytestmark = pytest.mark.gpu


def test_wait_that_nothing_completes_is_reported():
    dev = torch.device("cuda")
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    t0 = time.time()
    with torch.cuda.device(dev):
        cabi.check(cabi.lib.tdb_selftest_bounded_wait(cabi.ptr(status), 77, 2000, cabi.stream_ptr(dev)))
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0                        # 2 ms limit, not the kernels' 1 s
    assert status.tolist() == [77, 0, 0, 0]
    with pytest.raises(cabi.TdbError) as err:            # what the ops do with such a status word
        fa._check_status(status)
    assert err.value.code == cabi.ERR_TIMEOUT
    # the context is still usable: a normal call right after
    q = torch.randn(1, 2, 64, 64, device=dev, dtype=torch.bfloat16)
    o = fa.flash_attention_with_disentangled(q, q, q, None, None)
    assert torch.isfinite(o.float()).all()


def test_selftest_argument_errors():
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert cabi.lib.tdb_selftest_bounded_wait(None, 1, 10, None) == cabi.ERR_ARG
    assert cabi.lib.tdb_selftest_bounded_wait(cabi.ptr(status), 0, 10, None) == cabi.ERR_ARG
    assert cabi.lib.tdb_selftest_bounded_wait(cabi.ptr(status), 1, 10 ** 7, None) == cabi.ERR_ARG
