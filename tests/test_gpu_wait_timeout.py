"""A bounded device-side wait that runs out, without a fault.

Every mbarrier wait of the TMA / tcgen05 kernels gives up after a time limit, records a code in a per-device status
word, makes the rest of its CTA leave through an abort flag, lets copies in flight land, frees tensor memory and
returns; wino_device_status() turns the record into WINO_E_TIMEOUT.  In production those waits never run out, so
this test drives the same primitives through wino_selftest_wait_timeout: a CTA whose producer waits on an mbarrier
that nothing arrives on, with a limit of a few milliseconds.  The kernel must end by itself, the status must read
WINO_E_TIMEOUT exactly once, and the library must work normally afterwards.
"""
import time

import numpy as np
import pytest

import oracle
from util import make_inputs, maxrel, run_conv

pytestmark = pytest.mark.gpu


def test_wait_runs_out_and_the_context_stays_usable():
    import torch
    assert torch.cuda.is_available()
    import cudnntest_b200 as cb
    L = cb.lib()
    assert L.wino_device_status() == cb._lib.OK
    assert L.wino_selftest_wait_timeout(0, None) == cb._lib.E_BADARG          # limits outside 1 ... 1000 ms are refused
    t0 = time.perf_counter()
    assert L.wino_selftest_wait_timeout(5, None) == cb._lib.OK
    assert L.wino_device_status() == cb._lib.E_TIMEOUT                        # synchronises: the kernel returned by itself
    assert time.perf_counter() - t0 < 1.5                                     # a 5 ms limit, not the 2 s production limit
    assert b"code 90" in L.wino_last_error_string()
    assert L.wino_device_status() == cb._lib.OK                               # the record was cleared by the read
    # tensor memory was freed and nothing is stuck: a tensor-core convolution runs and is right
    x, wt, b = make_inputs(2, 64, 16, 16, 64, seed=5)
    y = run_conv(x, wt, b, "NHWC", dtype="bf16", relu=True, wino=4)
    ref = oracle.conv_f64(x, wt, bias=b, relu=True)
    d = y.astype(np.float64) - ref
    assert np.sqrt((d * d).sum() / (ref * ref).sum()) <= 5e-3
    with pytest.raises(cb.WinoError):                                        # the Python wrapper raises on the same record
        assert L.wino_selftest_wait_timeout(2, None) == cb._lib.OK
        cb.device_status()
    assert L.wino_device_status() == cb._lib.OK
