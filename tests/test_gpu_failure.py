"""Failure reporting of the device-side bounded waits, provoked from the host: nothing here faults or hangs the GPU.

The tensor-core GEMM's producers are told (``MOLT_OPT_WITHHOLD_BLOCKS``) to request one contraction block fewer than the
consumers expect and the wait limit is set to a few milliseconds, so one wait runs out.  The kernel must record the
time-out in the status word, return by itself, leave the context usable, and the next call must be correct again.
"""
from __future__ import annotations

import time

import pytest
import torch

from oracle import molt_oracle as oracle
from molt_b200 import _native
from tests.gpu_utils import TOL, make_case, run_forward

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("height", ["short", "tall"])
def test_bounded_wait_expires_reports_and_recovers(native_library, height):
    path = _native.PATH_TCGEN05 | (_native.PATH_TALL_TILES if height == "tall" else _native.PATH_SHORT_TILES)
    case = make_case(256, 128, 300, 8, seed=2)            # one or two pair tiles of three contraction blocks each
    y_ref = oracle.nf4_lora_forward(case.x, case.weight, case.a, case.b, case.scaling)
    y_good, _ = run_forward(case, path)
    assert _native.read_status() == 0
    _native.set_option(_native.OPT_WAIT_LIMIT_US, 3000)   # 3 ms instead of one second
    try:
        _native.set_option(_native.OPT_WITHHOLD_BLOCKS, 1)
        begin = time.perf_counter()
        run_forward(case, path)
        torch.cuda.synchronize()                          # the kernel returns by itself
        elapsed = time.perf_counter() - begin
        status = _native.read_status()
        assert status != 0 and (status >> 24) == _native.E_TIMEOUT, hex(status)
        assert 1 <= ((status >> 16) & 0xff) <= 9          # one of the GEMM's wait sites
        assert elapsed < 2.0
        assert _native.read_status() == 0                 # reading cleared it
        # the injection applied to one launch only; the context is intact and the next call is right again
        y_again, _ = run_forward(case, path)
        torch.cuda.synchronize()
        assert _native.read_status() == 0
        assert torch.equal(y_again, y_good)
        assert oracle.rel_frobenius(y_again, y_ref) <= TOL
    finally:
        _native.set_option(_native.OPT_WITHHOLD_BLOCKS, 0)
        _native.set_option(_native.OPT_WAIT_LIMIT_US, 1000000)


def test_few_token_kernel_wait_expires_reports_and_recovers(native_library):
    """The same for the few-token kernel: its code producer requests one block fewer than the decoders expect."""
    path = _native.PATH_FEW_TOKENS
    case = make_case(256, 128, 40, 8, seed=3)             # one CTA, two row tiles of two contraction blocks each
    y_ref = oracle.nf4_lora_forward(case.x, case.weight, case.a, case.b, case.scaling)
    y_good, _ = run_forward(case, path)
    assert _native.read_status() == 0
    _native.set_option(_native.OPT_WAIT_LIMIT_US, 3000)
    try:
        _native.set_option(_native.OPT_WITHHOLD_BLOCKS, 1)
        begin = time.perf_counter()
        run_forward(case, path)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - begin
        status = _native.read_status()
        assert status != 0 and (status >> 24) == _native.E_TIMEOUT, hex(status)
        assert 1 <= ((status >> 16) & 0xff) <= 9
        assert elapsed < 2.0
        y_again, _ = run_forward(case, path)
        torch.cuda.synchronize()
        assert _native.read_status() == 0
        assert torch.equal(y_again, y_good)
        assert oracle.rel_frobenius(y_again, y_ref) <= TOL
    finally:
        _native.set_option(_native.OPT_WITHHOLD_BLOCKS, 0)
        _native.set_option(_native.OPT_WAIT_LIMIT_US, 1000000)


def test_option_values_are_checked(native_library):
    with pytest.raises(ValueError):
        _native.set_option(_native.OPT_WAIT_LIMIT_US, 1)
    with pytest.raises(ValueError):
        _native.set_option(_native.OPT_WITHHOLD_BLOCKS, 99)
    with pytest.raises(ValueError):
        _native.set_option(77, 0)
