"""The forward entry point that brings its own scratch (``molt_nf4_lora_fwd_static``).

It exists for hosts that cannot allocate device memory at the point where they call the library; it must give
the same result as the regular entry point, call after call, although every call reuses one fixed scratch array
that still holds the previous call's data.  This file sorts last on purpose: a run that stops at the first failure
has then already exercised everything else.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from molt_b200 import _native
from tests.gpu_utils import make_case, run_forward

pytestmark = pytest.mark.gpu


def _static_forward(case, path=_native.PATH_AUTO):
    from molt_b200.methods._linear import weight_desc

    lib = _native.library()
    desc = weight_desc(case.packed, case.state)
    x = case.x.cuda().bfloat16()
    a, b = case.a.cuda(), case.b.cuda()
    y = torch.full((x.shape[0], int(desc.n)), float("nan"), dtype=torch.bfloat16, device="cuda")
    _native.check(lib.molt_nf4_lora_fwd_static(ctypes.byref(desc), x.data_ptr(), a.data_ptr(), b.data_ptr(),
                                               float(case.scaling), int(a.shape[0]), y.data_ptr(), x.shape[0], path,
                                               _native.stream_handle()))
    return y


@pytest.mark.parametrize("n,k,m,rank,nested", [(512, 256, 200, 16, False), (1536, 896, 300, 8, True),
                                               (256, 128, 4, 16, False), (70, 65, 5, 7, False)])
def test_static_scratch_forward_equals_workspace_forward_twice(native_library, n, k, m, rank, nested):
    case = make_case(n, k, m, rank, seed=77, nested=nested, order="high-first" if nested else "low-first")
    want, _ = run_forward(case)
    first = _static_forward(case)
    # a different problem in between leaves other data in the shared scratch
    other = make_case(256, 192, 96, 33, seed=5)
    _static_forward(other)
    second = _static_forward(case)
    torch.cuda.synchronize()
    assert _native.read_status() == 0
    # same kernels, same inputs: the results are identical, not merely close
    assert torch.equal(first, want)
    assert torch.equal(second, want)


def test_static_scratch_refuses_problems_that_do_not_fit(native_library):
    case = make_case(256, 128, 8, 16)
    from molt_b200.methods._linear import weight_desc

    lib = _native.library()
    desc = weight_desc(case.packed, case.state)
    huge_m = 1 << 20   # the low-rank product alone would need 128 MiB
    rc = lib.molt_nf4_lora_fwd_static(ctypes.byref(desc), 256, 256, 256, 1.0, 16, 256, huge_m, _native.PATH_AUTO, 0)
    assert rc == _native.E_VALUE
    assert b"built-in scratch" in lib.molt_last_error()
