"""CUDA dequantiser, SwiGLU and RMSNorm kernels against the oracle and the reference-made fixtures."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import molt_oracle as oracle
from tests.conftest import load_golden

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["q_8x8_b16", "q_64x64_b64", "q_70x65_b64", "q_96x64_b64", "q_48x1536_b64",
                                  "q_33x50_b32"])
def test_dequant_matches_reference_fixture_bits(native_library, name):
    from molt_b200.streaming import NF4DevicePayload

    fx = load_golden(name)
    shape = tuple(int(v) for v in fx["shape"])
    payload = NF4DevicePayload(torch.from_numpy(fx["packed"]).cuda(), torch.from_numpy(fx["scales"]).cuda(), shape,
                               int(fx["block"]), int(fx["elements"]))
    got = payload.dequantize(torch.bfloat16).cpu().view(torch.int16).numpy()
    assert np.array_equal(got, fx["deq_bf16_bits"])
    assert np.array_equal(payload.dequantize(torch.float32).cpu().numpy(), fx["deq_f32"])


@pytest.mark.parametrize("order", ["low-first", "high-first"])
@pytest.mark.parametrize("nested", [False, True])
def test_dequant_bit_exact_at_projection_size(native_library, order, nested):
    from molt_b200.methods.nf4_layer_cache import dequantize_nf4
    from tests.gpu_utils import make_case

    case = make_case(1536, 8960, 1, 16, nested=nested, order=order)
    got = dequantize_nf4(case.packed, case.state, torch.bfloat16)
    want = oracle.nf4_dequantize(case.q, torch.bfloat16, case.scales_f32)
    assert oracle.bits_equal_bf16(got, want)


def test_resolved_scales_match_oracle_bits(native_library):
    from molt_b200.methods import resolved_nf4_scales
    from tests.gpu_utils import make_case

    case = make_case(256, 1536, 1, 16, nested=True, order="high-first")
    got = resolved_nf4_scales(case.state).cpu()
    assert torch.equal(got, case.scales_f32)
    assert resolved_nf4_scales(case.state) is resolved_nf4_scales(case.state)  # cached on the state


def test_nf4tensor_roundtrip_is_idempotent_at_full_size(native_library):
    """Size-independent property at a full projection: quantise(dequantise(q)) reproduces the same bytes."""
    from molt_b200.streaming import NF4Tensor

    gen = torch.Generator().manual_seed(1337)
    w = (torch.randn(8960, 1536, generator=gen) * 0.02).cuda()
    q = NF4Tensor.quantize(w, block_size=64)
    dense = q.dequantize(device="cuda", dtype=torch.float32)
    again = NF4Tensor.quantize(dense, block_size=64)
    assert torch.equal(q.packed, again.packed)
    assert torch.equal(q.scales, again.scales)


@pytest.mark.parametrize("name,dtype", [("swiglu_3x5x17_f32", torch.float32), ("swiglu_2x31x128_bf16", torch.bfloat16)])
def test_swiglu_matches_reference_fixture(native_library, name, dtype):
    from molt_b200.kernels.gated_activation import fused_silu_multiply

    fx = load_golden(name)
    gate = torch.from_numpy(fx["gate"]).to(dtype).cuda().requires_grad_()
    up = torch.from_numpy(fx["up"]).to(dtype).cuda().requires_grad_()
    grad = torch.from_numpy(fx["grad"]).to(dtype).cuda()
    out = fused_silu_multiply(gate, up)
    out.backward(grad)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5  # reference tests/kernels/test_gated_activation.py:22
    torch.testing.assert_close(out.detach().float().cpu(), torch.from_numpy(fx["out"]), rtol=tol, atol=tol)
    torch.testing.assert_close(gate.grad.float().cpu(), torch.from_numpy(fx["dgate"]), rtol=tol, atol=tol)
    torch.testing.assert_close(up.grad.float().cpu(), torch.from_numpy(fx["dup"]), rtol=tol, atol=tol)


@pytest.mark.parametrize("shape", [(2, 31, 4864), (1, 7, 5), (0, 16), (3, 1031)])
def test_swiglu_bf16_against_oracle(native_library, shape):
    # shape (2, 31, 4864) and seed are those of reference tests/kernels/test_gated_activation.py:28-42
    from molt_b200.kernels.gated_activation import swiglu_backward, swiglu_forward

    gen = torch.Generator().manual_seed(3402)
    gate = torch.randn(*shape, generator=gen).bfloat16()
    up = torch.randn(*shape, generator=gen).bfloat16()
    grad = torch.randn(*shape, generator=gen).bfloat16()
    h = swiglu_forward(gate.cuda(), up.cuda())
    dg, du, h2 = swiglu_backward(grad.cuda(), gate.cuda(), up.cuda(), want_hidden=True)
    want_h = oracle.swiglu_forward(gate, up)
    want_dg, want_du = oracle.swiglu_backward(grad, gate, up)
    # one rounding from fp32; expf on the device and on the host may differ in the last fp32 bit, which can
    # flip a bf16 rounding for a handful of elements
    flips = int((h.cpu().view(torch.int16) != want_h.bfloat16().view(torch.int16)).sum())
    assert flips <= max(2, h.numel() // 10000)
    assert torch.equal(h, h2)
    if gate.numel():
        torch.testing.assert_close(dg.float().cpu(), want_dg, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(du.float().cpu(), want_du, rtol=2e-2, atol=2e-2)
        assert oracle.rel_frobenius(dg, want_dg) < 5e-3 and oracle.rel_frobenius(du, want_du) < 5e-3


def test_swiglu_linearity_in_up_at_full_size(native_library):
    """Size-independent property on the C3 activation size: h(g, 2u) == 2 h(g, u) exactly in bf16."""
    from molt_b200.kernels.gated_activation import swiglu_forward

    gen = torch.Generator(device="cuda").manual_seed(7)
    gate = torch.randn(8192, 8960, device="cuda", generator=gen).bfloat16()
    up = torch.randn(8192, 8960, device="cuda", generator=gen).bfloat16()
    assert torch.equal(swiglu_forward(gate, up * 2), swiglu_forward(gate, up) * 2)


def test_rmsnorm_matches_reference_fixture_bits(native_library):
    from molt_b200.methods.gated_replay import rmsnorm_bf16

    fx = load_golden("rmsnorm_6x96")
    hidden = torch.from_numpy(fx["hidden"]).bfloat16().cuda()
    out = rmsnorm_bf16(hidden, torch.from_numpy(fx["weight"]).cuda(), float(fx["eps"]))
    got = out.cpu().view(torch.int16).numpy()
    mismatches = int((got != fx["out_bits"]).sum())
    # rsqrt / reduction order may differ in the last bit of a few elements
    assert mismatches <= got.size // 50
    assert oracle.rel_frobenius(out, torch.from_numpy(fx["out_bits"]).view(torch.bfloat16)) < 4e-3
