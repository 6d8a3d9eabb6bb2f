"""The CPU oracle against fixtures produced by the reference implementation itself (tests/golden)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import molt_oracle as oracle
from tests.conftest import load_golden

QUANT_CASES = ["q_8x8_b16", "q_64x64_b64", "q_70x65_b64", "q_96x64_b64", "q_48x1536_b64", "q_33x50_b32"]
LINEAR_CASES = ["lin_8x8_r2", "lin_96x64_r8", "lin_70x65_r7", "lin_256x128_r16"]


def test_codebook_is_the_reference_table():
    fixture = load_golden("nf4_codebook")
    assert np.array_equal(fixture["codebook"], oracle.NF4_CODEBOOK.numpy())


@pytest.mark.parametrize("name", QUANT_CASES)
def test_quantize_matches_reference_bytes(name):
    fx = load_golden(name)
    q = oracle.nf4_quantize(torch.from_numpy(fx["value"]), int(fx["block"]))
    assert np.array_equal(q.packed.numpy(), fx["packed"])
    assert np.array_equal(q.scales.numpy(), fx["scales"])
    assert q.elements == int(fx["elements"])
    assert q.packed.numel() + q.scales.numel() * 4 == int(fx["storage_bytes"])


@pytest.mark.parametrize("name", QUANT_CASES)
def test_dequantize_is_bit_exact(name):
    fx = load_golden(name)
    q = oracle.OracleNF4(torch.from_numpy(fx["packed"]), torch.from_numpy(fx["scales"]),
                         tuple(int(v) for v in fx["shape"]), int(fx["block"]), int(fx["elements"]))
    assert np.array_equal(oracle.nf4_dequantize(q, torch.float32).numpy(), fx["deq_f32"])
    got = oracle.nf4_dequantize(q, torch.bfloat16).view(torch.int16).numpy()
    assert np.array_equal(got, fx["deq_bf16_bits"])


def test_storage_and_error_bound_of_reference_test():
    # reference tests/test_molt_stream_nf4.py:9-15
    torch.manual_seed(1)
    value = torch.randn(64, 64)
    q = oracle.nf4_quantize(value, 64)
    assert q.packed.numel() + q.scales.numel() * 4 == value.numel() // 2 + value.numel() // 64 * 4
    assert torch.mean((oracle.nf4_dequantize(q) - value) ** 2).sqrt() < 0.15


def test_high_first_order_is_the_byte_swap_of_low_first():
    torch.manual_seed(5)
    value = torch.randn(16, 64)
    low = oracle.nf4_quantize(value, 64, oracle.LOW_FIRST)
    high = oracle.nf4_quantize(value, 64, oracle.HIGH_FIRST)
    swapped = ((low.packed & 0x0F) << 4) | (low.packed >> 4)
    assert torch.equal(high.packed, swapped)
    assert torch.equal(oracle.nf4_dequantize(low), oracle.nf4_dequantize(high))


@pytest.mark.parametrize("name", LINEAR_CASES)
def test_linear_forward_backward_matches_reference(name):
    fx = load_golden(name)
    torch.set_num_threads(1)
    n, k = fx["w"].shape
    q = oracle.OracleNF4(torch.from_numpy(fx["packed"]), torch.from_numpy(fx["scales"]), (n, k), int(fx["block"]), n * k)
    x, dy = torch.from_numpy(fx["x"]), torch.from_numpy(fx["dy"])
    a, b = torch.from_numpy(fx["a"]), torch.from_numpy(fx["b"])
    y, dx, da, db = oracle.nf4_lora_fwd_bwd(q, x, dy, a, b, float(fx["scaling"]))
    for got, key in ((y, "y"), (dx, "dx"), (da, "da"), (db, "db")):
        assert oracle.rel_frobenius(got, torch.from_numpy(fx[key])) < 1e-6, key
    # against plain autograd of the same formula
    xin = x.clone().requires_grad_(True)
    ain, bin_ = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
    w = oracle.nf4_dequantize(q)
    out = oracle.nf4_lora_forward(xin, w, ain, bin_, float(fx["scaling"]))
    out.backward(dy)
    assert oracle.rel_frobenius(dx, xin.grad) < 1e-5
    assert oracle.rel_frobenius(da, ain.grad) < 1e-5
    assert oracle.rel_frobenius(db, bin_.grad) < 1e-5


@pytest.mark.parametrize("name", ["swiglu_3x5x17_f32", "swiglu_2x31x128_bf16"])
def test_swiglu_matches_reference(name):
    fx = load_golden(name)
    gate, up, grad = (torch.from_numpy(fx[k]) for k in ("gate", "up", "grad"))
    tol = 2e-2 if "bf16" in name else 1e-5  # reference tests/kernels/test_gated_activation.py:22
    torch.testing.assert_close(oracle.swiglu_forward(gate, up), torch.from_numpy(fx["out"]), rtol=tol, atol=tol)
    dgate, dup = oracle.swiglu_backward(grad, gate, up)
    torch.testing.assert_close(dgate, torch.from_numpy(fx["dgate"]), rtol=tol, atol=tol)
    torch.testing.assert_close(dup, torch.from_numpy(fx["dup"]), rtol=tol, atol=tol)


def test_rmsnorm_matches_reference_bits():
    fx = load_golden("rmsnorm_6x96")
    hidden, weight, grad = (torch.from_numpy(fx[k]) for k in ("hidden", "weight", "grad"))
    out = oracle.rmsnorm_forward(hidden, weight, float(fx["eps"])).bfloat16()
    assert np.array_equal(out.view(torch.int16).numpy(), fx["out_bits"])
    dh = oracle.rmsnorm_backward(grad, hidden, weight, float(fx["eps"])).bfloat16()
    assert np.array_equal(dh.view(torch.int16).numpy(), fx["dhidden_bits"])


def test_nested_absmax_round_trip_is_close_and_deterministic():
    torch.manual_seed(11)
    absmax = torch.rand(1000) * 0.05 + 0.04
    nested = oracle.nest_absmax(absmax)
    resolved = oracle.resolve_nested_absmax(nested)
    assert resolved.shape == absmax.shape
    assert (resolved - absmax).abs().max() < 0.05 / 127  # half a step of the 256-level table, scaled
    assert torch.equal(resolved, oracle.resolve_nested_absmax(oracle.nest_absmax(absmax)))


def test_gated_mlp_oracle_matches_autograd():
    torch.manual_seed(1221)
    hidden, inter, m, r = 64, 96, 12, 8

    def proj(n, k):
        q = oracle.nf4_quantize(torch.randn(n, k) * 0.02, 64)
        return oracle.OracleProjection(oracle.nf4_dequantize(q), (torch.randn(r, k) * 0.1).requires_grad_(),
                                       (torch.randn(n, r) * 0.1).requires_grad_(), 2.0)

    gp, up, dp = proj(inter, hidden), proj(inter, hidden), proj(hidden, inter)
    x = torch.randn(m, hidden).requires_grad_()
    dy = torch.randn(m, hidden)
    with torch.no_grad():
        res = oracle.gated_mlp_fwd_bwd(x, dy, gp, up, dp)
    g = oracle.nf4_lora_forward(x, gp.weight, gp.lora_a, gp.lora_b, 2.0)
    u = oracle.nf4_lora_forward(x, up.weight, up.lora_a, up.lora_b, 2.0)
    y = oracle.nf4_lora_forward(torch.nn.functional.silu(g) * u, dp.weight, dp.lora_a, dp.lora_b, 2.0)
    y.backward(dy)
    assert oracle.rel_frobenius(res["y"], y) < 1e-5
    assert oracle.rel_frobenius(res["dx"], x.grad) < 1e-4
    for key, p in (("gate_a", gp.lora_a), ("gate_b", gp.lora_b), ("up_a", up.lora_a), ("up_b", up.lora_b),
                   ("down_a", dp.lora_a), ("down_b", dp.lora_b)):
        assert oracle.rel_frobenius(res[key], p.grad) < 1e-4, key
