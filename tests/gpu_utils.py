"""Helpers for the GPU parity tests: seeded cases shared by the CUDA path and the CPU oracle."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from oracle import molt_oracle as oracle
from molt_b200 import _native
from molt_b200.methods.quant_state import NestedState, QuantState

TOL = 1e-2  # relative Frobenius bound for Y, dX, dA, dB (bf16 device path vs fp32 CPU oracle)


@dataclass
class LinearCase:
    q: oracle.OracleNF4
    scales_f32: torch.Tensor        # fp32 absmax actually in effect (resolved when nested)
    packed: torch.Tensor            # cuda uint8 [n*k/2, 1]
    state: QuantState               # cuda quant state
    a: torch.Tensor                 # cpu fp32
    b: torch.Tensor
    x: torch.Tensor                 # cpu fp32 holding bf16-rounded values
    dy: torch.Tensor
    scaling: float

    @property
    def weight(self) -> torch.Tensor:
        return oracle.nf4_dequantize(self.q, torch.float32, self.scales_f32)


def make_case(n, k, m, rank, *, seed=1337, scaling=2.0, nested=False, order="low-first", blocksize=64,
              w_std=0.02, ab_std=0.01) -> LinearCase:
    w, a, b, x, dy = oracle.seeded_linear_case(n, k, m, rank, seed=seed, w_std=w_std, ab_std=ab_std)
    q = oracle.nf4_quantize(w, blocksize, oracle.LOW_FIRST if order == "low-first" else oracle.HIGH_FIRST)
    dev = torch.device("cuda")
    if nested:
        nest = oracle.nest_absmax(q.scales)
        scales = oracle.resolve_nested_absmax(nest)
        state = QuantState(absmax=nest.codes.to(dev), shape=(n, k), blocksize=blocksize, nested=True,
                           state2=NestedState(nest.absmax2.to(dev), nest.code2.to(dev), nest.block2),
                           offset=nest.offset, nibble_order=order)
    else:
        scales = q.scales
        state = QuantState(absmax=q.scales.to(dev), shape=(n, k), blocksize=blocksize, nibble_order=order)
    return LinearCase(q, scales, q.packed.to(dev).reshape(-1, 1), state, a, b, x, dy, scaling)


def run_forward(case: LinearCase, path=_native.PATH_AUTO, keep_t=False):
    from molt_b200.methods._linear import linear_forward, weight_desc

    desc = weight_desc(case.packed, case.state)
    xb = case.x.cuda().bfloat16()
    return linear_forward(desc, xb, case.a.cuda(), case.b.cuda(), case.scaling, keep_t, path)


def run_backward(case: LinearCase, path=_native.PATH_AUTO, t=None):
    from molt_b200.methods._linear import linear_backward, weight_desc

    desc = weight_desc(case.packed, case.state)
    return linear_backward(desc, case.x.cuda().bfloat16(), case.dy.cuda().bfloat16(), case.a.cuda(), case.b.cuda(),
                           case.scaling, t, True, True, path=path)


def oracle_results(case: LinearCase):
    return oracle.nf4_lora_fwd_bwd(case.q, case.x, case.dy, case.a, case.b, case.scaling, case.scales_f32)


def assert_clean_status():
    status = _native.read_status()
    assert status == 0, f"device status word reports a bounded wait that expired: 0x{status:08x}"


def dense_from_state(packed: torch.Tensor, state) -> torch.Tensor:
    """deq(W) in fp32 on the host, computed by the oracle from the bytes and absmax a device-side quant state holds."""
    order = oracle.HIGH_FIRST if state.nibble_order == "high-first" else oracle.LOW_FIRST
    if state.nested:
        nested = oracle.NestedAbsmax(state.absmax.cpu(), state.state2.absmax.cpu(), state.state2.code.cpu(),
                                     float(state.offset), int(state.state2.blocksize))
        scales = oracle.resolve_nested_absmax(nested)
    else:
        scales = state.absmax.cpu()
    n, k = (int(v) for v in state.shape)
    q = oracle.OracleNF4(packed.reshape(-1).cpu(), scales, (n, k), int(state.blocksize), n * k, order)
    return oracle.nf4_dequantize(q)
