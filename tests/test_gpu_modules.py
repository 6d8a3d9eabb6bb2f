"""The reference-facing Python API on the GPU: autograd functions, modules, patchers, replay schedules."""
from __future__ import annotations

import pytest
import torch
from torch.nn import functional as F

from oracle import molt_oracle as oracle
from tests.gpu_utils import TOL, assert_clean_status, make_case, oracle_results

pytestmark = pytest.mark.gpu


def test_scheduled_nf4_lora_autograd(native_library):
    from molt_b200.methods import scheduled_nf4_lora

    case = make_case(1536, 256, 256, 8, seed=941, order="high-first", nested=True, scaling=0.3)
    x = case.x.cuda().bfloat16().reshape(1, 256, 256).requires_grad_()
    a = case.a.cuda().requires_grad_()
    b = case.b.cuda().requires_grad_()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = scheduled_nf4_lora(x, case.packed, a, b, case.state, case.scaling)
    assert y.shape == (1, 256, 1536) and y.dtype == torch.bfloat16
    y.backward(case.dy.cuda().bfloat16().reshape(1, 256, 1536))
    y_ref, dx_ref, da_ref, db_ref = oracle_results(case)
    assert a.grad.dtype == torch.float32 and b.grad.dtype == torch.float32
    assert x.grad.shape == x.shape
    for got, want in ((y, y_ref), (x.grad, dx_ref), (a.grad, da_ref), (b.grad, db_ref)):
        assert oracle.rel_frobenius(got.reshape(want.shape), want) <= TOL
    assert_clean_status()


def test_scheduled_nf4_lora_guards(native_library):
    from molt_b200.core.errors import CapabilityError
    from molt_b200.methods import scheduled_nf4_lora

    case = make_case(128, 64, 8, 8)
    x = case.x.cuda().bfloat16()
    a, b = case.a.cuda(), case.b.cuda()
    with pytest.raises(CapabilityError, match="FP32 adapter"):
        scheduled_nf4_lora(x, case.packed, a.bfloat16(), b, case.state, 1.0)
    with pytest.raises(CapabilityError, match="bfloat16"):
        scheduled_nf4_lora(x.float(), case.packed, a, b, case.state, 1.0)
    with pytest.raises(CapabilityError, match="cached NF4 backward weight"):
        scheduled_nf4_lora(x, case.packed, a, b, case.state, 1.0, torch.zeros(3, 3, device="cuda"))
    dense = torch.zeros(128, 64, device="cuda", dtype=torch.bfloat16)
    y0 = scheduled_nf4_lora(x, case.packed, a, b, case.state, 1.0)
    y1 = scheduled_nf4_lora(x, case.packed, a, b, case.state, 1.0, dense)
    assert torch.equal(y0, y1)  # reference tests/kernels/test_nf4_lora.py:48-79: cached and per-call paths agree bitwise


def test_streamed_lora_linear_matches_reference_eager_path(native_library):
    from molt_b200.streaming import NF4Tensor, StreamedLoRALinear

    w, a, b, x, dy = oracle.seeded_linear_case(192, 128, 24, 4, seed=17)
    source = NF4Tensor.quantize(w, block_size=64)
    linear = StreamedLoRALinear(source, rank=4, alpha=8, device=torch.device("cuda"))
    with torch.no_grad():
        linear.lora_a.copy_(a)
        linear.lora_b.copy_(b)
    xin = x.cuda().bfloat16().requires_grad_()
    y = linear(xin, source.stage("cuda"))
    y.backward(dy.cuda().bfloat16())
    q = oracle.nf4_quantize(w, 64)
    y_ref, dx_ref, da_ref, db_ref = oracle.nf4_lora_fwd_bwd(q, x, dy, a, b, 2.0)
    for got, want in ((y, y_ref), (xin.grad, dx_ref), (linear.lora_a.grad, da_ref), (linear.lora_b.grad, db_ref)):
        assert oracle.rel_frobenius(got, want) <= TOL
    assert source.packed.grad is None  # reference tests/test_molt_stream_nf4.py:28
    # dense staged weight is accepted for call-site compatibility
    y2 = linear(xin.detach(), source.dequantize(device="cuda", dtype=torch.bfloat16))
    assert torch.equal(y2, y.detach())


def _mlp(hidden, inter, rank=8, seed=1221, order="high-first"):
    from molt_b200.modules import GatedMLP, NF4LoRALinear

    gen = torch.Generator().manual_seed(seed)
    projs, dense = [], []
    for n, k in ((inter, hidden), (inter, hidden), (hidden, inter)):
        w = torch.randn(n, k, generator=gen) * 0.05
        lin = NF4LoRALinear.from_dense(w.cuda(), rank, 2.0 * rank, nibble_order=order)
        with torch.no_grad():
            lin.lora_A["default"].weight.copy_(torch.randn(rank, k, generator=gen) * 0.05)
            lin.lora_B["default"].weight.copy_(torch.randn(n, rank, generator=gen) * 0.05)
        projs.append(lin)
        q = oracle.nf4_quantize(w, 64, oracle.HIGH_FIRST)
        dense.append(oracle.OracleProjection(oracle.nf4_dequantize(q), lin.lora_A["default"].weight.detach().cpu(),
                                             lin.lora_B["default"].weight.detach().cpu(), 2.0))
    return GatedMLP(*projs), dense


def _adapter_grads(mlp):
    out = {}
    for name in ("gate", "up", "down"):
        proj = getattr(mlp, f"{name}_proj")
        out[f"{name}_a"] = proj.lora_A["default"].weight.grad
        out[f"{name}_b"] = proj.lora_B["default"].weight.grad
    return out


@pytest.mark.parametrize("hidden,inter", [(64, 128), (128, 256)])
@pytest.mark.parametrize("mode", ["keep", "replay", "offload_up", "offload_gate", "offload_both"])
def test_asymmetric_gated_replay_modes(native_library, hidden, inter, mode):
    # the five modes of reference tests/kernels/test_gated_replay.py:14-23, seed 1221
    from molt_b200.methods import enable_asymmetric_gated_replay

    mlp, dense = _mlp(hidden, inter)
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(1, 32, hidden, generator=gen).bfloat16()
    dy = torch.randn(1, 32, hidden, generator=gen).bfloat16()
    kwargs = {"keep": dict(rematerialize_up=False), "replay": dict(rematerialize_up=True),
              "offload_up": dict(rematerialize_up=False, offload_blocks=1),
              "offload_gate": dict(rematerialize_up=False, offload_gate_blocks=1),
              "offload_both": dict(rematerialize_up=False, offload_blocks=1, offload_gate_blocks=1)}[mode]
    assert enable_asymmetric_gated_replay(mlp, **kwargs) == 1
    xin = x.cuda().requires_grad_()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = mlp(xin)
    y.backward(dy.cuda())
    torch.cuda.synchronize()
    ref = oracle.gated_mlp_fwd_bwd(x.float().reshape(32, hidden), dy.float().reshape(32, hidden), *dense)
    assert oracle.rel_frobenius(y.reshape(32, hidden), ref["y"]) <= TOL
    assert oracle.rel_frobenius(xin.grad.reshape(32, hidden), ref["dx"]) <= TOL
    for key, grad in _adapter_grads(mlp).items():
        assert oracle.rel_frobenius(grad, ref[key]) <= TOL, key
    assert_clean_status()


@pytest.mark.parametrize("replay", [True, False])
@pytest.mark.parametrize("norm_replay", [False, True])
def test_whole_block_node(native_library, replay, norm_replay):
    from molt_b200.methods.gated_replay import rmsnorm_bf16

    hidden, inter, m = 128, 320, 200
    mlp, dense = _mlp(hidden, inter, rank=16, seed=77)
    gen = torch.Generator().manual_seed(6)
    source = torch.randn(m, hidden, generator=gen).bfloat16()
    dy = torch.randn(m, hidden, generator=gen).bfloat16()
    norm_w = (torch.randn(hidden, generator=gen) * 0.1 + 1.0)
    if norm_replay:
        x_dev = rmsnorm_bf16(source.cuda(), norm_w.cuda(), 1e-6).requires_grad_()
        y = mlp.fused(x_dev, rematerialize_up=replay, source=source.cuda(), norm_weight=norm_w.cuda(), norm_eps=1e-6)
        x_ref = oracle.rmsnorm_forward(source, norm_w, 1e-6).bfloat16().float()
    else:
        x_dev = source.cuda().requires_grad_()
        y = mlp.fused(x_dev, rematerialize_up=replay)
        x_ref = source.float()
    y.backward(dy.cuda())
    torch.cuda.synchronize()
    ref = oracle.gated_mlp_fwd_bwd(x_ref, dy.float(), *dense)
    assert oracle.rel_frobenius(y, ref["y"]) <= TOL
    assert oracle.rel_frobenius(x_dev.grad, ref["dx"]) <= TOL
    for key, grad in _adapter_grads(mlp).items():
        assert oracle.rel_frobenius(grad, ref[key]) <= TOL, key
    assert_clean_status()


def test_replay_and_keep_give_identical_gradients(native_library):
    """Replaying `up` recomputes exactly what the forward computed, so both schedules agree bit for bit."""
    results = []
    for replay in (True, False):
        mlp, _ = _mlp(128, 256, rank=16, seed=3)
        gen = torch.Generator().manual_seed(8)
        x = torch.randn(96, 128, generator=gen).bfloat16().cuda().requires_grad_()
        y = mlp.fused(x, rematerialize_up=replay)
        y.backward(torch.randn(96, 128, generator=gen).bfloat16().cuda())
        results.append((y.detach(), x.grad, _adapter_grads(mlp)))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    for key in results[0][2]:
        assert torch.equal(results[0][2][key], results[1][2][key]), key


def test_fused_silu_mlp_patcher_and_plain_module_agree(native_library):
    from molt_b200.kernels.gated_activation import enable_fused_silu_mlp

    mlp, dense = _mlp(64, 128)
    holder = torch.nn.Module()
    holder.mlp = mlp
    holder.config = type("Cfg", (), {"hidden_act": "silu", "model_type": "qwen2"})()
    x = torch.randn(16, 64, generator=torch.Generator().manual_seed(2)).bfloat16().cuda()
    before = mlp(x)
    assert enable_fused_silu_mlp(holder) == 1
    after = mlp(x)
    assert oracle.rel_frobenius(after, before.float()) < 1e-2
    want = oracle.gated_mlp_fwd_bwd(x.float().cpu(), torch.zeros(16, 64), *dense)["y"]
    assert oracle.rel_frobenius(after, want) <= TOL


def test_dense_layer_cache_context(native_library):
    from molt_b200.methods.nf4_layer_cache import dense_nf4_layer_cache

    mlp, dense = _mlp(64, 128)
    original = mlp.gate_proj.base_layer.forward
    x = torch.randn(4, 64, generator=torch.Generator().manual_seed(2)).bfloat16().cuda()
    with dense_nf4_layer_cache(mlp) as count:
        assert count == 3
        got = mlp.gate_proj.base_layer(x)
    assert mlp.gate_proj.base_layer.forward == original
    want = x.float().cpu() @ dense[0].weight.t()
    assert oracle.rel_frobenius(got, want) <= TOL
    with pytest.raises(RuntimeError):  # restored after an exception too (reference tests/training/test_nf4_layer_cache.py:65-75)
        with dense_nf4_layer_cache(mlp):
            raise RuntimeError("boom")
    assert mlp.gate_proj.base_layer.forward == original


def test_grad_arena_receives_kernel_gradients_in_place(native_library):
    from molt_b200.data_parallel import GradArena, lora_parameters

    mlp, dense = _mlp(128, 256, rank=16, seed=9)
    arena = GradArena(lora_parameters(mlp))
    gen = torch.Generator().manual_seed(4)
    x = torch.randn(64, 128, generator=gen).bfloat16()
    dy = torch.randn(64, 128, generator=gen).bfloat16()
    for _ in range(2):  # two micro-batches accumulate
        xin = x.cuda().requires_grad_()
        mlp.fused(xin).backward(dy.cuda())
    ref = oracle.gated_mlp_fwd_bwd(x.float(), dy.float(), *dense)
    for key, grad in _adapter_grads(mlp).items():
        assert grad.data_ptr() >= arena.flat.data_ptr()
        assert oracle.rel_frobenius(grad, 2 * ref[key]) <= TOL, key
    arena.zero()
    assert float(arena.flat.abs().sum()) == 0.0


@pytest.mark.parametrize("m", [5, 40, 200, 700])
@pytest.mark.parametrize("keep_up", [False, True])
def test_block_with_kept_low_rank_inputs_equals_the_plain_block(native_library, m, keep_up):
    """molt_mlp_fwd_t / molt_mlp_bwd_t (low-rank inputs kept, h rebuilt by the backward's own SwiGLU pass) against
    molt_mlp_fwd / molt_mlp_bwd: same kernels on the same operands in another order, so every output agrees bit for bit,
    on whatever path the token count selects."""
    import ctypes

    from molt_b200 import _native
    from molt_b200.methods._linear import weight_desc_for_tokens
    from molt_b200.methods.gated_replay import _proj_struct

    hidden, inter, rank = 128, 320, 16
    mlp, _ = _mlp(hidden, inter, rank=rank, seed=41)
    lins = (mlp.gate_proj, mlp.up_proj, mlp.down_proj)
    descs = [weight_desc_for_tokens(l.base_layer.weight.data, l.base_layer.weight.quant_state, m) for l in lins]
    adapters = [(l.lora_A["default"].weight.detach().contiguous(), l.lora_B["default"].weight.detach().contiguous()) for l in lins]
    projs = [_proj_struct(descs[i], adapters[i][0], adapters[i][1], 2.0) for i in range(3)]
    lib = native_library
    gen = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(m, hidden, device="cuda", generator=gen).bfloat16()
    dy = torch.randn(m, hidden, device="cuda", generator=gen).bfloat16()
    stream = _native.stream_handle(x.device)
    results = []
    for kept in (False, True):
        gate = torch.empty(m, inter, device="cuda", dtype=torch.bfloat16)
        up = torch.empty(m, inter, device="cuda", dtype=torch.bfloat16) if keep_up else None
        y = torch.empty(m, hidden, device="cuda", dtype=torch.bfloat16)
        dx = torch.empty(m, hidden, device="cuda", dtype=torch.bfloat16)
        low = torch.zeros(3, m, 64, device="cuda", dtype=torch.bfloat16) if kept else None
        grads = [torch.zeros_like(t, dtype=torch.float32) for pair in adapters for t in pair]
        pointers = (ctypes.c_void_p * 6)(*[g.data_ptr() for g in grads])
        nbytes = max(lib.molt_mlp_workspace_bytes(op, projs[0], projs[1], projs[2], m, int(keep_up))
                     for op in (_native.OP_MLP_FWD, _native.OP_MLP_BWD))
        ws = torch.empty(nbytes, device="cuda", dtype=torch.uint8)
        if kept:
            _native.check(lib.molt_mlp_fwd_t(projs[0], projs[1], projs[2], x.data_ptr(), gate.data_ptr(), _native.ptr(up),
                                             y.data_ptr(), low.data_ptr(), m, ws.data_ptr(), nbytes, stream))
            _native.check(lib.molt_mlp_bwd_t(projs[0], projs[1], projs[2], x.data_ptr(), gate.data_ptr(), _native.ptr(up),
                                             low.data_ptr(), dy.data_ptr(), dx.data_ptr(), pointers, 0, m, ws.data_ptr(),
                                             nbytes, stream))
        else:
            _native.check(lib.molt_mlp_fwd(projs[0], projs[1], projs[2], x.data_ptr(), gate.data_ptr(), _native.ptr(up),
                                           y.data_ptr(), m, ws.data_ptr(), nbytes, stream))
            _native.check(lib.molt_mlp_bwd(projs[0], projs[1], projs[2], x.data_ptr(), gate.data_ptr(), _native.ptr(up),
                                           dy.data_ptr(), dx.data_ptr(), pointers, 0, m, ws.data_ptr(), nbytes, stream))
        torch.cuda.synchronize()
        results.append((y, dx, gate, *grads, low))
    for index, (plain, kept) in enumerate(zip(results[0][:-1], results[1][:-1])):
        assert torch.equal(plain, kept), index
    low = results[1][-1]
    assert torch.equal(low[0][:, :rank], (x.float() @ adapters[0][0].bfloat16().float().t()).bfloat16()) or \
        oracle.rel_frobenius(low[0][:, :rank], x.float().cpu() @ adapters[0][0].bfloat16().float().cpu().t()) <= TOL
    assert not low[:, :, rank:].any()
    assert_clean_status()
