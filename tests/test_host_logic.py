"""Host-side behaviour that needs no GPU: error conventions of the reference API, the quantiser,
module patchers, and the data-parallel bookkeeping."""
from __future__ import annotations

import pytest
import torch

from oracle import molt_oracle as oracle
from molt_b200.core.errors import CapabilityError, MoltStreamError
from molt_b200.data_parallel import GradArena, shard_rows
from molt_b200.kernels.gated_activation import enable_fused_silu_mlp, fused_silu_multiply
from molt_b200.methods import (
    QuantState, enable_asymmetric_gated_replay, enable_scheduled_nf4_lora, packed_nf4_backward_input,
    quantize_nf4, resolved_nf4_scales, scheduled_nf4_lora,
)
from molt_b200.methods.nf4_layer_cache import dense_nf4_layer_cache
from molt_b200.modules import GatedMLP, NF4LoRALinear
from molt_b200.streaming import NF4Tensor, StreamedLoRALinear


def test_error_hierarchy_matches_reference():
    assert issubclass(CapabilityError, MoltStreamError) and issubclass(MoltStreamError, RuntimeError)


def test_nf4tensor_quantize_matches_oracle_and_reference_storage_rule():
    torch.manual_seed(1)
    value = torch.randn(64, 64)
    q = NF4Tensor.quantize(value, block_size=64)
    ref = oracle.nf4_quantize(value, 64)
    assert torch.equal(q.packed, ref.packed) and torch.equal(q.scales, ref.scales)
    assert q.storage_bytes == value.numel() // 2 + value.numel() // 64 * 4  # reference tests/test_molt_stream_nf4.py:14
    with pytest.raises(ValueError):
        NF4Tensor.quantize(torch.randn(4, 4), block_size=8)
    with pytest.raises(ValueError):
        NF4Tensor.quantize(torch.empty(0), block_size=64)


def test_quantize_nf4_high_first_and_nested_match_oracle():
    torch.manual_seed(2)
    w = torch.randn(32, 128) * 0.02
    packed, state = quantize_nf4(w, 64, compress_statistics=True)
    ref = oracle.nf4_quantize(w, 64, oracle.HIGH_FIRST)
    assert packed.shape == (32 * 128 // 2, 1)
    assert torch.equal(packed.reshape(-1), ref.packed)
    nested = oracle.nest_absmax(ref.scales)
    assert state.nested and torch.equal(state.absmax, nested.codes)
    assert torch.equal(state.state2.absmax, nested.absmax2)
    assert float(state.offset) == pytest.approx(nested.offset)
    assert torch.equal(resolved_nf4_scales(QuantState(absmax=ref.scales, shape=(32, 128))), ref.scales)


def test_scheduled_nf4_lora_refuses_cpu():
    # reference tests/kernels/test_nf4_lora.py:82-93
    x = torch.randn(2, 4, requires_grad=True)
    packed = torch.zeros(8, 1, dtype=torch.uint8)
    a = torch.randn(2, 4, requires_grad=True)
    b = torch.randn(4, 2, requires_grad=True)
    with pytest.raises(CapabilityError, match="requires CUDA"):
        scheduled_nf4_lora(x, packed, a, b, QuantState(absmax=torch.ones(1), shape=(4, 4)), 1.0)


def test_packed_backward_refuses_cpu_and_bad_width():
    state = QuantState(absmax=torch.ones(1), shape=(4, 4))
    with pytest.raises(CapabilityError):
        packed_nf4_backward_input(torch.randn(2, 4).bfloat16(), torch.zeros(8, 1, dtype=torch.uint8), state)


def test_resolved_scales_rejects_other_formats():
    with pytest.raises(CapabilityError, match="NF4"):
        resolved_nf4_scales(QuantState(absmax=torch.ones(1), shape=(4, 4), quant_type="fp4"))
    with pytest.raises(CapabilityError, match="block size 64"):
        resolved_nf4_scales(QuantState(absmax=torch.ones(1), shape=(4, 4), blocksize=32))


def test_fused_silu_multiply_rejects_mismatched_inputs():
    # reference tests/kernels/test_gated_activation.py:45-47
    with pytest.raises(ValueError, match="identical"):
        fused_silu_multiply(torch.randn(2, 3), torch.randn(2, 4))


def test_fused_silu_multiply_has_no_cpu_fallback():
    with pytest.raises(CapabilityError, match="CUDA"):
        fused_silu_multiply(torch.randn(2, 3), torch.randn(2, 3))


def test_streamed_linear_validates_source_and_initialises_like_reference():
    source = NF4Tensor.quantize(torch.randn(16, 16), block_size=16)
    linear = StreamedLoRALinear(source, rank=4, alpha=8, device=torch.device("cpu"))
    assert linear.scaling == 2.0 and linear.lora_a.shape == (4, 16) and linear.lora_b.shape == (16, 4)
    assert torch.count_nonzero(linear.lora_b) == 0
    with pytest.raises(ValueError, match="matrix"):
        StreamedLoRALinear(NF4Tensor.quantize(torch.randn(4, 4, 4), block_size=16), 2, 4, torch.device("cpu"))
    with pytest.raises(CapabilityError, match="CUDA"):
        linear(torch.randn(2, 16).bfloat16())


def _tiny_mlp():
    torch.manual_seed(3)
    mk = lambda n, k: NF4LoRALinear.from_dense(torch.randn(n, k) * 0.02, rank=4, alpha=8)
    return GatedMLP(mk(96, 64), mk(96, 64), mk(64, 96))


class _Block(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.mlp = _tiny_mlp()
        self.q_proj = NF4LoRALinear.from_dense(torch.randn(64, 64) * 0.02, rank=4, alpha=8)
        self.k_proj = NF4LoRALinear.from_dense(torch.randn(16, 64) * 0.02, rank=4, alpha=8)


def test_enable_scheduled_patches_and_filters():
    block = _Block()
    assert enable_scheduled_nf4_lora(block, module_suffixes=("down_proj",)) == 1
    assert hasattr(block.mlp.down_proj, "_molt_original_forward")
    assert enable_scheduled_nf4_lora(block, require_narrow_output=True) == 1   # k_proj: 16 < 64 (down already patched)
    assert enable_scheduled_nf4_lora(block) == 3                               # the rest
    with pytest.raises(CapabilityError, match="down_proj"):                    # reference test_nf4_lora.py:96-103
        enable_scheduled_nf4_lora(torch.nn.Sequential(torch.nn.Linear(4, 4)), module_suffixes=("down_proj",))


def test_patched_forward_falls_back_outside_bf16_autocast():
    block = _Block()
    enable_scheduled_nf4_lora(block, module_suffixes=("q_proj",))
    calls = []
    block.q_proj._molt_original_forward = lambda x, *a, **k: calls.append(1) or x
    block.q_proj(torch.randn(2, 64))
    assert calls == [1]


def test_enable_asymmetric_gated_replay_argument_rules():
    block = _Block()
    with pytest.raises(ValueError, match="mutually exclusive"):
        enable_asymmetric_gated_replay(block, rematerialize_up=True, offload_blocks=1)
    with pytest.raises(ValueError, match="negative"):
        enable_asymmetric_gated_replay(block, rematerialize_blocks=-1)
    with pytest.raises(CapabilityError, match="only 1 compatible"):
        enable_asymmetric_gated_replay(block, rematerialize_blocks=2)
    assert enable_asymmetric_gated_replay(block) == 1
    assert block.mlp._molt_rematerialize_up is True
    with pytest.raises(CapabilityError, match="No compatible"):
        enable_asymmetric_gated_replay(torch.nn.Linear(2, 2))


def test_enable_fused_silu_mlp_checks_activation():
    block = _Block()
    with pytest.raises(CapabilityError, match="silu"):
        enable_fused_silu_mlp(block)
    block.config = type("Cfg", (), {"hidden_act": "silu", "model_type": "qwen2"})()
    assert enable_fused_silu_mlp(block) == 1


def test_layer_cache_rejects_layers_without_nf4_projections_and_restores_on_error():
    with pytest.raises(CapabilityError, match="no PEFT NF4"):
        with dense_nf4_layer_cache(torch.nn.Linear(2, 2)):
            pass
    block = _Block()
    original = block.q_proj.base_layer.forward
    with pytest.raises(CapabilityError):  # CPU tensors: the dequantiser refuses, forwards must be restored
        with dense_nf4_layer_cache(block):
            pass
    assert block.q_proj.base_layer.forward == original


def test_shard_rows_partitions_exactly():
    for total, world in ((8192, 8), (10, 3), (5, 8)):
        spans = [shard_rows(total, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))


def test_grad_arena_layout_and_buckets():
    params = [torch.nn.Parameter(torch.zeros(16, 96)), torch.nn.Parameter(torch.zeros(256, 16)),
              torch.nn.Parameter(torch.zeros(7, 65)), torch.nn.Parameter(torch.zeros(3), requires_grad=False)]
    arena = GradArena(params, bucket_bytes=16 * 96 * 4 + 16)
    assert len(arena.params) == 3
    assert all(off % 64 == 0 for off in arena.offsets)
    for p, view in zip(arena.params, arena.views):
        assert p.grad.data_ptr() == view.data_ptr() and view.shape == p.shape
    # buckets tile the arena, last parameter first
    assert arena.buckets[0][1] == arena.flat.numel() and arena.buckets[-1][0] == 0
    covered = sorted(arena.buckets)
    assert all(covered[i][1] == covered[i + 1][0] for i in range(len(covered) - 1))
    arena.views[1].fill_(2.0)
    assert arena.flat.sum() == 2.0 * 256 * 16
    arena.zero()
    assert arena.flat.abs().sum() == 0


def test_describe_checks_every_buffer_against_the_declared_shape():
    """The native side sees raw pointers only, so the descriptor builder refuses tensors that do not cover the
    declared weight: wrong dtype, sliced (non-contiguous) or short buffers, a second-level table of the wrong size."""
    from molt_b200.methods.quant_state import NestedState, describe

    n, k = 8, 128
    packed = torch.zeros(n * k // 2, 1, dtype=torch.uint8)
    good = QuantState(absmax=torch.ones(n * k // 64), shape=(n, k))
    desc = describe(packed, good)
    assert (desc.n, desc.k, desc.blocksize) == (n, k, 64)
    with pytest.raises(ValueError, match="declared weight shape"):
        describe(packed[:-1], good)                                   # packed too short
    with pytest.raises(CapabilityError):
        describe(packed.float(), good)                                # packed not uint8
    with pytest.raises(ValueError, match="declared weight shape"):
        describe(packed, QuantState(absmax=torch.ones(n * k // 64 - 1), shape=(n, k)))
    with pytest.raises(ValueError, match="contiguous"):
        describe(packed, QuantState(absmax=torch.ones(2 * n * k // 64)[::2], shape=(n, k)))
    with pytest.raises(ValueError, match="non-empty matrix"):
        describe(packed, QuantState(absmax=torch.ones(16), shape=(n, k, 1)))
    codes = torch.zeros(n * k // 64, dtype=torch.uint8)
    table = torch.linspace(-1, 1, 256)
    nested = QuantState(absmax=codes, shape=(n, k), nested=True, state2=NestedState(torch.ones(1), table, 256), offset=0.5)
    assert describe(packed, nested).absmax_kind == 1
    nested.state2 = NestedState(torch.ones(1), table[:255], 256)
    with pytest.raises(ValueError):
        describe(packed, nested)                                      # second-level table too short
    nested.state2 = NestedState(torch.ones(0), table, 256)
    with pytest.raises(ValueError, match="declared weight shape"):
        describe(packed, nested)                                      # second-level absmax too short
    nested.state2 = None
    with pytest.raises(ValueError, match="state2"):
        describe(packed, nested)
    # absmax-only descriptor (what resolved_nf4_scales builds): no packed tensor to check
    assert describe(None, good).n == n


def test_grad_arena_survives_zero_grad_set_to_none():
    """optimizer.zero_grad() drops .grad by default; the arena rebinds its slices so the optimiser still sees the
    gradients the kernels accumulate there."""
    a = torch.nn.Parameter(torch.zeros(4, 8))
    b = torch.nn.Parameter(torch.zeros(8, 4))
    arena = GradArena([a, b])
    opt = torch.optim.SGD([a, b], lr=1.0)
    opt.zero_grad()                       # set_to_none=True
    assert a.grad is None
    arena.zero()
    assert a.grad is arena.views[0] and b.grad is arena.views[1]
    arena.flat.fill_(1.0)
    opt.step()
    assert torch.all(a == -1.0) and torch.all(b == -1.0)
    opt.zero_grad()
    arena.all_reduce()                    # single process: no collective, but the slices are bound again
    assert a.grad is arena.views[0]
