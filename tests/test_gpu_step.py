"""The QLoRA step harness on a tiny decoder: every projection goes through the NF4-LoRA kernels."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tiny_decoder_trains(native_library):
    from molt_b200 import _native
    from molt_b200.qlora_step import DecoderShape, QLoRAStep, hot_path_flops_per_token

    shape = DecoderShape(layers=2, hidden=128, heads=4, kv_heads=2, head_dim=32, intermediate=256, vocab=512,
                         rope_theta=1e4, rank=8, alpha=16.0, nested_absmax=True, seq_len=64, micro_batch=4)
    step = QLoRAStep(shape, torch.device("cuda"), lr=5e-3)
    gen = torch.Generator(device="cuda").manual_seed(0)
    tokens = torch.randint(0, shape.vocab, (shape.micro_batch, shape.seq_len), device="cuda", generator=gen)
    targets = torch.roll(tokens, -1, dims=1)
    losses = []
    with torch.autocast("cuda", dtype=torch.bfloat16):
        for _ in range(8):
            losses.append(float(step.run(tokens, targets)))
    assert all(torch.isfinite(torch.tensor(losses)))
    assert losses[-1] < losses[0]                      # the adapters learn the repeated batch
    assert float(step.arena.flat.abs().sum()) > 0      # gradients reached the arena
    assert _native.read_status() == 0
    assert step.lora_parameter_count() == 2 * 8 * ((128 + 128) + 2 * (64 + 128) + (128 + 128) + 2 * (256 + 128) + (128 + 256))
    assert hot_path_flops_per_token(shape) > 0
