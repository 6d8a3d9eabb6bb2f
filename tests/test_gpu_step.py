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


@pytest.mark.parametrize("rows,vocab", [(5, 512), (3, 151936), (2, 1000)])
def test_ce_softmax_grad_kernel(native_library, rows, vocab):
    """Loss and in-place gradient of the frozen-head cross-entropy against torch in fp32."""
    from molt_b200 import _native

    gen = torch.Generator().manual_seed(rows + vocab)
    logits = (torch.randn(rows, vocab, generator=gen) * 3).bfloat16()
    targets = torch.randint(0, vocab, (rows,), generator=gen)
    dev_logits = logits.cuda()
    loss = torch.empty(rows, device="cuda")
    _native.check(_native.library().molt_ce_softmax_grad(dev_logits.data_ptr(), targets.cuda().data_ptr(), loss.data_ptr(),
                                                         rows, vocab, 0.25, _native.stream_handle()))
    ref_logits = logits.float().requires_grad_()
    ref_loss = torch.nn.functional.cross_entropy(ref_logits, targets, reduction="none")
    (ref_loss.sum() * 0.25).backward()
    torch.testing.assert_close(loss.cpu(), ref_loss.detach(), rtol=1e-4, atol=1e-4)
    got = dev_logits.float().cpu()
    assert (got - ref_logits.grad).abs().max() <= 2e-3 * 0.25 + 1e-6   # bf16 rounding of values in [-0.25, 0.25]


def test_ce_softmax_grad_ignores_out_of_range_labels(native_library):
    """Labels outside [0, vocab) -- the usual ignore index -100, or an id past the vocabulary -- give zero loss and a
    plain softmax gradient with no one-hot term (reference kernels/frozen_linear_cross_entropy.py:42-43, 63, 94-95,
    133); the row before the first must not be touched."""
    from molt_b200 import _native

    rows, vocab = 6, 1000
    gen = torch.Generator().manual_seed(9)
    logits = (torch.randn(rows + 1, vocab, generator=gen) * 3).bfloat16()
    targets = torch.tensor([-100, 3, vocab, 999, -1, vocab + 7])
    buffer = logits.cuda()
    dev_logits = buffer[1:]                      # row 0 of the buffer sits in front of the kernel's first row
    loss = torch.full((rows,), 7.0, device="cuda")
    _native.check(_native.library().molt_ce_softmax_grad(dev_logits.data_ptr(), targets.cuda().data_ptr(), loss.data_ptr(),
                                                         rows, vocab, 0.5, _native.stream_handle()))
    torch.cuda.synchronize()
    assert torch.equal(buffer[0].cpu(), logits[0])
    ref = logits[1:].float()
    valid = (targets >= 0) & (targets < vocab)
    probs = torch.softmax(ref, dim=-1) * 0.5
    onehot = torch.zeros_like(probs)
    onehot[valid, targets[valid]] = 0.5
    want_grad = probs - onehot
    want_loss = torch.where(valid, torch.logsumexp(ref, -1) - ref[torch.arange(rows), targets.clamp(0, vocab - 1)],
                            torch.zeros(rows))
    torch.testing.assert_close(loss.cpu(), want_loss, rtol=1e-4, atol=1e-4)
    assert (dev_logits.float().cpu() - want_grad).abs().max() <= 2e-3 * 0.5 + 1e-6
