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


def _reference_decoder_gradients(model, tokens, targets, global_tokens):
    """The decoder's loss and adapter gradients recomputed on the host in fp32 with plain autograd: every projection is
    the oracle's eager composition y = x W^T + s (x A^T) B^T on the oracle-dequantised weight (reference
    streaming/engine.py:27-31), RMSNorm / RoPE / causal attention / mean cross-entropy are the textbook formulas."""
    import math

    from oracle import molt_oracle as oracle
    from tests.gpu_utils import dense_from_state

    sh = model.shape
    leaves = {}

    def linear(mod, x, name):
        weight = dense_from_state(mod.base_layer.weight.data, mod.base_layer.weight.quant_state)
        a = mod.lora_A["default"].weight.detach().cpu().clone().requires_grad_()
        b = mod.lora_B["default"].weight.detach().cpu().clone().requires_grad_()
        leaves[name] = (a, b)
        return oracle.nf4_lora_forward(x, weight, a, b, mod.scaling["default"])

    def norm(x, mod):
        v = x.float()
        return v * torch.rsqrt(v.square().mean(-1, keepdim=True) + mod.eps) * mod.weight.detach().float().cpu()

    def rope(x, cos, sin):
        half = x.shape[-1] // 2
        return x * cos + torch.cat((-x[..., half:], x[..., :half]), dim=-1) * sin

    cos, sin = model.cos.float().cpu(), model.sin.float().cpu()
    x = model.embed.detach().float().cpu()[tokens.cpu()]
    b, s, _ = x.shape
    for li, layer in enumerate(model.layers):
        h = norm(x, layer.input_norm)
        at = layer.attn
        q = linear(at.q_proj, h, f"{li}.q").view(b, s, sh.heads, sh.head_dim).transpose(1, 2)
        k = linear(at.k_proj, h, f"{li}.k").view(b, s, sh.kv_heads, sh.head_dim).transpose(1, 2)
        v = linear(at.v_proj, h, f"{li}.v").view(b, s, sh.kv_heads, sh.head_dim).transpose(1, 2)
        q, k = rope(q, cos, sin), rope(k, cos, sin)
        rep = sh.heads // sh.kv_heads
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
        scores = q @ k.transpose(-1, -2) / math.sqrt(sh.head_dim)
        scores = scores.masked_fill(torch.ones(s, s, dtype=torch.bool).triu(1), float("-inf"))
        ctx = (torch.softmax(scores, -1) @ v).transpose(1, 2).reshape(b, s, sh.heads * sh.head_dim)
        x = x + linear(at.o_proj, ctx, f"{li}.o")
        h = norm(x, layer.post_norm)
        gate, up = linear(layer.mlp.gate_proj, h, f"{li}.gate"), linear(layer.mlp.up_proj, h, f"{li}.up")
        x = x + linear(layer.mlp.down_proj, torch.nn.functional.silu(gate) * up, f"{li}.down")
    hidden = norm(x, model.final_norm).reshape(-1, sh.hidden)
    logits = hidden @ model.head.detach().float().cpu().t()
    loss = torch.nn.functional.cross_entropy(logits, targets.reshape(-1).cpu(), reduction="sum") / global_tokens
    loss.backward()
    return float(loss.detach()), {name: (a.grad, b.grad) for name, (a, b) in leaves.items()}


def test_decoder_layer_gradients_match_the_oracle_composition(native_library):
    """One decoder layer + frozen head: every adapter gradient the step leaves in the arena against an fp32 host
    recomputation.  Tolerance 3e-2 relative Frobenius: the device path rounds every activation to bf16 (about a dozen
    roundings between an adapter and the loss) where the single linear is held to 1e-2."""
    from molt_b200 import _native
    from molt_b200.qlora_step import DecoderShape, QLoRAStep
    from oracle import molt_oracle as oracle

    shape = DecoderShape(layers=1, hidden=256, heads=4, kv_heads=2, head_dim=64, intermediate=512, vocab=1024,
                         rope_theta=1e4, rank=16, alpha=32.0, nested_absmax=True, seq_len=128, micro_batch=2)
    step = QLoRAStep(shape, torch.device("cuda"), lr=1e-3)
    gen = torch.Generator(device="cuda").manual_seed(3)
    tokens = torch.randint(0, shape.vocab, (shape.micro_batch, shape.seq_len), device="cuda", generator=gen)
    targets = torch.randint(0, shape.vocab, (shape.micro_batch, shape.seq_len), device="cuda", generator=gen)
    ref_loss, ref = _reference_decoder_gradients(step.model, tokens, targets, shape.tokens)   # before the step changes A, B
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = float(step._forward_backward(tokens, targets))
    torch.cuda.synchronize()
    assert _native.read_status() == 0
    assert abs(loss - ref_loss) <= 1e-2 * abs(ref_loss)
    layer = step.model.layers[0]
    modules = {"0.q": layer.attn.q_proj, "0.k": layer.attn.k_proj, "0.v": layer.attn.v_proj, "0.o": layer.attn.o_proj,
               "0.gate": layer.mlp.gate_proj, "0.up": layer.mlp.up_proj, "0.down": layer.mlp.down_proj}
    for name, mod in modules.items():
        da, db = ref[name]
        assert oracle.rel_frobenius(mod.lora_A["default"].weight.grad, da) <= 3e-2, name
        assert oracle.rel_frobenius(mod.lora_B["default"].weight.grad, db) <= 3e-2, name


def test_rmsnorm_backward_matches_reference_fixture(native_library):
    """dhidden of the frozen RMSNorm against the reference's own backward (fixture made from
    reference kernels/frozen_rmsnorm.py:25-37), and against the oracle on a wide, unaligned and a bf16-weight case."""
    from molt_b200 import _native
    from oracle import molt_oracle as oracle
    from tests.conftest import load_golden

    lib = _native.library()

    def run(x, w, dy, eps, offset):
        out = torch.empty_like(x)
        dtype = _native.DTYPE_F32 if w.dtype == torch.float32 else _native.DTYPE_BF16
        _native.check(lib.molt_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), dtype, eps, offset, out.data_ptr(),
                                           x.shape[0], x.shape[1], _native.stream_handle()))
        return out

    fx = load_golden("rmsnorm_6x96")
    x = torch.from_numpy(fx["hidden"]).bfloat16().cuda()
    dy = torch.from_numpy(fx["grad"]).bfloat16().cuda()
    got = run(x, torch.from_numpy(fx["weight"]).cuda(), dy, float(fx["eps"]), 0.0)
    want = torch.from_numpy(fx["dhidden_bits"]).view(torch.bfloat16)
    assert oracle.rel_frobenius(got, want.float()) <= 4e-3      # both are bf16 roundings of the same fp32 value
    # rsqrt / reduction order may differ in the last bit of a few elements
    assert int((got.cpu().view(torch.int16) != want.view(torch.int16)).sum()) <= got.numel() // 50
    gen = torch.Generator().manual_seed(12)
    for rows, width, wdtype in ((33, 1536, torch.float32), (7, 100, torch.float32), (64, 4096, torch.bfloat16)):
        x = torch.randn(rows, width, generator=gen).bfloat16()
        dy = torch.randn(rows, width, generator=gen).bfloat16()
        w = (torch.randn(width, generator=gen) * 0.1 + 1.0).to(wdtype)
        got = run(x.cuda(), w.cuda(), dy.cuda(), 1e-6, 0.25)
        want = oracle.rmsnorm_backward(dy, x, w, 1e-6, 0.25)
        assert oracle.rel_frobenius(got, want) <= 4e-3, (rows, width)


def test_fused_adamw_matches_torch(native_library):
    """Five steps of the flat AdamW kernel against torch.optim.AdamW on the same gradients."""
    from molt_b200.data_parallel import GradArena, ParamArena

    gen = torch.Generator(device="cuda").manual_seed(4)
    shapes = [(16, 128), (256, 16), (5, 7)]
    ours = [torch.nn.Parameter(torch.randn(*s, device="cuda", generator=gen)) for s in shapes]
    theirs = [torch.nn.Parameter(p.detach().clone()) for p in ours]
    arena = GradArena(ours)
    opt = ParamArena(arena, lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref = torch.optim.AdamW(theirs, lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(5):
        arena.zero()
        for p, q in zip(ours, theirs):
            g = torch.randn(p.shape, device="cuda", generator=gen)
            p.grad.add_(2.0 * g)          # the kernel scales by grad_scale = 0.5
            q.grad = g.clone()
        opt.step(grad_scale=0.5)
        ref.step()
    for p, q in zip(ours, theirs):
        torch.testing.assert_close(p.detach(), q.detach(), rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("n,k,m", [(1024, 256, 300), (151936, 1536, 512), (4096, 1024, 4096), (320, 64, 1)])
@pytest.mark.parametrize("over_rows", [False, True])
def test_dense_gemm_matches_fp32_matmul(native_library, n, k, m, over_rows):
    """The frozen-head GEMMs (logits = h . head^T and dh = dlogits . head) on the library's dense tensor-core kernel against
    an fp32 matmul of the same bf16 operands; tolerance 1e-2 relative Frobenius like the linears (measured ~2e-3)."""
    from molt_b200 import _native
    from molt_b200.qlora_step import dense_gemm
    from oracle import molt_oracle as oracle

    gen = torch.Generator(device="cuda").manual_seed(n + k + m)
    weight = (torch.randn(n, k, device="cuda", generator=gen) * 0.05).bfloat16()
    x = torch.randn(m, n if over_rows else k, device="cuda", generator=gen).bfloat16()
    if n > 100000 and over_rows:
        x *= 0.01          # keep the long contraction's result in a comfortable range
    for flags in (0, _native.PATH_SHORT_TILES, _native.PATH_TALL_TILES | _native.PATH_FORCE_SPLIT):
        got = dense_gemm(weight, x, over_rows, flags)
        want = x.float() @ (weight.float() if over_rows else weight.float().t())
        assert oracle.rel_frobenius(got, want) <= 1e-2, flags
    assert _native.read_status() == 0


def test_add_rmsnorm_matches_the_separate_ops(native_library):
    """Residual add fused with the norm behind it: the sum is the bf16 add, the norm equals molt_rmsnorm_fwd on that sum,
    and the backward equals RMSNorm backward plus the gradient arriving on the stream (fp32 reference, 1e-2)."""
    from molt_b200.qlora_step import RMSNorm, _AddFrozenRMSNorm

    gen = torch.Generator(device="cuda").manual_seed(5)
    rows, width = 300, 1536
    x = (torch.randn(2, rows // 2, width, device="cuda", generator=gen)).bfloat16().requires_grad_()
    delta = (torch.randn(2, rows // 2, width, device="cuda", generator=gen) * 0.5).bfloat16().requires_grad_()
    norm = RMSNorm(width, torch.device("cuda"))
    with torch.no_grad():
        norm.weight.copy_((1 + 0.1 * torch.randn(width, device="cuda", generator=gen)).bfloat16())
    stream, normed = _AddFrozenRMSNorm.apply(x, delta, norm.weight, norm.eps)
    assert torch.equal(stream, x.detach() + delta.detach())
    assert torch.equal(normed, norm(stream.detach()))
    g_stream = torch.randn_like(stream)
    g_normed = torch.randn_like(normed)
    torch.autograd.backward([stream, normed], [g_stream, g_normed])
    # fp32 reference
    xs = (x.detach().float() + delta.detach().float()).bfloat16().float().requires_grad_()
    ref = torch.nn.functional.rms_norm(xs, (width,), norm.weight.float(), norm.eps)
    ref.backward(g_normed.float())
    expected = xs.grad + g_stream.float()
    for grad in (x.grad, delta.grad):
        assert (grad.float() - expected).norm() / expected.norm() <= 1e-2
    assert torch.equal(x.grad, delta.grad)


def test_rope_kernel_matches_torch(native_library):
    """Rotary embedding of q and k in one kernel each against the cat/mul formulation in fp32; the gradient is the
    transposed rotation."""
    from molt_b200.qlora_step import _Rope, _rope

    gen = torch.Generator(device="cuda").manual_seed(6)
    b, s, heads, kv, d = 2, 96, 6, 2, 64
    inv = 1.0 / (1e4 ** (torch.arange(0, d, 2, device="cuda").float() / d))
    angles = torch.outer(torch.arange(s, device="cuda").float(), inv)
    angles = torch.cat((angles, angles), dim=-1)
    cos, sin = angles.cos().bfloat16(), angles.sin().bfloat16()
    q0 = torch.randn(b, s, heads * d, device="cuda", generator=gen).bfloat16()
    k0 = torch.randn(b, s, kv * d, device="cuda", generator=gen).bfloat16()
    ql, kl = q0.clone().requires_grad_(), k0.clone().requires_grad_()
    q = _Rope.apply(ql, cos, sin, heads, d)
    k = _Rope.apply(kl, cos, sin, kv, d)

    def reference(x, n):
        x = x.float().view(b, s, n, d).transpose(1, 2)
        return _rope(x, cos.float()[None, None], sin.float()[None, None]).transpose(1, 2).reshape(b, s, n * d)

    qr, kr = q0.float().requires_grad_(), k0.float().requires_grad_()
    q_ref, k_ref = reference(qr, heads), reference(kr, kv)
    assert (q.float() - q_ref).abs().max() <= 2e-2 and (k.float() - k_ref).abs().max() <= 2e-2
    gq, gk = torch.randn_like(q), torch.randn_like(k)
    torch.autograd.backward([q, k], [gq, gk])
    torch.autograd.backward([q_ref, k_ref], [gq.float(), gk.float()])
    assert (ql.grad.float() - qr.grad).abs().max() <= 3e-2 and (kl.grad.float() - kr.grad).abs().max() <= 3e-2


def test_step_with_lora_shadows_equals_step_without(native_library):
    """The adapters' bf16 operands refreshed behind each optimizer step, against converting them in front of every
    call: the same kernels see the same operands, so losses and adapters agree bit for bit over several steps."""
    from molt_b200 import _native
    from molt_b200.qlora_step import DecoderShape, QLoRAStep

    shape = DecoderShape(layers=2, hidden=128, heads=4, kv_heads=2, head_dim=32, intermediate=256, vocab=512,
                         rope_theta=1e4, rank=8, alpha=16.0, nested_absmax=False, seq_len=64, micro_batch=4)
    gen = torch.Generator(device="cuda").manual_seed(3)
    tokens = torch.randint(0, shape.vocab, (shape.micro_batch, shape.seq_len), device="cuda", generator=gen)
    targets = torch.roll(tokens, -1, dims=1)
    runs = []
    for shadows in (True, False):
        step = QLoRAStep(shape, torch.device("cuda"), lr=5e-3, lora_shadows=shadows)
        assert (step.shadows is not None) == shadows
        if shadows:
            assert len(step.shadows.shadows) == 2 * 7
        with torch.autocast("cuda", dtype=torch.bfloat16):
            losses = [step.run(tokens, targets).clone() for _ in range(4)]
        runs.append((torch.stack(losses), step.optimizer.flat.clone()))
    assert torch.equal(runs[0][0], runs[1][0])
    assert torch.equal(runs[0][1], runs[1][1])
    assert float(runs[0][0][-1]) < float(runs[0][0][0])
    assert _native.read_status() == 0


@pytest.mark.parametrize("joint", [False, True])
def test_static_cuda_microbatch_replays_the_fused_ops(native_library, joint):
    """The reference's captured micro-batch runner (training/static_cuda_graph.py:139-308) around a small stack of
    NF4-LoRA linears: replays give the eager loss and gradients, gradients accumulate until zero_grad, inputs of
    another signature are refused."""
    from molt_b200.core.errors import CapabilityError
    from molt_b200.methods import quantize_nf4
    from molt_b200.modules import NF4LoRALinear
    from molt_b200.training import StaticCudaMicrobatch

    gen = torch.Generator(device="cuda").manual_seed(11)
    layers = []
    for n, k in ((256, 128), (128, 256)):
        packed, state = quantize_nf4(torch.randn(n, k, device="cuda", generator=gen) * 0.05, 64, True)
        lin = NF4LoRALinear(packed, state, 8, 16.0)
        with torch.no_grad():
            lin.lora_B["default"].weight.normal_(0.0, 0.02, generator=gen)
        layers.append(lin)
    params = [p for lin in layers for p in lin.parameters() if p.requires_grad]
    assert len(params) == 4

    def loss_of(x, target):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            h = layers[1](torch.nn.functional.silu(layers[0](x)))
        return ((h.float() - target) ** 2).mean()

    x = torch.randn(96, 128, device="cuda", generator=gen).bfloat16()
    target = torch.randn(96, 128, device="cuda", generator=gen)
    x2 = torch.randn(96, 128, device="cuda", generator=gen).bfloat16()
    def eager_pass(*inputs):   # nothing of its autograd graph outlives the call (a live graph would pin the
        for p in params:       # gradient-accumulation nodes to this stream and break the capture below)
            p.grad = None
        loss = loss_of(*inputs)
        loss.backward()
        return loss.detach().clone(), [p.grad.clone() for p in params]

    eager = [eager_pass(x, target), eager_pass(x2, target)]
    for p in params:
        p.grad = None
    runner = StaticCudaMicrobatch(loss_of, (x, target), params, warmup_steps=2, joint_forward_backward=joint)
    assert [s.shape for s in runner.signatures] == [(96, 128), (96, 128)]
    assert all(float(p.grad.abs().sum()) == 0.0 for p in params)
    for (loss_ref, grads_ref), inputs in zip(eager, ((x, target), (x2, target))):
        runner.zero_grad()
        loss = runner.replay(*inputs)
        torch.cuda.synchronize()
        assert torch.equal(loss, loss_ref)
        assert all(torch.equal(p.grad, g) for p, g in zip(params, grads_ref))
    runner.replay(x2, target)                      # a second replay accumulates, like a second eager backward
    torch.cuda.synchronize()
    assert all(torch.allclose(p.grad, 2 * g, rtol=1e-6, atol=0) for p, g in zip(params, eager[1][1]))
    with pytest.raises(ValueError):
        runner.replay(x[:10], target)
    with pytest.raises(ValueError):
        runner.replay(x)
    with pytest.raises(RuntimeError):
        (runner.replay_forward if joint else runner.replay_staged)(*(() if not joint else (x, target)))
    runner.close()
    with pytest.raises(ValueError):
        StaticCudaMicrobatch(loss_of, (x, target), params, warmup_steps=0)
    with pytest.raises(CapabilityError):
        StaticCudaMicrobatch(loss_of, (x.cpu(), target), params)
    from molt_b200 import _native
    assert _native.read_status() == 0


def test_bnb_format_checkpoint_feeds_the_kernels(native_library, tmp_path):
    """A double-quantised NF4 weight written in the bitsandbytes state-dict layout, read back from a .safetensors file
    and handed to the fused linear, gives what the original quant state gives."""
    from molt_b200.methods import quantize_nf4, scheduled_nf4_lora
    from molt_b200.training import bnb_nf4_weight, export_bnb_nf4_weight, read_safetensors, write_safetensors

    gen = torch.Generator(device="cuda").manual_seed(21)
    packed, state = quantize_nf4(torch.randn(320, 192, device="cuda", generator=gen) * 0.03, 64, True)
    name = "model.layers.3.mlp.up_proj.weight"
    write_safetensors(tmp_path / "m.safetensors", export_bnb_nf4_weight(name, packed, state))
    packed2, state2 = bnb_nf4_weight(read_safetensors(tmp_path / "m.safetensors"), name, device="cuda")
    a = torch.randn(8, 192, device="cuda", generator=gen) * 0.01
    b = torch.randn(320, 8, device="cuda", generator=gen) * 0.01
    for m in (4, 40, 300):
        x = torch.randn(m, 192, device="cuda", generator=gen).bfloat16()
        assert torch.equal(scheduled_nf4_lora(x, packed2, a, b, state2, 2.0), scheduled_nf4_lora(x, packed, a, b, state, 2.0))
