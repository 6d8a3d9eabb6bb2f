"""A minimal QLoRA training step on a synthetic-weight decoder whose seven projections per layer run through the
NF4-LoRA kernels: the caller-side harness for BASELINE configs 4 (Qwen2.5-1.5B shape) and 5 (Llama-3-8B shape).

The reference drives this path from its trainer (reference training/qlora.py:485-1109) with Hugging Face
checkpoints; checkpoints and datasets are not available here, so the decoder is random-initialised with the same
architecture and fed uniform random token ids.  Attention (torch SDPA) and RoPE are plain PyTorch -- they are callers of the hot path, not part of it.  The frozen
RMSNorm (forward and backward), the in-place softmax gradient of the frozen-head cross-entropy and the AdamW step over
the flat adapter arena are this library's kernels.  Data parallelism: one process per GPU; the LoRA gradients live in
one flat arena whose per-layer buckets are all-reduced over NCCL on a side stream while the backward of the earlier
layers is still running (``molt_b200.data_parallel``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
from torch import nn
from torch.nn import functional as F

from molt_b200 import _native
from molt_b200.data_parallel import GradArena, ParamArena, StepGuard, lora_parameters
from molt_b200.methods._linear import LoraShadows, ShadowTable
from molt_b200.methods.quant_state import NestedState, QuantState
from molt_b200.modules import GatedMLP, NF4LoRALinear
from molt_b200.streaming.nf4 import NF4_CODEBOOK


@dataclass(frozen=True)
class DecoderShape:
    layers: int
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    rope_theta: float
    rank: int
    alpha: float
    nested_absmax: bool
    seq_len: int
    micro_batch: int

    @property
    def tokens(self) -> int:
        return self.seq_len * self.micro_batch


QWEN25_1P5B = DecoderShape(28, 1536, 12, 2, 128, 8960, 151936, 1e6, 16, 32.0, False, 1024, 8)      # BASELINE config 4
LLAMA3_8B = DecoderShape(32, 4096, 32, 8, 128, 14336, 128256, 5e5, 64, 128.0, True, 2048, 4)       # BASELINE config 5


def quantize_fast(weight: torch.Tensor, nested: bool, nibble_order: str = "high-first"):
    """NF4-quantise a freshly drawn synthetic weight on its device.  The nearest level is found through the
    midpoints between codebook entries (identical to the arg-min quantiser except at exact midpoints), which is
    what makes building a 28- or 32-layer model take seconds."""
    device = weight.device
    blocks = weight.float().reshape(-1, 64)
    absmax = blocks.abs().amax(dim=1).clamp_min(torch.finfo(torch.float32).tiny)
    levels = NF4_CODEBOOK.to(device)
    codes = torch.bucketize(blocks / absmax[:, None], (levels[1:] + levels[:-1]) / 2).to(torch.uint8)
    packed = ((codes[:, 0::2] << 4) | codes[:, 1::2]) if nibble_order == "high-first" else (codes[:, 0::2] | (codes[:, 1::2] << 4))
    state = QuantState(absmax=absmax.contiguous(), shape=tuple(weight.shape), code=levels, nibble_order=nibble_order)
    if nested:
        table = torch.linspace(-1.0, 1.0, 256, device=device)
        offset = absmax.mean()
        residual = absmax - offset
        pad = (-residual.numel()) % 256
        groups = (F.pad(residual, (0, pad)) if pad else residual).reshape(-1, 256)
        absmax2 = groups.abs().amax(dim=1).clamp_min(torch.finfo(torch.float32).tiny)
        codes2 = torch.bucketize(groups / absmax2[:, None], (table[1:] + table[:-1]) / 2).to(torch.uint8)
        state.absmax = codes2.reshape(-1)[: residual.numel()].contiguous()
        state.nested = True
        state.state2 = NestedState(absmax2.contiguous(), table, 256)
        state.offset = float(offset)
    return packed.reshape(-1, 1).contiguous(), state


def _projection(out_features: int, in_features: int, shape: DecoderShape, gen: torch.Generator, device) -> NF4LoRALinear:
    weight = torch.randn(out_features, in_features, device=device, generator=gen) * 0.02
    packed, state = quantize_fast(weight, shape.nested_absmax)
    lin = NF4LoRALinear(packed, state, shape.rank, shape.alpha)
    with torch.no_grad():  # B = 0 would make every dA vanish; draw it as BASELINE's configs do
        lin.lora_A["default"].weight.normal_(0.0, 0.01, generator=gen)
        lin.lora_B["default"].weight.normal_(0.0, 0.01, generator=gen)
    return lin


class _FrozenRMSNorm(torch.autograd.Function):
    """RMSNorm with a frozen weight: fp32 reduction, bf16 in and out, gradient for the input only (the contract of
    reference kernels/frozen_rmsnorm.py:9-37)."""

    @staticmethod
    def forward(ctx, hidden, weight, eps):
        rows = hidden.reshape(-1, hidden.shape[-1])
        if not rows.is_contiguous():
            rows = rows.contiguous()
        out = torch.empty_like(rows)
        dtype = _native.DTYPE_F32 if weight.dtype == torch.float32 else _native.DTYPE_BF16
        with torch.cuda.device(rows.device):
            _native.check(_native.library().molt_rmsnorm_fwd(rows.data_ptr(), weight.data_ptr(), dtype, float(eps), 0.0,
                                                             out.data_ptr(), rows.shape[0], rows.shape[1],
                                                             _native.stream_handle(rows.device)))
        ctx.save_for_backward(rows, weight)
        ctx.eps, ctx.weight_dtype, ctx.shape = float(eps), dtype, hidden.shape
        return out.reshape(hidden.shape)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_output):
        rows, weight = ctx.saved_tensors
        grad = grad_output.reshape(rows.shape)
        if grad.dtype != torch.bfloat16:
            grad = grad.to(torch.bfloat16)
        if not grad.is_contiguous():
            grad = grad.contiguous()
        out = torch.empty_like(rows)
        with torch.cuda.device(rows.device):
            _native.check(_native.library().molt_rmsnorm_bwd(grad.data_ptr(), rows.data_ptr(), weight.data_ptr(),
                                                             ctx.weight_dtype, ctx.eps, 0.0, out.data_ptr(), rows.shape[0],
                                                             rows.shape[1], _native.stream_handle(rows.device)))
        return out.reshape(ctx.shape), None, None


class _AddFrozenRMSNorm(torch.autograd.Function):
    """``stream = residual + delta`` and ``normed = RMSNorm(stream)`` in one pass over the hidden states; in backward one
    kernel adds the RMSNorm gradient to the gradient arriving on ``stream`` (what autograd would otherwise accumulate
    with a separate add)."""

    @staticmethod
    def forward(ctx, residual, delta, weight, eps):
        rows = residual.reshape(-1, residual.shape[-1])
        other = delta.reshape(rows.shape)
        rows = rows if rows.is_contiguous() else rows.contiguous()
        other = other if other.is_contiguous() else other.contiguous()
        stream, normed = torch.empty_like(rows), torch.empty_like(rows)
        dtype = _native.DTYPE_F32 if weight.dtype == torch.float32 else _native.DTYPE_BF16
        with torch.cuda.device(rows.device):
            _native.check(_native.library().molt_add_rmsnorm_fwd(rows.data_ptr(), other.data_ptr(), weight.data_ptr(), dtype,
                                                                 float(eps), 0.0, stream.data_ptr(), normed.data_ptr(),
                                                                 rows.shape[0], rows.shape[1],
                                                                 _native.stream_handle(rows.device)))
        ctx.save_for_backward(stream, weight)
        ctx.eps, ctx.weight_dtype, ctx.shape = float(eps), dtype, residual.shape
        return stream.reshape(residual.shape), normed.reshape(residual.shape)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_stream, grad_normed):
        stream, weight = ctx.saved_tensors

        def rows_of(grad):
            grad = grad.reshape(stream.shape)
            if grad.dtype != torch.bfloat16:
                grad = grad.to(torch.bfloat16)
            return grad if grad.is_contiguous() else grad.contiguous()

        gs, gn = rows_of(grad_stream), rows_of(grad_normed)
        out = torch.empty_like(stream)
        with torch.cuda.device(stream.device):
            _native.check(_native.library().molt_add_rmsnorm_bwd(gn.data_ptr(), gs.data_ptr(), stream.data_ptr(),
                                                                 weight.data_ptr(), ctx.weight_dtype, ctx.eps, 0.0,
                                                                 out.data_ptr(), stream.shape[0], stream.shape[1],
                                                                 _native.stream_handle(stream.device)))
        out = out.reshape(ctx.shape)
        return out, out, None, None


class _Rope(torch.autograd.Function):
    """Rotary embedding of one projection output (``[batch, seq, heads * head_dim]``) in one kernel; the gradient is
    the transposed rotation."""

    @staticmethod
    def forward(ctx, x, cos, sin, heads, head_dim):
        ctx.save_for_backward(cos, sin)
        ctx.dims = (x.shape[0], x.shape[1], heads, head_dim)
        x = x.contiguous()
        out = torch.empty_like(x)
        _Rope._launch(x, out, cos, sin, ctx.dims, 0)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad):
        cos, sin = ctx.saved_tensors
        grad = grad.contiguous()
        out = torch.empty_like(grad)   # the incoming buffer is autograd's
        _Rope._launch(grad, out, cos, sin, ctx.dims, 1)
        return out, None, None, None, None

    @staticmethod
    def _launch(x, out, cos, sin, dims, inverse):
        batch, seq, heads, head_dim = dims
        with torch.cuda.device(x.device):
            _native.check(_native.library().molt_rope(x.data_ptr(), x.data_ptr(), out.data_ptr(), out.data_ptr(),
                                                      cos.data_ptr(), sin.data_ptr(), batch, seq, heads, 0, head_dim,
                                                      inverse, _native.stream_handle(x.device)))


class RMSNorm(nn.Module):
    def __init__(self, width: int, device, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width, device=device, dtype=torch.bfloat16), requires_grad=False)
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda and x.dtype == torch.bfloat16:
            return _FrozenRMSNorm.apply(x, self.weight, self.eps)
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)

    def add_and_norm(self, residual: torch.Tensor, delta: torch.Tensor):
        """``(residual + delta, self(residual + delta))``, fused on the GPU."""
        if residual.is_cuda and residual.dtype == torch.bfloat16 and delta.dtype == torch.bfloat16 and residual.shape[-1] % 8 == 0:
            return _AddFrozenRMSNorm.apply(residual, delta, self.weight, self.eps)
        stream = residual + delta
        return stream, self(stream)


class Attention(nn.Module):
    def __init__(self, shape: DecoderShape, gen, device):
        super().__init__()
        self.shape = shape
        h, kv, d = shape.heads, shape.kv_heads, shape.head_dim
        self.q_proj = _projection(h * d, shape.hidden, shape, gen, device)
        self.k_proj = _projection(kv * d, shape.hidden, shape, gen, device)
        self.v_proj = _projection(kv * d, shape.hidden, shape, gen, device)
        self.o_proj = _projection(shape.hidden, h * d, shape, gen, device)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        b, s, _ = x.shape
        sh = self.shape
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        fused = q.is_cuda and q.dtype == torch.bfloat16 and sh.head_dim % 16 == 0 and cos.shape[-2] == s
        if fused:   # one kernel per projection ([batch, seq, heads, head_dim] layout)
            cos2, sin2 = cos.reshape(s, sh.head_dim), sin.reshape(s, sh.head_dim)
            q = _Rope.apply(q, cos2, sin2, sh.heads, sh.head_dim)
            k = _Rope.apply(k, cos2, sin2, sh.kv_heads, sh.head_dim)
        q = q.view(b, s, sh.heads, sh.head_dim).transpose(1, 2)
        k = k.view(b, s, sh.kv_heads, sh.head_dim).transpose(1, 2)
        v = v.view(b, s, sh.kv_heads, sh.head_dim).transpose(1, 2)
        if not fused:
            q = _rope(q, cos, sin)
            k = _rope(k, cos, sin)
        out = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        return self.o_proj(out.transpose(1, 2).reshape(b, s, sh.heads * sh.head_dim))


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    rotated = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos + rotated * sin


class DecoderLayer(nn.Module):
    def __init__(self, shape: DecoderShape, gen, device):
        super().__init__()
        self.input_norm = RMSNorm(shape.hidden, device)
        self.attn = Attention(shape, gen, device)
        self.post_norm = RMSNorm(shape.hidden, device)
        self.mlp = GatedMLP(_projection(shape.intermediate, shape.hidden, shape, gen, device),
                            _projection(shape.intermediate, shape.hidden, shape, gen, device),
                            _projection(shape.hidden, shape.intermediate, shape, gen, device))

    def forward(self, x, cos, sin, replay_up: bool, on_backward_done=None):
        """The layer on its own: returns the residual stream after it."""
        stream, delta = self.step(x, None, cos, sin, replay_up, on_backward_done)
        return stream + delta

    def step(self, residual, delta, cos, sin, replay_up: bool, on_backward_done=None):
        """The layer inside a stack.  The stream entering it is ``residual + delta`` (``delta`` None: just ``residual``);
        returns ``(stream after the attention block, output of the MLP)``, so that the add of the MLP output is fused
        with the next norm (the next layer's, or the final one)."""
        if delta is None:
            stream, normed = residual, self.input_norm(residual)
        else:
            stream, normed = self.input_norm.add_and_norm(residual, delta)
        if on_backward_done is not None and normed.requires_grad:
            # fires when the gradient of the attention block's input exists, i.e. when every adapter gradient of the
            # layer has been written (the MLP's came first): the moment its bucket can go to the all-reduce
            normed.register_hook(on_backward_done)
        stream, normed = self.post_norm.add_and_norm(stream, self.attn(normed, cos, sin))
        b, s, w = normed.shape
        return stream, self.mlp.fused(normed.reshape(b * s, w), rematerialize_up=replay_up).view(b, s, w)


def dense_gemm(weight: torch.Tensor, x: torch.Tensor, contract_over_rows: bool, flags: int = 0) -> torch.Tensor:
    """``x @ weight.T`` (or ``x @ weight`` with ``contract_over_rows``) for a frozen bf16 weight ``[n, k]`` on the library's
    tensor-core kernel (the NF4 linears' kernel with ready-made B tiles)."""
    n, k = int(weight.shape[0]), int(weight.shape[1])
    m = int(x.shape[0])
    lib = _native.library()
    out = torch.empty((m, k if contract_over_rows else n), dtype=torch.bfloat16, device=x.device)
    ws = _native.workspace(lib.molt_dense_gemm_workspace_bytes(), x.device)
    with torch.cuda.device(x.device):
        _native.check(lib.molt_dense_gemm(weight.data_ptr(), n, k, x.data_ptr(), out.data_ptr(), m, int(contract_over_rows),
                                          ws.data_ptr(), ws.numel(), int(flags), _native.stream_handle(x.device)))
    return out


class _FrozenHeadLoss(torch.autograd.Function):
    """Mean token cross-entropy through a frozen bf16 LM head, in row chunks, without keeping the logits:
    logits = h . head^T, then one fused kernel turns the bf16 logits in place into the softmax gradient and emits the
    per-row loss, then dh = grad . head -- both GEMMs on the library's dense tensor-core kernel (the scheme of reference
    kernels/frozen_linear_cross_entropy.py:181-236; with 180 GB of HBM a chunk is the whole micro-batch by default)."""

    @staticmethod
    def forward(ctx, hidden, head, targets, chunk, denominator):
        lib = _native.library()
        rows, vocab = hidden.shape[0], head.shape[0]
        grad = torch.empty_like(hidden)
        row_loss = torch.empty(rows, device=hidden.device, dtype=torch.float32)
        targets = targets.contiguous()
        hidden = hidden.contiguous()
        native = hidden.dtype == torch.bfloat16 and head.dtype == torch.bfloat16 and vocab % 64 == 0 and hidden.shape[1] % 64 == 0
        for start in range(0, rows, chunk):
            h = hidden[start:start + chunk]
            logits = dense_gemm(head, h, False) if native else h @ head.t()
            with torch.cuda.device(hidden.device):
                _native.check(lib.molt_ce_softmax_grad(
                    logits.data_ptr(), targets[start:start + chunk].data_ptr(), row_loss[start:start + chunk].data_ptr(),
                    logits.shape[0], vocab, 1.0 / denominator, _native.stream_handle(hidden.device)))
            grad[start:start + chunk] = dense_gemm(head, logits, True) if native else logits @ head
        ctx.save_for_backward(grad)
        return row_loss.sum() / denominator

    @staticmethod
    def backward(ctx, grad_output):
        (grad,) = ctx.saved_tensors
        return grad * grad_output.to(grad.dtype), None, None, None, None


class SyntheticDecoder(nn.Module):
    def __init__(self, shape: DecoderShape, device, seed: int = 1337, layers: Optional[int] = None):
        super().__init__()
        self.shape = shape
        gen = torch.Generator(device=device).manual_seed(seed)
        self.embed = nn.Parameter((torch.randn(shape.vocab, shape.hidden, device=device, generator=gen) * 0.02).bfloat16(),
                                  requires_grad=False)
        self.head = nn.Parameter((torch.randn(shape.vocab, shape.hidden, device=device, generator=gen) * 0.02).bfloat16(),
                                 requires_grad=False)
        self.layers = nn.ModuleList(DecoderLayer(shape, gen, device) for _ in range(layers or shape.layers))
        self.final_norm = RMSNorm(shape.hidden, device)
        self.head_chunk = 8192   # rows of logits alive at a time (8192 x 151936 bf16 = 2.5 GB at config 4's vocabulary)
        inv = 1.0 / (shape.rope_theta ** (torch.arange(0, shape.head_dim, 2, device=device).float() / shape.head_dim))
        angles = torch.outer(torch.arange(shape.seq_len, device=device).float(), inv)
        angles = torch.cat((angles, angles), dim=-1)
        self.register_buffer("cos", angles.cos().bfloat16()[None, None], persistent=False)
        self.register_buffer("sin", angles.sin().bfloat16()[None, None], persistent=False)

    def loss(self, tokens: torch.Tensor, targets: torch.Tensor, global_tokens: int, replay_up: bool = True,
             layer_done=None) -> torch.Tensor:
        """``layer_done(index)``, when given, is called during backward as soon as layer ``index`` has produced all of
        its adapter gradients (layers finish from the last to the first)."""
        stream, delta = F.embedding(tokens, self.embed).requires_grad_(), None
        for index, layer in enumerate(self.layers):
            hook = None
            if layer_done is not None:
                def hook(grad, index=index):
                    layer_done(index)
                    return grad
            stream, delta = layer.step(stream, delta, self.cos, self.sin, replay_up, hook)
        _, hidden = self.final_norm.add_and_norm(stream, delta)
        hidden = hidden.reshape(-1, self.shape.hidden)
        return _FrozenHeadLoss.apply(hidden, self.head, targets.reshape(-1), self.head_chunk, float(global_tokens))


def attach_lora_shadows(model: nn.Module) -> list:
    """Give every active adapter of ``model``'s NF4-LoRA linears its bf16 operand buffers and make the fused ops use them;
    returns the list (for a :class:`ShadowTable`).  The caller refreshes them whenever the masters change."""
    made = []
    for module in model.modules():
        if isinstance(module, NF4LoRALinear):
            for adapter in module.active_adapters:
                shadow = LoraShadows(module.lora_A[adapter].weight, module.lora_B[adapter].weight,
                                     float(module.scaling[adapter]))
                shadow.attach()
                made.append(shadow)
    return made


class QLoRAStep:
    """Holds model, gradient arena and optimiser; ``run(tokens, targets)`` is one data-parallel training step.

    Step anatomy: zero the gradient arena; forward; backward, during which every decoder layer's bucket of the arena
    goes to the all-reduce (side stream) as soon as the layer's backward has run, so the exchange overlaps the backward
    of the layers before it; join; one fused AdamW launch over the flat parameter arena (gradients scaled by 1 / world
    in the same pass).  Forward + backward + collectives replay as one CUDA graph once warmed up.  Every
    ``status_interval`` steps the device status word of the bounded waits is read (a host synchronisation) and a
    non-zero value raises; with a :class:`StepGuard` the ranks also check each other on the host before each step."""

    def __init__(self, shape: DecoderShape, device, layers: Optional[int] = None, lr: float = 1e-4,
                 cuda_graph: bool = False, status_interval: int = 50, guard: Optional[StepGuard] = None,
                 lora_shadows: bool = True):
        self.shape = shape
        self.device = device
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.model = SyntheticDecoder(shape, device, layers=layers)
        params = lora_parameters(self.model)
        # one bucket per decoder layer: the index of each layer's first adapter parameter
        identity = {id(p): i for i, p in enumerate(params)}
        starts = sorted(min(identity[id(p)] for p in layer.parameters() if p.requires_grad) for layer in self.model.layers)
        self.arena = GradArena(params, bucket_starts=starts)
        self.layer_bucket = [self.arena.bucket_of_param(start) for start in starts]
        self.optimizer = ParamArena(self.arena, lr=lr, weight_decay=0.0)
        # bf16 operands of every adapter, rebuilt by one launch behind each optimizer step (made after the parameter
        # arena: they record the masters' final addresses), so that no linear call converts its adapter first
        self.shadows = ShadowTable(attach_lora_shadows(self.model)) if lora_shadows else None
        if self.shadows is not None:
            self.shadows.refresh()
        self.cuda_graph = cuda_graph
        self.status_interval = int(status_interval)
        self.guard = guard
        self.steps = 0
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._static_tokens = self._static_targets = self._static_loss = None
        self._eager_steps = 0
        self.graph_launches = 0      # library kernel launches recorded in the CUDA graph
        self.replayed_launches = 0   # library kernel launches executed through graph replays so far

    def _layer_done(self, index: int) -> None:
        if self.world > 1:
            self.arena.all_reduce_bucket(self.layer_bucket[index])

    def _forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        self.arena.zero()
        loss = self.model.loss(tokens, targets, self.shape.tokens * self.world,
                               layer_done=self._layer_done if self.world > 1 else None)
        loss.backward()
        self.arena.wait()            # the current stream joins the collectives issued from the backward
        return loss.detach()

    def _capture(self, tokens: torch.Tensor, targets: torch.Tensor) -> None:
        """Record forward + backward (+ the overlapped collectives) of one micro-batch once; every later step replays
        the recording (the kernels take raw pointers and never allocate or synchronise, so they are capture-safe)."""
        self._static_tokens = tokens.clone()
        self._static_targets = targets.clone()
        self._graph = torch.cuda.CUDAGraph()
        lib = _native.library()
        before = lib.molt_launch_count()
        with torch.cuda.graph(self._graph):
            self._static_loss = self._forward_backward(self._static_tokens, self._static_targets)
        self.graph_launches = int(lib.molt_launch_count() - before)   # library kernels recorded; each replay runs them

    def run(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        if self.guard is not None:
            self.guard.check(self.steps)     # host-side: every peer is alive and about to run the same step
        if self.cuda_graph and self._graph is None and self._eager_steps >= 2:
            self._capture(tokens, targets)
        if self._graph is not None:
            self._static_tokens.copy_(tokens)
            self._static_targets.copy_(targets)
            self._graph.replay()
            self.replayed_launches += self.graph_launches
            loss = self._static_loss
        else:
            loss = self._forward_backward(tokens, targets)
            self._eager_steps += 1
        self.optimizer.step(grad_scale=1.0)  # the loss is already normalised by the global token count
        if self.shadows is not None:
            self.shadows.refresh()           # same stream, behind the step: the next forward sees the new adapters
        self.steps += 1
        if self.status_interval > 0 and self.steps % self.status_interval == 0:
            self.check_status()
        return loss

    def check_status(self) -> None:
        """Read the device status word (synchronises the stream); a bounded wait that expired left outputs incomplete."""
        status = _native.read_status(self.device)
        if status:
            raise RuntimeError(f"a bounded device-side wait expired (status 0x{status:08x}); the step's results are invalid")

    def lora_parameter_count(self) -> int:
        return sum(p.numel() for p in self.arena.params)


def hot_path_flops_per_token(shape: DecoderShape) -> float:
    """Algorithmic forward+backward FLOPs of the seven NF4-LoRA projections per token: 4·N·K + 6·r·(K+N) each."""
    h, kvw, qw, inter = shape.hidden, shape.kv_heads * shape.head_dim, shape.heads * shape.head_dim, shape.intermediate
    projections = [(qw, h), (kvw, h), (kvw, h), (h, qw), (inter, h), (inter, h), (h, inter)]
    per_layer = sum(4.0 * n * k + 6.0 * shape.rank * (n + k) for n, k in projections)
    return per_layer * shape.layers
