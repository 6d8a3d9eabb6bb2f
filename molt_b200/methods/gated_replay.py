"""Gated-MLP (SwiGLU) schedules that re-materialise activations instead of saving them.

Public names follow the reference's ``methods/gated_replay.py``:

* ``asymmetric_gated_nf4_lora`` / ``enable_asymmetric_gated_replay`` -- the down-projection node that keeps
  ``x`` and ``gate``, and replays the ``up`` projection in backward (reference :256-457, :540-607);
* ``gated_mlp_nf4_lora`` -- the whole block (gate, up, SwiGLU, down) as one autograd node, optionally
  re-materialising its RMS-normalised input from the residual stream (reference :13-208).

All arithmetic runs in the fused CUDA kernels; the eager ``silu`` / ``*`` / ``silu_backward`` chain of the
reference is one HBM pass forward and one backward.
"""
from __future__ import annotations

import ctypes
from types import MethodType
from typing import Any, Optional

import torch

from molt_b200 import _native
from molt_b200.core.errors import CapabilityError
from molt_b200.kernels.gated_activation import swiglu_backward, swiglu_forward
from molt_b200.methods._linear import (GRAD_SLOT, SHADOW_SLOT, check_linear_inputs, linear_backward, linear_forward,
                                       weight_desc_for_tokens)
from molt_b200.methods.nf4_lora import _adapter_of, _bf16_autocast_active, is_lora_4bit_linear


def _as_rows(tensor: torch.Tensor) -> torch.Tensor:
    flat = tensor.reshape(-1, tensor.shape[-1])
    return flat if flat.is_contiguous() else flat.contiguous()


class _AsymmetricGatedNF4LoRA(torch.autograd.Function):
    """Down projection of a gated MLP that re-materialises only the ``up`` branch.

    Forward receives the already computed gate/up projection results (their own autograd nodes stay in charge
    of the gate/up adapter gradients).  Kept for backward: ``x``, ``gate`` and -- unless replayed or
    offloaded -- ``up``; never ``silu(gate)`` or the gated product.
    """

    @staticmethod
    def forward(ctx: Any, x, gate, up, up_packed_weight, up_lora_a, up_lora_b, down_packed_weight, down_lora_a,
                down_lora_b, up_quant_state, down_quant_state, up_scaling, down_scaling, rematerialize_up,
                offload_up, host_up, offload_gate, host_gate):
        if x.device.type != "cuda" or x.dtype != torch.bfloat16:
            raise CapabilityError("asymmetric gated replay requires CUDA BF16 tensors")
        check_linear_inputs(gate, down_packed_weight, down_lora_a, down_lora_b, "asymmetric gated replay")
        ctx.rematerialize_up = bool(rematerialize_up)
        ctx.offload_up = bool(offload_up)
        ctx.offload_gate = bool(offload_gate)
        if ctx.rematerialize_up and ctx.offload_up:
            raise CapabilityError("up projection cannot be replayed and offloaded")
        if ctx.offload_up:
            if host_up.device.type != "cpu" or not host_up.is_pinned():
                raise CapabilityError("gated activation offload requires pinned host storage")
            if host_up.shape != up.shape or host_up.dtype != up.dtype:
                raise CapabilityError("gated activation host storage must match the up result")
        if ctx.offload_gate:
            if host_gate.device.type != "cpu" or not host_gate.is_pinned():
                raise CapabilityError("gated activation offload requires pinned gate storage")
            if host_gate.shape != gate.shape or host_gate.dtype != gate.dtype:
                raise CapabilityError("gated activation host storage must match the gate result")
        gate2, up2 = _as_rows(gate), _as_rows(up)
        hidden = swiglu_forward(gate2, up2)
        tokens = int(hidden.shape[0])
        down_desc = weight_desc_for_tokens(down_packed_weight, down_quant_state, tokens)
        result, t_down = linear_forward(down_desc, hidden, down_lora_a, down_lora_b, float(down_scaling), True)
        ctx.up_desc = weight_desc_for_tokens(up_packed_weight, up_quant_state, tokens)
        ctx.down_desc = down_desc
        ctx.states = (up_quant_state, down_quant_state)
        ctx.up_scaling = float(up_scaling)
        ctx.down_scaling = float(down_scaling)
        ctx.gate_shape = gate.shape
        ctx.slots = (getattr(down_lora_a, GRAD_SLOT, None), getattr(down_lora_b, GRAD_SLOT, None))
        if ctx.offload_up:
            host_up.copy_(up.detach(), non_blocking=True)
        if ctx.offload_gate:
            host_gate.copy_(gate.detach(), non_blocking=True)
        saved = (_as_rows(x), host_gate if ctx.offload_gate else gate2, up_packed_weight, up_lora_a, up_lora_b,
                 down_packed_weight, down_lora_a, down_lora_b, t_down)
        if ctx.offload_up:
            saved += (host_up,)
        elif not ctx.rematerialize_up:
            saved += (up2,)
        ctx.save_for_backward(*saved)
        return result.reshape(*gate.shape[:-1], result.shape[-1])

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_output: torch.Tensor):
        (x2, stored_gate, _up_w, up_a, up_b, _down_w, down_a, down_b, t_down, *retained) = ctx.saved_tensors
        device = grad_output.device
        gate2 = _as_rows(stored_gate.to(device, non_blocking=True)) if ctx.offload_gate else stored_gate
        if ctx.rematerialize_up:
            up2, _ = linear_forward(ctx.up_desc, x2, up_a, up_b, ctx.up_scaling, False)
        elif ctx.offload_up:
            up2 = _as_rows(retained[0].to(device, non_blocking=True))
        else:
            up2 = retained[0]
        dy2 = _as_rows(grad_output)
        if dy2.dtype != torch.bfloat16:
            dy2 = dy2.to(torch.bfloat16)
        hidden = swiglu_forward(gate2, up2)
        slot_a, slot_b = ctx.slots
        dh, d_down_a, d_down_b = linear_backward(ctx.down_desc, hidden, dy2, down_a, down_b, ctx.down_scaling, t_down,
                                                 True, True, slot_a, slot_b)
        dgate, dup = swiglu_backward(dh, gate2, up2)
        return (None, dgate.reshape(ctx.gate_shape), dup.reshape(ctx.gate_shape), None, None, None, None,
                d_down_a, d_down_b, None, None, None, None, None, None, None, None, None)


def asymmetric_gated_nf4_lora(
    x: torch.Tensor,
    gate: torch.Tensor,
    up: torch.Tensor,
    up_packed_weight: torch.Tensor,
    up_lora_a: torch.Tensor,
    up_lora_b: torch.Tensor,
    down_packed_weight: torch.Tensor,
    down_lora_a: torch.Tensor,
    down_lora_b: torch.Tensor,
    up_quant_state: Any,
    down_quant_state: Any,
    up_scaling: float,
    down_scaling: float,
    rematerialize_up: bool = True,
    offload_up: bool = False,
    host_up: torch.Tensor | None = None,
    offload_gate: bool = False,
    host_gate: torch.Tensor | None = None,
) -> torch.Tensor:
    """Signature and error behaviour of reference methods/gated_replay.py:410-457."""
    if offload_up and host_up is None:
        raise CapabilityError("gated activation offload requires a host buffer")
    if offload_gate and host_gate is None:
        raise CapabilityError("gated activation offload requires a gate host buffer")
    empty = torch.empty(0)
    return _AsymmetricGatedNF4LoRA.apply(
        x, gate, up, up_packed_weight, up_lora_a, up_lora_b, down_packed_weight, down_lora_a, down_lora_b,
        up_quant_state, down_quant_state, up_scaling, down_scaling, rematerialize_up, offload_up,
        empty if host_up is None else host_up, offload_gate, empty if host_gate is None else host_gate,
    )


# --------------------------------------------------------------------------------------------------------
# Whole block as one node.
# --------------------------------------------------------------------------------------------------------

def _proj_struct(desc, lora_a, lora_b, scaling, shadow=None) -> _native.LoraProj:
    proj = _native.LoraProj()
    proj.w = ctypes.pointer(desc)
    proj.lora_a = lora_a.data_ptr()
    proj.lora_b = lora_b.data_ptr()
    proj.scaling = float(scaling)
    proj.rank = int(lora_a.shape[0])
    if shadow is not None:   # the adapter's bf16 operands are kept up to date by its owner
        proj.shadow = ctypes.pointer(shadow.struct)
    return proj


def rmsnorm_bf16(source: torch.Tensor, weight: torch.Tensor, eps: float, weight_offset: float = 0.0) -> torch.Tensor:
    """``bf16(x * rsqrt(mean(x^2) + eps) * (w + offset))`` -- the norm-replay recipe (reference :22-29)."""
    if source.device.type != "cuda" or source.dtype != torch.bfloat16:
        raise CapabilityError("RMSNorm replay requires CUDA BF16 activations")
    rows = _as_rows(source)
    out = torch.empty_like(rows)
    w = weight.contiguous()
    if w.dtype not in (torch.float32, torch.bfloat16):
        raise CapabilityError("RMSNorm weight must be float32 or bfloat16")
    if rows.numel():
        with torch.cuda.device(rows.device):
            _native.check(_native.library().molt_rmsnorm_fwd(
                rows.data_ptr(), w.data_ptr(), _native.DTYPE_F32 if w.dtype == torch.float32 else _native.DTYPE_BF16,
                float(eps), float(weight_offset), out.data_ptr(), rows.shape[0], rows.shape[1],
                _native.stream_handle(rows.device)))
    return out.reshape(source.shape)


class _GatedMLPNF4LoRA(torch.autograd.Function):
    """gate, up, SwiGLU and down in one node; keeps ``gate`` and either ``x`` or the residual ``source``.

    The counterpart of the reference's ``_ResidualRecipeGatedNF4LoRA`` (methods/gated_replay.py:50-208): the
    gradient is returned for the normalised input, the six adapter gradients come back in fp32.
    """

    @staticmethod
    def forward(ctx: Any, x, source, norm_weight, gate_w, gate_a, gate_b, up_w, up_a, up_b, down_w, down_a, down_b,
                gate_state, up_state, down_state, gate_scaling, up_scaling, down_scaling, rematerialize_up, norm_eps,
                norm_weight_offset):
        for w, a, b in ((gate_w, gate_a, gate_b), (up_w, up_a, up_b), (down_w, down_a, down_b)):
            check_linear_inputs(x, w, a, b, "gated NF4-LoRA MLP")
        x2 = _as_rows(x)
        m = x2.shape[0]
        descs = tuple(weight_desc_for_tokens(w, st, int(m)) for w, st in ((gate_w, gate_state), (up_w, up_state),
                                                                          (down_w, down_state)))
        inter, hidden_width = int(descs[0].n), int(descs[0].k)
        if x2.shape[1] != hidden_width:
            raise ValueError("input width must match the gate/up projection in_features")
        adapters = [t.contiguous() for t in (gate_a, gate_b, up_a, up_b, down_a, down_b)]
        scalings = (float(gate_scaling), float(up_scaling), float(down_scaling))
        ctx.shadows = tuple(getattr(t, SHADOW_SLOT, None) for t in (gate_a, up_a, down_a))
        projs = [_proj_struct(descs[i], adapters[2 * i], adapters[2 * i + 1], scalings[i], ctx.shadows[i]) for i in range(3)]
        lib = _native.library()
        device = x2.device
        gate_out = torch.empty((m, inter), dtype=torch.bfloat16, device=device)
        keep_up = not bool(rematerialize_up)
        up_out = torch.empty((m, inter), dtype=torch.bfloat16, device=device) if keep_up else None
        y = torch.empty((m, int(descs[2].n)), dtype=torch.bfloat16, device=device)
        # the three low-rank inputs (x A^T of gate and up, h A^T of down; 384 bytes per token) are kept for the backward,
        # which then recomputes none of them
        needs_backward = any(ctx.needs_input_grad)
        low_rank = torch.empty((3, m, 64), dtype=torch.bfloat16, device=device) if needs_backward else None
        if m:
            nbytes = lib.molt_mlp_workspace_bytes(_native.OP_MLP_FWD, projs[0], projs[1], projs[2], m, int(keep_up))
            ws = _native.workspace(nbytes, device)
            with torch.cuda.device(device):
                _native.check(lib.molt_mlp_fwd_t(projs[0], projs[1], projs[2], x2.data_ptr(), gate_out.data_ptr(),
                                                 _native.ptr(up_out), y.data_ptr(), _native.ptr(low_rank), m, ws.data_ptr(),
                                                 ws.numel(), _native.stream_handle(device)))
        ctx.descs = descs
        ctx.states = (gate_state, up_state, down_state)
        ctx.scalings = scalings
        ctx.input_shape = x.shape
        ctx.replay_norm = source is not None
        ctx.norm = (float(norm_eps), float(norm_weight_offset))
        ctx.keep_up = keep_up
        ctx.slots = tuple(getattr(t, GRAD_SLOT, None) for t in (gate_a, gate_b, up_a, up_b, down_a, down_b))
        kept_input = source if ctx.replay_norm else x2
        saved = [kept_input, gate_out, gate_w, up_w, down_w, *adapters]
        if ctx.replay_norm:
            saved.append(norm_weight)
        if keep_up:
            saved.append(up_out)
        ctx.keep_low_rank = low_rank is not None
        if low_rank is not None:
            saved.append(low_rank)
        ctx.save_for_backward(*saved)
        return y.reshape(*x.shape[:-1], y.shape[-1])

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_output: torch.Tensor):
        saved = list(ctx.saved_tensors)
        kept_input, gate_out = saved[0], saved[1]
        adapters = saved[5:11]
        rest = saved[11:]
        if ctx.replay_norm:
            norm_weight = rest.pop(0)
            x2 = _as_rows(rmsnorm_bf16(kept_input, norm_weight, ctx.norm[0], ctx.norm[1]))
        else:
            x2 = kept_input
        up_saved = rest.pop(0) if ctx.keep_up else None
        low_rank = rest.pop(0) if ctx.keep_low_rank else None
        dy2 = _as_rows(grad_output)
        if dy2.dtype != torch.bfloat16:
            dy2 = dy2.to(torch.bfloat16)
        m = x2.shape[0]
        device = x2.device
        projs = [_proj_struct(ctx.descs[i], adapters[2 * i], adapters[2 * i + 1], ctx.scalings[i], ctx.shadows[i])
                 for i in range(3)]
        lib = _native.library()
        dx = torch.empty_like(x2)
        use_slots = all(slot is not None for slot in ctx.slots)
        if use_slots:
            grads = list(ctx.slots)
        else:
            grads = [torch.empty_like(t, dtype=torch.float32) for t in adapters]
        if m:
            pointers = (ctypes.c_void_p * 6)(*[g.data_ptr() for g in grads])
            nbytes = lib.molt_mlp_workspace_bytes(_native.OP_MLP_BWD, projs[0], projs[1], projs[2], m,
                                                  int(up_saved is not None))
            ws = _native.workspace(nbytes, device)
            with torch.cuda.device(device):
                _native.check(lib.molt_mlp_bwd_t(projs[0], projs[1], projs[2], x2.data_ptr(), gate_out.data_ptr(),
                                                 _native.ptr(up_saved), _native.ptr(low_rank), dy2.data_ptr(),
                                                 dx.data_ptr(), pointers, int(use_slots), m, ws.data_ptr(), ws.numel(),
                                                 _native.stream_handle(device)))
        elif not use_slots:
            for g in grads:
                g.zero_()
        out_grads = [None] * 6 if use_slots else grads
        return (dx.reshape(ctx.input_shape), None, None, None, out_grads[0], out_grads[1], None, out_grads[2],
                out_grads[3], None, out_grads[4], out_grads[5], None, None, None, None, None, None, None, None, None)


def gated_mlp_nf4_lora(
    x: torch.Tensor,
    gate_packed_weight: torch.Tensor, gate_lora_a: torch.Tensor, gate_lora_b: torch.Tensor,
    up_packed_weight: torch.Tensor, up_lora_a: torch.Tensor, up_lora_b: torch.Tensor,
    down_packed_weight: torch.Tensor, down_lora_a: torch.Tensor, down_lora_b: torch.Tensor,
    gate_quant_state: Any, up_quant_state: Any, down_quant_state: Any,
    gate_scaling: float, up_scaling: float, down_scaling: float,
    rematerialize_up: bool = True,
    source: Optional[torch.Tensor] = None,
    norm_weight: Optional[torch.Tensor] = None,
    norm_eps: float = 1e-6,
    norm_weight_offset: float = 0.0,
) -> torch.Tensor:
    """Whole gated MLP block on NF4 + LoRA projections.

    ``x`` is the (normalised) block input.  With ``source`` and ``norm_weight`` given, ``x`` must equal
    ``rmsnorm_bf16(source, norm_weight, norm_eps, norm_weight_offset)``; the node then keeps the residual
    ``source`` instead of ``x`` and re-materialises ``x`` in backward.
    """
    if (source is None) != (norm_weight is None):
        raise ValueError("source and norm_weight must be given together")
    return _GatedMLPNF4LoRA.apply(
        x, source, norm_weight, gate_packed_weight, gate_lora_a, gate_lora_b, up_packed_weight, up_lora_a, up_lora_b,
        down_packed_weight, down_lora_a, down_lora_b, gate_quant_state, up_quant_state, down_quant_state,
        gate_scaling, up_scaling, down_scaling, rematerialize_up, norm_eps, norm_weight_offset)


# --------------------------------------------------------------------------------------------------------
# Module patcher.
# --------------------------------------------------------------------------------------------------------

def _adapter_parts(module: torch.nn.Module):
    adapter = _adapter_of(module)
    if adapter is None:
        return None
    weight = module.base_layer.weight
    return (weight, module.lora_A[adapter].weight, module.lora_B[adapter].weight, weight.quant_state,
            float(module.scaling[adapter]))


def _host_mirror(module: torch.nn.Module, attr: str, like: torch.Tensor, what: str) -> torch.Tensor:
    host = getattr(module, attr, None)
    if host is None or host.shape != like.shape or host.dtype != like.dtype:
        if torch.cuda.is_current_stream_capturing():
            raise CapabilityError(f"gated activation {what} storage was not warmed up")
        host = torch.empty_like(like, device="cpu", pin_memory=True)
        setattr(module, attr, host)
    return host


def _asymmetric_mlp_forward(module: torch.nn.Module, x: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
    """Patched MLP forward with the reference's strict fallbacks (methods/gated_replay.py:482-537)."""
    if args or kwargs or not torch.is_grad_enabled() or x.dtype != torch.bfloat16 or not _bf16_autocast_active():
        return module._molt_original_forward(x, *args, **kwargs)
    up_parts = _adapter_parts(module.up_proj)
    down_parts = _adapter_parts(module.down_proj)
    if up_parts is None or down_parts is None:
        return module._molt_original_forward(x, *args, **kwargs)
    gate = module.gate_proj(x)
    up = module.up_proj(x)
    host_up = _host_mirror(module, "_molt_host_up", up, "host") if module._molt_offload_up else None
    host_gate = _host_mirror(module, "_molt_host_gate", gate, "gate") if module._molt_offload_gate else None
    return asymmetric_gated_nf4_lora(
        x, gate, up, up_parts[0], up_parts[1], up_parts[2], down_parts[0], down_parts[1], down_parts[2],
        up_parts[3], down_parts[3], up_parts[4], down_parts[4], module._molt_rematerialize_up,
        module._molt_offload_up, host_up, module._molt_offload_gate, host_gate,
    )


def enable_asymmetric_gated_replay(
    model: torch.nn.Module,
    *,
    rematerialize_up: bool = True,
    rematerialize_blocks: int | None = None,
    offload_blocks: int = 0,
    offload_gate_blocks: int = 0,
) -> int:
    """Patch every structurally compatible SiLU-gated NF4-LoRA MLP (reference :540-607).  The first
    ``rematerialize_blocks`` blocks replay ``up`` (all when None); ``offload_*`` select pinned-host offload."""
    if rematerialize_blocks is not None and rematerialize_blocks < 0:
        raise ValueError("rematerialize_blocks cannot be negative")
    if offload_blocks < 0:
        raise ValueError("offload_blocks cannot be negative")
    if offload_gate_blocks < 0:
        raise ValueError("offload_gate_blocks cannot be negative")
    if rematerialize_up and (offload_blocks or offload_gate_blocks):
        raise ValueError("up projection replay and offload are mutually exclusive")
    compatible = []
    for module in model.modules():
        if hasattr(module, "_molt_original_forward"):
            continue
        if not all(hasattr(module, name) for name in ("gate_proj", "up_proj", "down_proj", "act_fn")):
            continue
        if not all(is_lora_4bit_linear(getattr(module, name)) for name in ("gate_proj", "up_proj", "down_proj")):
            continue
        if type(module.act_fn).__name__ not in {"SiLU", "SiLUActivation"}:
            continue
        if _adapter_parts(module.up_proj) is None or _adapter_parts(module.down_proj) is None:
            continue
        compatible.append(module)
    if not compatible:
        raise CapabilityError("No compatible SiLU-gated PEFT NF4 MLP blocks were found")
    for count, what in ((rematerialize_blocks, "replay"), (offload_blocks, "offload"),
                        (offload_gate_blocks, "gate offload")):
        if count is not None and count > len(compatible):
            raise CapabilityError(
                f"requested {count} {what} blocks but only {len(compatible)} compatible blocks were found"
            )
    selected = len(compatible) if rematerialize_blocks is None else rematerialize_blocks
    for index, module in enumerate(compatible):
        module._molt_original_forward = module.forward
        module._molt_rematerialize_up = bool(rematerialize_up and index < selected)
        module._molt_offload_up = bool(index < offload_blocks)
        module._molt_offload_gate = bool(index < offload_gate_blocks)
        module.forward = MethodType(_asymmetric_mlp_forward, module)
    return len(compatible)
