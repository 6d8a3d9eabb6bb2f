"""Fused ``silu(gate) * up`` with its backward; same names as the reference's ``kernels/gated_activation.py``.
Both directions are one vectorised, HBM-bound CUDA kernel each (``molt_swiglu_fwd`` / ``molt_swiglu_bwd``).
"""
from __future__ import annotations

from types import MethodType
from typing import Any

import torch

from molt_b200 import _native
from molt_b200.core.errors import CapabilityError

_DTYPES = {torch.bfloat16: _native.DTYPE_BF16, torch.float32: _native.DTYPE_F32}


def _check_device(tensor: torch.Tensor) -> int:
    if tensor.device.type != "cuda":
        raise CapabilityError("fused SiLU multiply requires CUDA tensors")
    if tensor.dtype not in _DTYPES:
        raise CapabilityError("fused SiLU multiply supports bfloat16 and float32 tensors")
    return _DTYPES[tensor.dtype]


def swiglu_forward(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    dtype = _check_device(gate)
    out = torch.empty_like(gate)
    if gate.numel():
        with torch.cuda.device(gate.device):
            _native.check(_native.library().molt_swiglu_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(),
                                                            gate.numel(), dtype, _native.stream_handle(gate.device)))
    return out


def swiglu_backward(grad_output: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, want_hidden: bool = False):
    """Returns (dgate, dup[, hidden]) -- ``hidden = silu(gate) * up`` is re-emitted on request for the replay path."""
    dtype = _check_device(gate)
    dgate = torch.empty_like(gate)
    dup = torch.empty_like(up)
    hidden = torch.empty_like(gate) if want_hidden else None
    if gate.numel():
        with torch.cuda.device(gate.device):
            _native.check(_native.library().molt_swiglu_bwd(
                grad_output.data_ptr(), gate.data_ptr(), up.data_ptr(), dgate.data_ptr(), dup.data_ptr(),
                _native.ptr(hidden), gate.numel(), dtype, _native.stream_handle(gate.device)))
    return (dgate, dup, hidden) if want_hidden else (dgate, dup)


class _FusedSiLUMultiply(torch.autograd.Function):
    """Saves contiguous gate and up, nothing else (reference kernels/gated_activation.py:54-93)."""

    @staticmethod
    def forward(ctx: Any, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        if gate.shape != up.shape or gate.dtype != up.dtype or gate.device != up.device:
            raise ValueError("gate and up tensors must have identical shape, dtype, and device")
        _check_device(gate)
        gate_c = gate.contiguous()
        up_c = up.contiguous()
        ctx.original_shape = gate.shape
        ctx.save_for_backward(gate_c, up_c)
        return swiglu_forward(gate_c, up_c)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_output: torch.Tensor):
        gate, up = ctx.saved_tensors
        grad = grad_output.contiguous()
        if grad.dtype != gate.dtype:
            grad = grad.to(gate.dtype)
        dgate, dup = swiglu_backward(grad, gate, up)
        return dgate.reshape(ctx.original_shape), dup.reshape(ctx.original_shape)


def fused_silu_multiply(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return _FusedSiLUMultiply.apply(gate, up)


def _fused_mlp_forward(module: torch.nn.Module, hidden: torch.Tensor) -> torch.Tensor:
    return module.down_proj(fused_silu_multiply(module.gate_proj(hidden), module.up_proj(hidden)))


def enable_fused_silu_mlp(model: torch.nn.Module) -> int:
    """Patch every gate/up/down MLP of a SiLU-gated decoder (reference kernels/gated_activation.py:106-130).
    The activation is read from ``model.config.hidden_activation`` / ``hidden_act`` as the reference does."""
    config = getattr(model, "config", None)
    activation = str(getattr(config, "hidden_activation", getattr(config, "hidden_act", ""))).lower()
    family = str(getattr(config, "model_type", type(model).__name__))
    if activation not in {"silu", "swish"}:
        raise CapabilityError(
            f"fused SiLU MLP requires silu/swish, but {family} uses {activation or '<unknown>'}"
        )
    patched = 0
    for module in model.modules():
        if hasattr(module, "_molt_original_mlp_forward"):
            continue
        if not all(hasattr(module, name) for name in ("gate_proj", "up_proj", "down_proj")):
            continue
        module._molt_original_mlp_forward = module.forward
        module.forward = MethodType(_fused_mlp_forward, module)
        patched += 1
    if patched == 0:
        raise CapabilityError(f"No compatible {family} gated MLP modules found")
    return patched
