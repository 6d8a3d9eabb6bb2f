"""Packed-NF4 input-gradient operators: ``grad_output @ deq(W)`` without a dense weight, optionally with the
rank-r LoRA term added.  Same functions as the reference's ``methods/nf4_backward.py`` (there: a Triton kernel).
"""
from __future__ import annotations

import ctypes
from typing import Any

import torch

from molt_b200 import _native
from molt_b200.core.errors import CapabilityError
from molt_b200.methods._linear import weight_desc


def resolved_nf4_scales(quant_state: Any) -> torch.Tensor:
    """fp32 absmax per block, un-nesting a double-quantised state once; the result is cached on the state
    (reference methods/nf4_backward.py:145-164)."""
    if getattr(quant_state, "quant_type", None) != "nf4":
        raise CapabilityError("packed backward requires NF4 quantization")
    if int(getattr(quant_state, "blocksize", 0)) != 64:
        raise CapabilityError("packed backward currently requires NF4 block size 64")
    cached = getattr(quant_state, "_molt_resolved_scales", None)
    if isinstance(cached, torch.Tensor) and cached.device == quant_state.absmax.device:
        return cached
    absmax = quant_state.absmax
    if not quant_state.nested:
        scales = absmax.float()
    else:
        if absmax.device.type != "cuda":
            raise CapabilityError("resolving nested NF4 scales requires CUDA tensors")
        scales = torch.empty(absmax.numel(), dtype=torch.float32, device=absmax.device)
        from molt_b200.methods.quant_state import describe

        desc = describe(None, quant_state)   # only the absmax fields of the descriptor are read here
        with torch.cuda.device(absmax.device):
            _native.check(_native.library().molt_nf4_resolve_absmax(
                ctypes.byref(desc), scales.data_ptr(), _native.stream_handle(absmax.device)))
    quant_state._molt_resolved_scales = scales
    return scales


def _flat_gradient(grad_output: torch.Tensor, quant_state: Any, who: str):
    if grad_output.device.type != "cuda":
        raise CapabilityError(f"{who} requires CUDA tensors")
    if grad_output.dtype != torch.bfloat16:
        raise CapabilityError(f"{who} currently requires BF16 gradients")
    shape = tuple(int(v) for v in quant_state.shape)
    if len(shape) != 2 or grad_output.shape[-1] != shape[0]:
        raise ValueError("gradient width must match the NF4 output dimension")
    flat = grad_output.reshape(-1, shape[0])
    if not flat.is_contiguous():
        flat = flat.contiguous()
    return flat, shape


def _scales_override(quant_state: Any, scales: torch.Tensor | None):
    """A caller-supplied fp32 scale vector replaces the state's absmax for this call."""
    if scales is None:
        return quant_state
    from molt_b200.methods.quant_state import QuantState

    return QuantState(absmax=scales.float().contiguous(), shape=tuple(quant_state.shape), code=quant_state.code,
                      blocksize=int(quant_state.blocksize),
                      nibble_order=getattr(quant_state, "nibble_order", "high-first"))


def packed_nf4_backward_input(
    grad_output: torch.Tensor,
    packed_weight: torch.Tensor,
    quant_state: Any,
    scales: torch.Tensor | None = None,
) -> torch.Tensor:
    """``grad_output @ dequant(weight)`` straight from the packed codes (reference :167-217)."""
    flat, (n, k) = _flat_gradient(grad_output, quant_state, "packed NF4 backward")
    state = _scales_override(quant_state, scales)
    desc = weight_desc(packed_weight, state)
    out = torch.empty((flat.shape[0], k), dtype=flat.dtype, device=flat.device)
    if flat.shape[0]:
        lib = _native.library()
        ws = _native.workspace(lib.molt_workspace_bytes(_native.OP_DX, flat.shape[0], n, k, 1), flat.device)
        with torch.cuda.device(flat.device):
            _native.check(lib.molt_nf4_dx(ctypes.byref(desc), flat.data_ptr(), None, None, 0, 0.0, 0, out.data_ptr(),
                                          flat.shape[0], ws.data_ptr(), ws.numel(), _native.PATH_AUTO,
                                          _native.stream_handle(flat.device)))
    return out.reshape(*grad_output.shape[:-1], k)


def packed_nf4_lora_backward_input(
    grad_output: torch.Tensor,
    packed_weight: torch.Tensor,
    quant_state: Any,
    lora_grad: torch.Tensor,
    lora_a: torch.Tensor,
    scaling: float,
    scales: torch.Tensor | None = None,
) -> torch.Tensor:
    """Base plus rank-r LoRA contribution to ``grad_input`` in one operator (reference :220-284).
    The base term is rounded to bf16 before the LoRA term is added, as the reference does (:127-136).
    Ranks up to 64 are accepted (the reference stops at 16)."""
    flat, (n, k) = _flat_gradient(grad_output, quant_state, "packed NF4-LoRA backward")
    if lora_grad.dtype != torch.bfloat16:
        raise CapabilityError("packed NF4-LoRA backward requires BF16 gradients")
    if lora_a.dtype not in {torch.bfloat16, torch.float32}:
        raise CapabilityError("LoRA A must use BF16 compute or an FP32 master")
    flat_lora = lora_grad.reshape(-1, lora_grad.shape[-1])
    if not flat_lora.is_contiguous():
        flat_lora = flat_lora.contiguous()
    if flat_lora.shape[0] != flat.shape[0]:
        raise ValueError("LoRA gradient rows must match the output gradient")
    if lora_a.ndim != 2 or flat_lora.shape[1] != lora_a.shape[0] or lora_a.shape[1] != k:
        raise ValueError("LoRA gradient and A matrix dimensions are incompatible")
    if lora_a.shape[0] > 64:
        raise CapabilityError("fused packed NF4-LoRA backward supports rank <= 64")
    lora_a = lora_a.contiguous()
    state = _scales_override(quant_state, scales)
    desc = weight_desc(packed_weight, state)
    out = torch.empty((flat.shape[0], k), dtype=flat.dtype, device=flat.device)
    if flat.shape[0]:
        lib = _native.library()
        rank = int(lora_a.shape[0])
        ws = _native.workspace(lib.molt_workspace_bytes(_native.OP_DX, flat.shape[0], n, k, rank), flat.device)
        a_dtype = _native.DTYPE_BF16 if lora_a.dtype == torch.bfloat16 else _native.DTYPE_F32
        with torch.cuda.device(flat.device):
            _native.check(lib.molt_nf4_dx(ctypes.byref(desc), flat.data_ptr(), flat_lora.data_ptr(), lora_a.data_ptr(),
                                          a_dtype, float(scaling), rank, out.data_ptr(), flat.shape[0], ws.data_ptr(),
                                          ws.numel(), _native.PATH_AUTO, _native.stream_handle(flat.device)))
    return out.reshape(*grad_output.shape[:-1], k)
