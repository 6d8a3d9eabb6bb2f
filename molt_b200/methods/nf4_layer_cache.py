"""``dense_nf4_layer_cache``: temporarily hold dense bf16 copies of one decoder layer's NF4 bases.

Same context-manager contract as the reference's ``methods/nf4_layer_cache.py:22-66`` (yields the number of
patched projections; restores every ``base.forward`` in ``finally``; rejects trainable or biased bases).
The dense copies come from the CUDA dequantiser.  With the decode fused into the GEMMs the cache is not
needed for speed; it remains for callers that want a plain dense ``F.linear`` on the base path.
"""
from __future__ import annotations

import ctypes
from contextlib import contextmanager
from types import MethodType
from typing import Iterator

import torch
from torch.nn import functional as F

from molt_b200 import _native
from molt_b200.core.errors import CapabilityError
from molt_b200.methods._linear import weight_desc
from molt_b200.methods.nf4_lora import is_lora_4bit_linear


def dequantize_nf4(packed: torch.Tensor, quant_state, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Dense ``[n, k]`` weight from a packed NF4 weight and its quant_state (the role of
    ``bnb.functional.dequantize_4bit`` at reference methods/nf4_layer_cache.py:51)."""
    if packed.device.type != "cuda":
        raise CapabilityError("NF4 dequantisation requires CUDA tensors")
    if dtype not in (torch.bfloat16, torch.float32):
        raise CapabilityError("NF4 dequantisation produces bfloat16 or float32")
    desc = weight_desc(packed, quant_state)
    out = torch.empty((int(desc.n), int(desc.k)), dtype=dtype, device=packed.device)
    with torch.cuda.device(packed.device):
        _native.check(_native.library().molt_nf4_dequant(
            ctypes.byref(desc), out.data_ptr(),
            _native.DTYPE_BF16 if dtype == torch.bfloat16 else _native.DTYPE_F32,
            _native.stream_handle(packed.device)))
    return out


def _dense_forward(weight: torch.Tensor):
    def forward(_module: torch.nn.Module, inputs: torch.Tensor) -> torch.Tensor:
        return F.linear(inputs, weight, None)

    return forward


@contextmanager
def dense_nf4_layer_cache(layer: torch.nn.Module) -> Iterator[int]:
    patched: list[tuple[torch.nn.Module, object]] = []
    try:
        for module in layer.modules():
            if not is_lora_4bit_linear(module):
                continue
            base = module.base_layer
            weight = base.weight
            if weight.requires_grad or getattr(weight, "quant_state", None) is None:
                raise CapabilityError("layer cache requires frozen NF4 base weights")
            if base.bias is not None:
                raise CapabilityError("layer cache has not qualified biased NF4 projections")
            dense = dequantize_nf4(weight.data, weight.quant_state, torch.bfloat16)
            patched.append((base, base.forward))
            base.forward = MethodType(_dense_forward(dense), base)
        if not patched:
            raise CapabilityError("decoder layer contains no PEFT NF4 projections")
        yield len(patched)
    finally:
        for base, original in reversed(patched):
            base.forward = original
