"""A minimal stand-in for the bitsandbytes ``QuantState`` the reference reads by attribute.

The reference touches ``quant_type``, ``blocksize``, ``shape``, ``absmax``, ``nested``, ``state2`` (``absmax``,
``code``, ``blocksize``), ``offset`` and ``code`` (reference methods/nf4_backward.py:147-163, :180, :197).
bitsandbytes is not a dependency of this package, so the same attribute set lives here, plus one
explicit field the third-party object leaves implicit: ``nibble_order``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Tuple

import torch

from molt_b200 import _native
from molt_b200.core.errors import CapabilityError
from molt_b200.streaming.nf4 import NF4_CODEBOOK

NIBBLE_ORDERS = {"low-first": _native.NIBBLE_LOW_FIRST, "high-first": _native.NIBBLE_HIGH_FIRST}


@dataclass
class NestedState:
    """Second-level quantisation of the absmax vector (``quant_state.state2``)."""

    absmax: torch.Tensor          # fp32 [ceil(blocks / blocksize)]
    code: torch.Tensor            # fp32 [256]
    blocksize: int = 256


@dataclass
class QuantState:
    absmax: torch.Tensor                      # fp32 [blocks] or uint8 [blocks] when nested
    shape: Tuple[int, int]
    code: torch.Tensor = field(default_factory=lambda: NF4_CODEBOOK.clone())
    blocksize: int = 64
    quant_type: str = "nf4"
    dtype: torch.dtype = torch.bfloat16
    nested: bool = False
    state2: Optional[NestedState] = None
    offset: Any = 0.0
    nibble_order: str = "high-first"          # bitsandbytes order (reference methods/nf4_backward.py:97-98)

    def to(self, device: torch.device | str) -> "QuantState":
        self.absmax = self.absmax.to(device)
        self.code = self.code.to(device)
        if self.state2 is not None:
            self.state2.absmax = self.state2.absmax.to(device)
            self.state2.code = self.state2.code.to(device)
        if isinstance(self.offset, torch.Tensor):
            self.offset = self.offset.to(device)
        return self


def _nearest_code(normalized: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """argmin_j |v - table[j]| with the first index winning ties, evaluated in slices to bound memory."""
    flat = normalized.reshape(-1)
    out = torch.empty(flat.shape, dtype=torch.uint8, device=flat.device)
    step = 1 << 20
    for start in range(0, flat.numel(), step):
        part = flat[start:start + step]
        out[start:start + step] = (part[:, None] - table[None, :]).abs().argmin(dim=1).to(torch.uint8)
    return out.reshape(normalized.shape)


def quantize_nf4(weight: torch.Tensor, blocksize: int = 64, compress_statistics: bool = False,
                 nibble_order: str = "high-first", code2: Optional[torch.Tensor] = None
                 ) -> Tuple[torch.Tensor, QuantState]:
    """Quantise a 2-D weight to packed NF4 on the weight's own device.

    Plays the role ``bnb.functional.quantize_4bit(w, blocksize=64, compress_statistics=..., quant_type="nf4")``
    plays in the reference's tests and benchmarks (reference tests/kernels/test_nf4_lora.py:24-26): returns
    ``(packed [n*k/2, 1] uint8, quant_state)``.  The arithmetic is the reference's own quantiser
    (streaming/nf4.py:46-68).  With ``compress_statistics`` the absmax vector is itself quantised to 8 bits in
    blocks of 256 around its mean; ``code2`` is that second table (default: 256 evenly spaced values on [-1, 1]).
    This is offline preparation and runs as ordinary torch ops.
    """
    if weight.dim() != 2 or weight.numel() == 0 or blocksize < 16 or blocksize % 2:
        raise ValueError("invalid tensor or NF4 block size")
    if nibble_order not in NIBBLE_ORDERS:
        raise ValueError(f"nibble_order must be one of {sorted(NIBBLE_ORDERS)}")
    device = weight.device
    flat = weight.detach().float().reshape(-1)
    pad = (-flat.numel()) % blocksize
    if pad:
        flat = torch.nn.functional.pad(flat, (0, pad))
    blocks = flat.reshape(-1, blocksize)
    absmax = blocks.abs().amax(dim=1).clamp_min(torch.finfo(torch.float32).tiny)
    codes = _nearest_code(blocks / absmax[:, None], NF4_CODEBOOK.to(device))
    if nibble_order == "low-first":
        packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    else:
        packed = (codes[:, 0::2] << 4) | codes[:, 1::2]
    packed = packed.reshape(-1, 1).contiguous()
    state = QuantState(absmax=absmax.contiguous(), shape=tuple(weight.shape), code=NF4_CODEBOOK.to(device),
                       blocksize=blocksize, dtype=weight.dtype, nibble_order=nibble_order)
    if compress_statistics:
        table = (torch.linspace(-1.0, 1.0, 256) if code2 is None else code2.float()).to(device)
        offset = absmax.mean()
        residual = absmax - offset
        pad2 = (-residual.numel()) % 256
        padded = torch.nn.functional.pad(residual, (0, pad2)) if pad2 else residual
        groups = padded.reshape(-1, 256)
        absmax2 = groups.abs().amax(dim=1).clamp_min(torch.finfo(torch.float32).tiny)
        codes2 = _nearest_code(groups / absmax2[:, None], table).reshape(-1)[: residual.numel()]
        state.absmax = codes2.contiguous()
        state.nested = True
        state.state2 = NestedState(absmax=absmax2.contiguous(), code=table.contiguous(), blocksize=256)
        state.offset = offset
    return packed, state


def _require_buffer(tensor: Any, what: str, dtype: torch.dtype, min_numel: int, device: torch.device) -> None:
    """The C side only sees raw pointers: every buffer must be what the declared shape says it is."""
    if not isinstance(tensor, torch.Tensor):
        raise ValueError(f"{what} must be a tensor")
    if tensor.dtype != dtype:
        raise CapabilityError(f"{what} must be {dtype}, got {tensor.dtype}")
    if tensor.device != device:
        raise ValueError(f"{what} must be on the same device as the packed weight ({tensor.device} != {device})")
    if not tensor.is_contiguous():
        raise ValueError(f"{what} must be contiguous")
    if tensor.numel() < min_numel:
        raise ValueError(f"{what} holds {tensor.numel()} elements but the declared weight shape needs {min_numel}")


def describe(packed: Optional[torch.Tensor], quant_state: Any) -> _native.NF4Desc:
    """Build the C descriptor for a ``(packed, quant_state)`` pair.  The returned struct borrows the tensors'
    memory; callers keep the tensors alive for the duration of the native call.

    Every buffer is checked against the declared weight shape (dtype, device, contiguity, element count) because
    the native side cannot: a state whose shape disagrees with its tensors would make the kernels read out of
    bounds.  ``packed=None`` builds a descriptor for calls that read only the absmax fields
    (``resolved_nf4_scales``); its packed pointer aliases the absmax and must not be dereferenced."""
    if getattr(quant_state, "quant_type", None) != "nf4":
        raise CapabilityError("the packed NF4 kernels require NF4 quantization")
    shape = tuple(int(v) for v in quant_state.shape)
    if len(shape) != 2 or shape[0] <= 0 or shape[1] <= 0:
        raise ValueError("the NF4 weight must be a non-empty matrix")
    order = getattr(quant_state, "nibble_order", "high-first")
    if order not in NIBBLE_ORDERS:
        raise ValueError(f"unknown nibble order {order!r}")
    blocksize = int(quant_state.blocksize)
    if blocksize < 16 or blocksize % 2:
        raise ValueError(f"invalid NF4 block size {blocksize}")
    absmax = quant_state.absmax
    if not isinstance(absmax, torch.Tensor):
        raise ValueError("absmax must be a tensor")
    device = absmax.device if packed is None else packed.device
    blocks = -(-(shape[0] * shape[1]) // blocksize)
    if packed is not None:
        _require_buffer(packed, "the packed weight", torch.uint8, -(-(shape[0] * shape[1]) // 2), device)
    nested = bool(getattr(quant_state, "nested", False))
    code = quant_state.code
    codebook = code.detach().float().cpu().tolist() if isinstance(code, torch.Tensor) else list(code)
    if len(codebook) != 16:
        raise CapabilityError("the NF4 codebook must have 16 entries")
    packed_arg = absmax if packed is None else packed
    if nested:
        state2 = quant_state.state2
        if state2 is None:
            raise ValueError("a nested quant state needs state2")
        block2 = int(state2.blocksize)
        if block2 <= 0:
            raise ValueError(f"invalid nested block size {block2}")
        if absmax.dtype != torch.uint8:
            raise CapabilityError("nested absmax must be stored as uint8 codes")
        _require_buffer(absmax, "the nested absmax codes", torch.uint8, blocks, device)
        if state2.absmax.dtype != torch.float32 or state2.code.dtype != torch.float32:
            raise CapabilityError("the nested absmax scale and its 256-entry table must be float32")
        _require_buffer(state2.absmax, "the second-level absmax", torch.float32, -(-blocks // block2), device)
        _require_buffer(state2.code, "the second-level table", torch.float32, 256, device)
        if state2.code.numel() != 256:
            raise ValueError("the second-level table must have exactly 256 entries")
        offset = quant_state.offset
        offset_value = float(offset.item()) if isinstance(offset, torch.Tensor) else float(offset)
        return _native.make_desc(packed_arg, absmax, shape[0], shape[1], blocksize, NIBBLE_ORDERS[order],
                                 codebook, absmax2=state2.absmax, code2=state2.code,
                                 offset=offset_value, block2=block2)
    if absmax.dtype != torch.float32:
        raise CapabilityError("absmax must be float32 (or uint8 codes with a nested state)")
    _require_buffer(absmax, "absmax", torch.float32, blocks, device)
    return _native.make_desc(packed_arg, absmax, shape[0], shape[1], blocksize, NIBBLE_ORDERS[order], codebook)
