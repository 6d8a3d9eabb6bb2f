"""NF4 tensors in MOLT's own format: two codes per byte with the even element in the low nibble,
one fp32 absmax per block.  Same classes, fields and method signatures as the reference's
``streaming/nf4.py``; dequantisation on the device is the CUDA kernel ``molt_nf4_dequant``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from molt_b200.core.errors import CapabilityError

# The 16 NormalFloat-4 levels of QLoRA (reference streaming/nf4.py:10-18).
NF4_CODEBOOK = torch.tensor(
    [
        -1.0, -0.6961928, -0.52507305, -0.3949175,
        -0.28444138, -0.18477343, -0.09105004, 0.0,
        0.0795803, 0.1609302, 0.2461123, 0.33791524,
        0.44070983, 0.562617, 0.72295684, 1.0,
    ],
    dtype=torch.float32,
)


@dataclass(frozen=True)
class NF4DevicePayload:
    """A packed weight staged on a device (reference streaming/nf4.py:21-35)."""

    packed: torch.Tensor
    scales: torch.Tensor
    shape: tuple[int, ...]
    block_size: int
    elements: int

    def describe(self):
        """C descriptor of this payload viewed as a ``[rows, columns]`` matrix."""
        from molt_b200 import _native

        columns = int(self.shape[-1]) if len(self.shape) else 1
        rows = self.elements // columns
        return _native.make_desc(self.packed, self.scales, rows, columns, self.block_size, _native.NIBBLE_LOW_FIRST,
                                 NF4_CODEBOOK.tolist())

    def dequantize(self, dtype: torch.dtype) -> torch.Tensor:
        """``codebook[code] * absmax`` in fp32, cast last (reference streaming/nf4.py:29-35); CUDA only."""
        from molt_b200 import _native

        if self.packed.device.type != "cuda":
            raise CapabilityError("NF4 dequantisation runs on a CUDA device; stage the payload first")
        if dtype not in (torch.bfloat16, torch.float32):
            raise CapabilityError("NF4 dequantisation produces bfloat16 or float32")
        out = torch.empty(self.shape, dtype=dtype, device=self.packed.device)
        desc = self.describe()
        with torch.cuda.device(self.packed.device):
            _native.check(_native.library().molt_nf4_dequant(
                desc, out.data_ptr(), _native.DTYPE_BF16 if dtype == torch.bfloat16 else _native.DTYPE_F32,
                _native.stream_handle(self.packed.device)))
        return out


@dataclass(frozen=True)
class NF4Tensor:
    """A packed weight in host memory (reference streaming/nf4.py:38-91)."""

    packed: torch.Tensor
    scales: torch.Tensor
    shape: tuple[int, ...]
    block_size: int
    elements: int

    @classmethod
    def quantize(cls, value: torch.Tensor, *, block_size: int = 64, pin_memory: bool = False) -> "NF4Tensor":
        """Blockwise absmax quantisation to the nearest NF4 level (reference streaming/nf4.py:46-68).

        Offline preparation: runs as torch ops on the tensor's current device, result lives on the host.
        """
        if value.numel() == 0 or block_size < 16 or block_size % 2:
            raise ValueError("invalid tensor or NF4 block size")
        flat = value.detach().float().reshape(-1)
        elements = flat.numel()
        padding = (-elements) % block_size
        if padding:
            flat = torch.nn.functional.pad(flat, (0, padding))
        blocks = flat.reshape(-1, block_size)
        scales = blocks.abs().amax(dim=1).clamp_min(torch.finfo(torch.float32).tiny)
        normalized = blocks / scales[:, None]
        levels = NF4_CODEBOOK.to(normalized.device)
        codes = torch.empty(normalized.shape, dtype=torch.uint8, device=normalized.device)
        rows_per_slice = max(1, (1 << 22) // (block_size * 16))
        for start in range(0, normalized.shape[0], rows_per_slice):
            part = normalized[start:start + rows_per_slice]
            codes[start:start + rows_per_slice] = (part[..., None] - levels).abs().argmin(dim=-1).to(torch.uint8)
        packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).reshape(-1).contiguous().cpu()
        scales = scales.contiguous().cpu()
        if pin_memory and torch.cuda.is_available():
            packed = packed.pin_memory()
            scales = scales.pin_memory()
        return cls(packed, scales, tuple(value.shape), block_size, elements)

    @property
    def storage_bytes(self) -> int:
        return self.packed.numel() * self.packed.element_size() + self.scales.numel() * 4

    def stage(self, device: torch.device | str, *, non_blocking: bool = False) -> NF4DevicePayload:
        target = torch.device(device)
        return NF4DevicePayload(
            self.packed.to(target, non_blocking=non_blocking),
            self.scales.to(target, non_blocking=non_blocking),
            self.shape, self.block_size, self.elements,
        )

    def dequantize(self, *, device: torch.device | str = "cuda", dtype: torch.dtype = torch.float32,
                   non_blocking: bool = False) -> torch.Tensor:
        return self.stage(torch.device(device), non_blocking=non_blocking).dequantize(dtype)
