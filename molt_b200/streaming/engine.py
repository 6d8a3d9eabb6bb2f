"""``StreamedLoRALinear``: a frozen NF4 base held in MOLT's own packed format with trainable LoRA
parameters, as in the reference's ``streaming/engine.py:51-80``.

The reference dequantises the whole weight to a dense tensor for every forward and again for every
backward (engine.py:36).  Here the packed payload is staged on the device once and the fused kernels
read it directly; ``forward`` still accepts the reference's ``staged_weight`` argument.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Union

import torch
from torch import nn

from molt_b200.methods._linear import NF4LoRAFunction
from molt_b200.streaming.nf4 import NF4DevicePayload, NF4Tensor


class _PayloadState:
    """Adapts an ``NF4DevicePayload`` to the attribute set the shared linear reads."""

    quant_type = "nf4"
    nested = False
    nibble_order = "low-first"

    def __init__(self, payload: NF4DevicePayload):
        from molt_b200.streaming.nf4 import NF4_CODEBOOK

        self.absmax = payload.scales
        self.blocksize = payload.block_size
        self.shape = payload.shape
        self.code = NF4_CODEBOOK


class StreamedLoRALinear(nn.Module):
    """Frozen NF4 base with device-resident trainable LoRA parameters (``lora_a``, ``lora_b``)."""

    def __init__(self, source: NF4Tensor, rank: int, alpha: float, device: torch.device):
        super().__init__()
        if len(source.shape) != 2:
            raise ValueError("streamed linear base must be a matrix")
        out_features, in_features = source.shape
        self.source = source
        self.scaling = alpha / rank
        self.lora_a = nn.Parameter(torch.empty(rank, in_features, device=device))
        self.lora_b = nn.Parameter(torch.zeros(out_features, rank, device=device))
        nn.init.kaiming_uniform_(self.lora_a, a=5**0.5)
        self._payload: Optional[NF4DevicePayload] = None
        self._state: Optional[_PayloadState] = None

    def payload(self, device: torch.device) -> NF4DevicePayload:
        """The packed weight on ``device`` (staged on first use and kept)."""
        if self._payload is None or self._payload.packed.device != device:
            self._payload = self.source.stage(device)
            self._state = _PayloadState(self._payload)
        return self._payload

    def forward(self, x: torch.Tensor, staged_weight: Union[torch.Tensor, NF4DevicePayload, None] = None
                ) -> torch.Tensor:
        """``x @ deq(W)^T + scaling * (x @ A^T) @ B^T``.

        ``staged_weight`` may be an ``NF4DevicePayload`` of this layer's source, or -- for call-site
        compatibility with the reference, which passes ``source.dequantize()`` -- a dense tensor, whose
        values are by construction those of the packed payload and are not read.
        """
        if isinstance(staged_weight, NF4DevicePayload):
            if self._payload is not staged_weight:
                self._payload = staged_weight
                self._state = _PayloadState(staged_weight)
        else:
            self.payload(x.device)
        return NF4LoRAFunction.apply(x, self._payload.packed, self.lora_a, self.lora_b, self._state, self.scaling,
                                     None, "streamed NF4-LoRA")


@dataclass
class StreamedLayer:
    """Residual SiLU wrapper around one streamed linear (reference streaming/engine.py:71-80)."""

    linear: StreamedLoRALinear

    @property
    def source(self) -> NF4Tensor:
        return self.linear.source

    def __call__(self, x: torch.Tensor, weight=None) -> torch.Tensor:
        return x + torch.nn.functional.silu(self.linear(x, weight))
