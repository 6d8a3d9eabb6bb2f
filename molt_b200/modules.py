"""Modules that carry a frozen NF4 base plus a LoRA adapter in the attribute layout PEFT's ``Linear4bit``
uses (``base_layer.weight`` with a ``quant_state``, ``lora_A`` / ``lora_B`` module dicts, ``scaling``,
``active_adapters`` ...), so the ``enable_*`` patchers -- which the reference applies to PEFT modules
(reference methods/nf4_lora.py:168-220, methods/gated_replay.py:540-607) -- work on them unchanged.
PEFT and bitsandbytes themselves are not dependencies.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from molt_b200.methods.nf4_layer_cache import dequantize_nf4
from molt_b200.methods.nf4_lora import scheduled_nf4_lora
from molt_b200.methods.quant_state import QuantState, quantize_nf4


class PackedWeight(nn.Parameter):
    """Frozen uint8 parameter that carries its ``quant_state`` (as bitsandbytes' ``Params4bit`` does)."""

    quant_state: QuantState

    def __new__(cls, data: torch.Tensor, quant_state: QuantState):
        self = torch.Tensor._make_subclass(cls, data, False)
        self.quant_state = quant_state
        return self


class NF4BaseLinear(nn.Module):
    """The frozen 4-bit base: ``forward`` is the dense ``x @ deq(W)^T`` (used only on the unpatched route)."""

    def __init__(self, packed: torch.Tensor, quant_state: QuantState):
        super().__init__()
        self.weight = PackedWeight(packed, quant_state)
        self.bias = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        dense = dequantize_nf4(self.weight.data, self.weight.quant_state, torch.bfloat16)
        return torch.nn.functional.linear(x, dense.to(x.dtype))


class NF4LoRALinear(nn.Module):
    """LoRA-wrapped NF4 linear with PEFT's attribute layout.  The default ``forward`` already runs the fused
    path when the input is bf16 on CUDA; the unpatched route is dense base + eager LoRA."""

    def __init__(self, packed: torch.Tensor, quant_state: QuantState, rank: int, alpha: float,
                 adapter: str = "default"):
        super().__init__()
        out_features, in_features = (int(v) for v in quant_state.shape)
        self.in_features, self.out_features = in_features, out_features
        self.base_layer = NF4BaseLinear(packed, quant_state)
        device = packed.device
        self.lora_A = nn.ModuleDict({adapter: nn.Linear(in_features, rank, bias=False, device=device,
                                                        dtype=torch.float32)})
        self.lora_B = nn.ModuleDict({adapter: nn.Linear(rank, out_features, bias=False, device=device,
                                                        dtype=torch.float32)})
        nn.init.kaiming_uniform_(self.lora_A[adapter].weight, a=5**0.5)
        nn.init.zeros_(self.lora_B[adapter].weight)
        self.lora_dropout = nn.ModuleDict({adapter: nn.Identity()})
        self.scaling = {adapter: alpha / rank}
        self.active_adapters = [adapter]
        self.disable_adapters = False
        self.merged = False
        self.lora_variant: dict = {}
        self.use_dora = {adapter: False}

    @classmethod
    def from_dense(cls, weight: torch.Tensor, rank: int, alpha: float, blocksize: int = 64,
                   compress_statistics: bool = False, nibble_order: str = "high-first") -> "NF4LoRALinear":
        packed, state = quantize_nf4(weight, blocksize, compress_statistics, nibble_order)
        return cls(packed, state, rank, alpha)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        adapter = self.active_adapters[0]
        a, b = self.lora_A[adapter].weight, self.lora_B[adapter].weight
        if x.is_cuda and x.dtype == torch.bfloat16 and not self.disable_adapters:
            return scheduled_nf4_lora(x, self.base_layer.weight, a, b, self.base_layer.weight.quant_state,
                                      self.scaling[adapter])
        base = self.base_layer(x)
        if self.disable_adapters:
            return base
        linear = torch.nn.functional.linear
        return base + linear(linear(x, a.to(x.dtype)), b.to(x.dtype)) * self.scaling[adapter]


class GatedMLP(nn.Module):
    """``down_proj(act_fn(gate_proj(x)) * up_proj(x))`` over three :class:`NF4LoRALinear` (HF decoder layout)."""

    def __init__(self, gate_proj: NF4LoRALinear, up_proj: NF4LoRALinear, down_proj: NF4LoRALinear):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj
        self.act_fn = nn.SiLU()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))

    def fused(self, x: torch.Tensor, rematerialize_up: bool = True, source: Optional[torch.Tensor] = None,
              norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 1e-6) -> torch.Tensor:
        """The whole block as one autograd node (see ``gated_mlp_nf4_lora``)."""
        from molt_b200.methods.gated_replay import gated_mlp_nf4_lora

        g, u, d = self.gate_proj, self.up_proj, self.down_proj
        name = g.active_adapters[0]
        return gated_mlp_nf4_lora(
            x,
            g.base_layer.weight, g.lora_A[name].weight, g.lora_B[name].weight,
            u.base_layer.weight, u.lora_A[name].weight, u.lora_B[name].weight,
            d.base_layer.weight, d.lora_A[name].weight, d.lora_B[name].weight,
            g.base_layer.weight.quant_state, u.base_layer.weight.quant_state, d.base_layer.weight.quant_state,
            g.scaling[name], u.scaling[name], d.scaling[name], rematerialize_up, source, norm_weight, norm_eps)
