"""``scheduled_nf4_lora`` and its module patcher, same public surface as the reference's
``methods/nf4_lora.py`` -- with the bitsandbytes GEMM, the dense dequantised temporary and the five
cuBLAS calls replaced by the fused sm_100a kernels.
"""
from __future__ import annotations

from types import MethodType
from typing import Any

import torch

from molt_b200.core.errors import CapabilityError
from molt_b200.methods._linear import NF4LoRAFunction

_WHO = "scheduled NF4-LoRA"


def scheduled_nf4_lora(
    x: torch.Tensor,
    packed_weight: torch.Tensor,
    lora_a: torch.Tensor,
    lora_b: torch.Tensor,
    quant_state: Any,
    scaling: float,
    decoded_backward_weight: torch.Tensor | None = None,
) -> torch.Tensor:
    """``x @ deq(W)^T + scaling * (x @ A^T) @ B^T`` with gradients for x, A and B.

    Signature of reference methods/nf4_lora.py:116-133.  ``decoded_backward_weight`` is the reference's
    optional dense bf16 copy of the weight for its backward; the fused backward here never needs one, so
    the argument is only validated (same checks and error as reference :55-63) and otherwise unused.
    """
    if decoded_backward_weight is not None and (
        decoded_backward_weight.shape != (lora_b.shape[0], x.shape[-1])
        or decoded_backward_weight.device != x.device
        or decoded_backward_weight.dtype != x.dtype
    ):
        raise CapabilityError(
            "cached NF4 backward weight must match the decoded weight geometry, device, and compute dtype"
        )
    return NF4LoRAFunction.apply(x, packed_weight, lora_a, lora_b, quant_state, scaling, None, _WHO)


def _adapter_of(module: torch.nn.Module):
    """The single active, plain LoRA adapter of a PEFT-shaped module, or None (reference :145-156)."""
    if getattr(module, "disable_adapters", False) or getattr(module, "merged", False):
        return None
    active = list(getattr(module, "active_adapters", ()))
    if len(active) != 1:
        return None
    name = active[0]
    if name not in module.lora_A or name in getattr(module, "lora_variant", {}):
        return None
    if getattr(module, "use_dora", {}).get(name, False):
        return None
    if not isinstance(module.lora_dropout[name], torch.nn.Identity):
        return None
    if module.base_layer.bias is not None:
        return None
    return name


def _bf16_autocast_active() -> bool:
    return torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16


def _scheduled_forward(module: torch.nn.Module, x: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
    """Patched ``forward`` of a LoRA-wrapped 4-bit linear.  Anything outside the qualified envelope goes to the
    module's original forward, exactly as the reference does (methods/nf4_lora.py:136-165)."""
    if args or kwargs or x.dtype != torch.bfloat16 or not _bf16_autocast_active():
        return module._molt_original_forward(x, *args, **kwargs)
    adapter = _adapter_of(module)
    if adapter is None:
        return module._molt_original_forward(x, *args, **kwargs)
    weight = module.base_layer.weight
    return scheduled_nf4_lora(
        x, weight, module.lora_A[adapter].weight, module.lora_B[adapter].weight, weight.quant_state,
        float(module.scaling[adapter]), getattr(module, "_molt_decoded_backward_weight", None),
    )


def is_lora_4bit_linear(module: torch.nn.Module) -> bool:
    """PEFT's ``Linear4bit`` when PEFT is importable, else any module with the same structure:
    ``base_layer.weight.quant_state`` plus ``lora_A`` / ``lora_B`` / ``scaling`` / ``active_adapters``."""
    try:  # pragma: no cover - PEFT is optional
        from peft.tuners.lora.bnb import Linear4bit

        if isinstance(module, Linear4bit):
            return True
    except ImportError:
        pass
    base = getattr(module, "base_layer", None)
    weight = getattr(base, "weight", None)
    return (
        weight is not None
        and getattr(weight, "quant_state", None) is not None
        and all(hasattr(module, name) for name in ("lora_A", "lora_B", "scaling", "active_adapters"))
    )


def enable_scheduled_nf4_lora(
    model: torch.nn.Module,
    *,
    module_suffixes: tuple[str, ...] | None = None,
    require_narrow_output: bool = False,
    cache_backward_weights: bool = False,
) -> int:
    """Route the selected LoRA-wrapped NF4 projections through the fused path.

    Arguments and return value as reference methods/nf4_lora.py:168-220: ``module_suffixes`` restricts by
    module-name suffix, ``require_narrow_output`` keeps only projections with out_features < in_features,
    and the count of patched modules is returned (``CapabilityError`` when it would be zero).
    ``cache_backward_weights`` asks the reference to hold a dense bf16 weight per module; the fused backward
    decodes inside the GEMM, so the flag is accepted and nothing is cached.
    """
    del cache_backward_weights
    patched = 0
    for name, module in model.named_modules():
        if not is_lora_4bit_linear(module) or hasattr(module, "_molt_original_forward"):
            continue
        if module_suffixes is not None and not name.endswith(tuple(module_suffixes)):
            continue
        if require_narrow_output:
            narrow = (
                isinstance(getattr(module, "in_features", None), int)
                and isinstance(getattr(module, "out_features", None), int)
                and module.out_features < module.in_features
            )
            if not narrow:
                continue
        module._molt_original_forward = module.forward
        module.forward = MethodType(_scheduled_forward, module)
        patched += 1
    if patched == 0:
        wanted = "all modules" if module_suffixes is None else ", ".join(module_suffixes)
        raise CapabilityError(
            f"No compatible PEFT NF4-LoRA modules were found for {wanted}"
            + (" with grouped-query geometry" if require_narrow_output else "")
        )
    return patched
