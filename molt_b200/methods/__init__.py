"""Autograd functions and patchers of the NF4 + LoRA hot path (mirrors ``molt_stream.methods``)."""
from molt_b200.methods.quant_state import NestedState, QuantState, quantize_nf4
from molt_b200.methods.nf4_lora import enable_scheduled_nf4_lora, scheduled_nf4_lora
from molt_b200.methods.nf4_backward import (
    packed_nf4_backward_input,
    packed_nf4_lora_backward_input,
    resolved_nf4_scales,
)
from molt_b200.methods.gated_replay import (
    asymmetric_gated_nf4_lora,
    enable_asymmetric_gated_replay,
    gated_mlp_nf4_lora,
)
from molt_b200.methods.nf4_layer_cache import dense_nf4_layer_cache

__all__ = [
    "NestedState", "QuantState", "quantize_nf4", "enable_scheduled_nf4_lora", "scheduled_nf4_lora",
    "packed_nf4_backward_input", "packed_nf4_lora_backward_input", "resolved_nf4_scales",
    "asymmetric_gated_nf4_lora", "enable_asymmetric_gated_replay", "gated_mlp_nf4_lora", "dense_nf4_layer_cache",
]
