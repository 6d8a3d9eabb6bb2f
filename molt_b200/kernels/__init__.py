from molt_b200.kernels.gated_activation import enable_fused_silu_mlp, fused_silu_multiply

__all__ = ["enable_fused_silu_mlp", "fused_silu_multiply"]
