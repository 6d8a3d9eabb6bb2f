"""Pieces of the reference's trainer that sit directly around the hot path: the static CUDA-graph micro-batch runner
(reference training/static_cuda_graph.py:139-308) and the import of bitsandbytes-format NF4 checkpoints."""
from molt_b200.training.checkpoint import (bnb_nf4_weight, export_bnb_nf4_weight, nf4_weight_prefixes,
                                           read_safetensors, write_safetensors)
from molt_b200.training.graph_microbatch import StaticCudaMicrobatch, TensorSignature

__all__ = ["StaticCudaMicrobatch", "TensorSignature", "read_safetensors", "write_safetensors", "bnb_nf4_weight",
           "export_bnb_nf4_weight", "nf4_weight_prefixes"]
