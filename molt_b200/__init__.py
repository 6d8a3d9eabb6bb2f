"""molt_b200: the MOLT QLoRA hot path (frozen NF4 linear + LoRA, fused SwiGLU with replay, small-token
GEMV, data-parallel LoRA-gradient reduction) as hand-written sm_100a CUDA behind MOLT's own module and
autograd-function names.  Sub-packages mirror ``molt_stream``: ``streaming``, ``methods``, ``kernels``, ``core``.
"""

__version__ = "0.1.0"
