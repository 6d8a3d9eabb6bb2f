from molt_b200.streaming.nf4 import NF4_CODEBOOK, NF4DevicePayload, NF4Tensor
from molt_b200.streaming.engine import StreamedLayer, StreamedLoRALinear

__all__ = ["NF4_CODEBOOK", "NF4DevicePayload", "NF4Tensor", "StreamedLayer", "StreamedLoRALinear"]
