"""Import (and export) of NF4 weights in the layout bitsandbytes writes into a Hugging Face state dict, from
``.safetensors`` files, without either package.

The reference gets its quantised base model from ``AutoModelForCausalLM.from_pretrained(...,
quantization_config=BitsAndBytesConfig(load_in_4bit=True, bnb_4bit_quant_type="nf4",
bnb_4bit_use_double_quant=True))`` (reference training/qlora.py:332-347) and reads the resulting
``weight.quant_state`` by attribute (reference methods/nf4_backward.py:145-164).  A pre-quantised checkpoint
stores, per ``Linear4bit`` weight ``<prefix>.weight`` (bitsandbytes ``QuantState.as_dict(packed=True)``):

    <prefix>.weight                                   uint8 [n * k / 2, 1]   two codes per byte, even element in the HIGH nibble
    <prefix>.weight.absmax                            fp32 [blocks]  (uint8 [blocks] when double-quantised)
    <prefix>.weight.quant_map                         fp32 [16]      the NF4 code book
    <prefix>.weight.nested_absmax                     fp32 [ceil(blocks / 256)]       (double-quantised only)
    <prefix>.weight.nested_quant_map                  fp32 [256]                      (double-quantised only)
    <prefix>.weight.quant_state.bitsandbytes__nf4     uint8, UTF-8 JSON: quant_type, blocksize, dtype, shape and, when
                                                      double-quantised, nested_blocksize, nested_dtype, nested_offset

Parity of this layout is UNPINNED: bitsandbytes (pinned 0.50.2 by the reference's lock file) is not installed where
this package is built, so no file written by it has been read here; the tests round-trip files written by
``export_bnb_nf4_weight`` below, which follows the same published layout.

The ``.safetensors`` container itself is simple and documented: 8 bytes little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``, then the raw little-endian
buffers; ``read_safetensors`` / ``write_safetensors`` implement exactly that.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch

from molt_b200.core.errors import CapabilityError
from molt_b200.methods.quant_state import NestedState, QuantState

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {dtype: name for name, (dtype, _) in _DTYPES.items()}
_TORCH_NAMES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def read_safetensors(path, device: str | torch.device = "cpu", names: Optional[Iterable[str]] = None
                     ) -> Dict[str, torch.Tensor]:
    """All (or the named) tensors of one ``.safetensors`` file.  The file is mapped, each tensor copied out once."""
    path = Path(path)
    with open(path, "rb") as handle:
        raw = handle.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path.name}: not a safetensors file")
        (header_bytes,) = struct.unpack("<Q", raw)
        if header_bytes > 100 * 1024 * 1024:
            raise ValueError(f"{path.name}: header of {header_bytes} bytes")
        header = json.loads(handle.read(header_bytes).decode("utf-8"))
    data = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + header_bytes)
    wanted = None if names is None else set(names)
    out: Dict[str, torch.Tensor] = {}
    for name, entry in header.items():
        if name == "__metadata__" or (wanted is not None and name not in wanted):
            continue
        if entry["dtype"] not in _DTYPES:
            raise CapabilityError(f"{path.name}: tensor {name} has unsupported dtype {entry['dtype']}")
        dtype, width = _DTYPES[entry["dtype"]]
        begin, end = (int(v) for v in entry["data_offsets"])
        shape = tuple(int(v) for v in entry["shape"])
        count = 1
        for extent in shape:
            count *= extent
        if end - begin != count * width or end > data.shape[0]:
            raise ValueError(f"{path.name}: tensor {name} does not match its byte range")
        flat = torch.from_numpy(np.array(data[begin:end]))          # one copy out of the mapping
        tensor = flat.view(dtype).reshape(shape) if count else torch.empty(shape, dtype=dtype)
        out[name] = tensor.to(device)
    if wanted is not None and wanted - set(out):
        raise KeyError(f"{path.name}: missing tensors {sorted(wanted - set(out))}")
    return out


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    """Write tensors as one ``.safetensors`` file (sorted by name, buffers back to back, header padded to 8 bytes)."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs: List[bytes] = []
    offset = 0
    for name in sorted(tensors):
        tensor = tensors[name].detach().cpu().contiguous()
        if tensor.dtype not in _NAMES:
            raise CapabilityError(f"tensor {name} has unsupported dtype {tensor.dtype}")
        blob = tensor.reshape(-1).view(torch.uint8).numpy().tobytes() if tensor.numel() else b""
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape), "data_offsets": [offset, offset + len(blob)]}
        blobs.append(blob)
        offset += len(blob)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * ((-len(encoded)) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(encoded)))
        handle.write(encoded)
        for blob in blobs:
            handle.write(blob)


_STATE_SUFFIX = ".quant_state.bitsandbytes__nf4"


def nf4_weight_prefixes(tensors: Dict[str, torch.Tensor]) -> List[str]:
    """Names ``<prefix>.weight`` of every NF4-quantised weight in a state dict."""
    return sorted(name[: -len(_STATE_SUFFIX)] for name in tensors if name.endswith(_STATE_SUFFIX))


def bnb_nf4_weight(tensors: Dict[str, torch.Tensor], weight_name: str, device: str | torch.device = "cpu"
                   ) -> Tuple[torch.Tensor, QuantState]:
    """``(packed, quant_state)`` of one bitsandbytes-format NF4 weight, ready for ``scheduled_nf4_lora`` and friends.

    ``weight_name`` is the state-dict key of the packed bytes (``...q_proj.weight``, or
    ``...q_proj.base_layer.weight`` under PEFT).  Raises ``KeyError`` for missing pieces, ``CapabilityError`` for
    anything but NF4 with block size 64 (the reference's own guard, methods/nf4_backward.py:149-152)."""
    blob = tensors[weight_name + _STATE_SUFFIX]
    meta = json.loads(bytes(blob.detach().cpu().reshape(-1).tolist()).decode("utf-8"))
    if meta.get("quant_type") != "nf4" or int(meta.get("blocksize", 0)) != 64:
        raise CapabilityError("only NF4 weights with block size 64 are supported")
    shape = tuple(int(v) for v in meta["shape"])
    if len(shape) != 2:
        raise ValueError(f"{weight_name}: expected a 2-D weight, found shape {shape}")
    packed = tensors[weight_name]
    if packed.dtype != torch.uint8 or packed.numel() * 2 < shape[0] * shape[1]:
        raise ValueError(f"{weight_name}: packed bytes do not cover shape {shape}")
    absmax = tensors[weight_name + ".absmax"]
    blocks = -(-shape[0] * shape[1] // 64)
    if absmax.numel() != blocks:
        raise ValueError(f"{weight_name}: {absmax.numel()} absmax entries for {blocks} blocks")
    state = QuantState(absmax=absmax.reshape(-1).contiguous().to(device), shape=shape,
                       code=tensors[weight_name + ".quant_map"].float().reshape(-1).contiguous().to(device), blocksize=64,
                       dtype=_TORCH_NAMES.get(str(meta.get("dtype", "bfloat16")), torch.bfloat16), nibble_order="high-first")
    if state.code.numel() != 16:
        raise ValueError(f"{weight_name}: the code book has {state.code.numel()} entries")
    if "nested_blocksize" in meta:
        if absmax.dtype != torch.uint8:
            raise ValueError(f"{weight_name}: a double-quantised absmax must be uint8")
        nested_absmax = tensors[weight_name + ".nested_absmax"].float().reshape(-1).contiguous()
        nested_map = tensors[weight_name + ".nested_quant_map"].float().reshape(-1).contiguous()
        block2 = int(meta["nested_blocksize"])
        if nested_map.numel() != 256 or nested_absmax.numel() != -(-blocks // block2):
            raise ValueError(f"{weight_name}: second-level statistics do not match {blocks} blocks of {block2}")
        state.nested = True
        state.state2 = NestedState(nested_absmax.to(device), nested_map.to(device), block2)
        state.offset = float(meta["nested_offset"])
    elif absmax.dtype != torch.float32:
        state.absmax = state.absmax.float()
    return packed.reshape(-1, 1).contiguous().to(device), state


def export_bnb_nf4_weight(weight_name: str, packed: torch.Tensor, state: QuantState) -> Dict[str, torch.Tensor]:
    """The state-dict entries of one NF4 weight in the layout above (the inverse of :func:`bnb_nf4_weight`)."""
    if state.quant_type != "nf4" or state.blocksize != 64 or state.nibble_order != "high-first":
        raise CapabilityError("the bitsandbytes layout holds NF4, block size 64, even element in the high nibble")
    meta: Dict[str, object] = {"quant_type": "nf4", "blocksize": 64, "dtype": str(state.dtype).replace("torch.", ""),
                               "shape": [int(v) for v in state.shape]}
    out = {weight_name: packed.detach().cpu().reshape(-1, 1), weight_name + ".absmax": state.absmax.detach().cpu(),
           weight_name + ".quant_map": state.code.detach().cpu().float()}
    if state.nested:
        meta.update(nested_blocksize=int(state.state2.blocksize), nested_dtype="float32", nested_offset=float(state.offset))
        out[weight_name + ".nested_absmax"] = state.state2.absmax.detach().cpu().float()
        out[weight_name + ".nested_quant_map"] = state.state2.code.detach().cpu().float()
    out[weight_name + _STATE_SUFFIX] = torch.tensor(list(json.dumps(meta).encode("utf-8")), dtype=torch.uint8)
    return out
