"""ctypes binding of ``libmolt_b200.so`` (the C ABI declared in ``include/molt_b200.h``).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
Tensors are handed over as raw device pointers together with the current CUDA stream; outputs and
scratch are allocated here with ``torch.empty`` (stream-ordered, CUDA-graph friendly) because the
library itself never allocates.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path
from typing import Optional, Sequence

import torch

from molt_b200.core.errors import CapabilityError

LIBRARY_PATH = Path(__file__).resolve().parent / "libmolt_b200.so"

OK, E_VALUE, E_CAPABILITY, E_RUNTIME, E_TIMEOUT = 0, 1, 2, 3, 4
ABSMAX_F32, ABSMAX_NESTED = 0, 1
NIBBLE_LOW_FIRST, NIBBLE_HIGH_FIRST = 0, 1
DTYPE_BF16, DTYPE_F32 = 0, 1
PATH_AUTO, PATH_GENERAL, PATH_TCGEN05, PATH_GEMV, PATH_FEW_TOKENS = 0, 1, 2, 3, 4
PATH_EXACT_DECODE = 0x1000
PATH_NO_SPLIT, PATH_FORCE_SPLIT, PATH_TALL_TILES, PATH_SHORT_TILES = 0x100, 0x200, 0x400, 0x800   # flags OR-ed onto a path
OPT_WAIT_LIMIT_US, OPT_WITHHOLD_BLOCKS = 1, 2
OP_LORA_FWD, OP_LORA_BWD, OP_DX, OP_MLP_FWD, OP_MLP_BWD = 1, 2, 3, 4, 5

EXPORTS = (
    "molt_version", "molt_last_error", "molt_launch_count", "molt_set_option", "molt_read_status", "molt_nf4_dequant", "molt_nf4_resolve_absmax",
    "molt_workspace_bytes", "molt_nf4_lora_fwd", "molt_nf4_lora_fwd_static", "molt_nf4_lora_bwd", "molt_nf4_dx", "molt_nf4_gemv",
    "molt_swiglu_fwd", "molt_swiglu_bwd", "molt_rmsnorm_fwd", "molt_rmsnorm_bwd", "molt_add_rmsnorm_fwd",
    "molt_add_rmsnorm_bwd", "molt_rope", "molt_adamw_step", "molt_dense_gemm", "molt_nf4_lora_fwd_prepared",
    "molt_nf4_lora_bwd_prepared", "molt_lora_shadow_refresh",
    "molt_dense_gemm_workspace_bytes", "molt_ce_softmax_grad", "molt_mlp_workspace_bytes", "molt_mlp_fwd",
    "molt_mlp_bwd", "molt_mlp_fwd_t", "molt_mlp_bwd_t",
)


class NF4Desc(ctypes.Structure):
    """Mirror of ``molt_nf4_desc``."""

    _fields_ = [
        ("packed", ctypes.c_void_p),
        ("absmax", ctypes.c_void_p),
        ("absmax2", ctypes.c_void_p),
        ("code2", ctypes.c_void_p),
        ("offset", ctypes.c_float),
        ("absmax_kind", ctypes.c_int32),
        ("block2", ctypes.c_int32),
        ("blocksize", ctypes.c_int32),
        ("nibble_order", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("n", ctypes.c_int64),
        ("k", ctypes.c_int64),
        ("codebook", ctypes.c_float * 16),
    ]


class LoraShadow(ctypes.Structure):
    """Mirror of ``molt_lora_shadow``: bf16 operands of one adapter kept up to date by the caller."""

    _fields_ = [("a16", ctypes.c_void_p), ("bs", ctypes.c_void_p), ("bt", ctypes.c_void_p)]


class LoraShadowItem(ctypes.Structure):
    """Mirror of ``molt_lora_shadow_item``."""

    _fields_ = [
        ("lora_a", ctypes.c_void_p),
        ("lora_b", ctypes.c_void_p),
        ("scaling", ctypes.c_float),
        ("rank", ctypes.c_int32),
        ("n", ctypes.c_int64),
        ("k", ctypes.c_int64),
        ("a16", ctypes.c_void_p),
        ("bs", ctypes.c_void_p),
        ("bt", ctypes.c_void_p),
    ]


class LoraProj(ctypes.Structure):
    """Mirror of ``molt_lora_proj``."""

    _fields_ = [
        ("w", ctypes.POINTER(NF4Desc)),
        ("lora_a", ctypes.c_void_p),
        ("lora_b", ctypes.c_void_p),
        ("scaling", ctypes.c_float),
        ("rank", ctypes.c_int32),
        ("shadow", ctypes.POINTER(LoraShadow)),
    ]


_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


def _declare(lib: ctypes.CDLL) -> None:
    vp, i32, i64, f32, sz, up = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t,
                                 ctypes.c_size_t)
    desc = ctypes.POINTER(NF4Desc)
    proj = ctypes.POINTER(LoraProj)
    lib.molt_version.restype = i32
    lib.molt_version.argtypes = []
    lib.molt_last_error.restype = ctypes.c_char_p
    lib.molt_last_error.argtypes = []
    lib.molt_launch_count.restype = ctypes.c_uint64
    lib.molt_launch_count.argtypes = []
    lib.molt_set_option.restype = i32
    lib.molt_set_option.argtypes = [i32, i64]
    lib.molt_read_status.restype = i32
    lib.molt_read_status.argtypes = [up, ctypes.POINTER(ctypes.c_int32)]
    lib.molt_nf4_dequant.restype = i32
    lib.molt_nf4_dequant.argtypes = [desc, vp, i32, up]
    lib.molt_nf4_resolve_absmax.restype = i32
    lib.molt_nf4_resolve_absmax.argtypes = [desc, vp, up]
    lib.molt_workspace_bytes.restype = sz
    lib.molt_workspace_bytes.argtypes = [i32, i64, i64, i64, i32]
    lib.molt_nf4_lora_fwd.restype = i32
    lib.molt_nf4_lora_fwd.argtypes = [desc, vp, vp, vp, f32, i32, vp, i64, vp, vp, sz, i32, up]
    shadow = ctypes.POINTER(LoraShadow)
    lib.molt_nf4_lora_fwd_prepared.restype = i32
    lib.molt_nf4_lora_fwd_prepared.argtypes = [desc, vp, vp, vp, f32, i32, shadow, vp, i64, vp, vp, sz, i32, up]
    lib.molt_nf4_lora_bwd_prepared.restype = i32
    lib.molt_nf4_lora_bwd_prepared.argtypes = [desc, vp, vp, vp, vp, f32, i32, shadow, vp, vp, vp, i64, vp, i32, vp, sz,
                                               i32, up]
    lib.molt_lora_shadow_refresh.restype = i32
    lib.molt_lora_shadow_refresh.argtypes = [vp, i32, i64, i64, up]
    lib.molt_nf4_lora_fwd_static.restype = i32
    lib.molt_nf4_lora_fwd_static.argtypes = [desc, vp, vp, vp, f32, i32, vp, i64, i32, up]
    lib.molt_nf4_lora_bwd.restype = i32
    lib.molt_nf4_lora_bwd.argtypes = [desc, vp, vp, vp, vp, f32, i32, vp, vp, vp, i64, vp, i32, vp, sz, i32, up]
    lib.molt_nf4_dx.restype = i32
    lib.molt_nf4_dx.argtypes = [desc, vp, vp, vp, i32, f32, i32, vp, i64, vp, sz, i32, up]
    lib.molt_nf4_gemv.restype = i32
    lib.molt_nf4_gemv.argtypes = [desc, vp, vp, vp, f32, i32, vp, i64, vp, sz, up]
    lib.molt_swiglu_fwd.restype = i32
    lib.molt_swiglu_fwd.argtypes = [vp, vp, vp, i64, i32, up]
    lib.molt_swiglu_bwd.restype = i32
    lib.molt_swiglu_bwd.argtypes = [vp, vp, vp, vp, vp, vp, i64, i32, up]
    lib.molt_rmsnorm_fwd.restype = i32
    lib.molt_rmsnorm_fwd.argtypes = [vp, vp, i32, f32, f32, vp, i64, i64, up]
    lib.molt_rmsnorm_bwd.restype = i32
    lib.molt_rmsnorm_bwd.argtypes = [vp, vp, vp, i32, f32, f32, vp, i64, i64, up]
    lib.molt_add_rmsnorm_fwd.restype = i32
    lib.molt_add_rmsnorm_fwd.argtypes = [vp, vp, vp, i32, f32, f32, vp, vp, i64, i64, up]
    lib.molt_add_rmsnorm_bwd.restype = i32
    lib.molt_add_rmsnorm_bwd.argtypes = [vp, vp, vp, vp, i32, f32, f32, vp, i64, i64, up]
    lib.molt_rope.restype = i32
    lib.molt_rope.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, i32, i32, up]
    lib.molt_adamw_step.restype = i32
    lib.molt_adamw_step.argtypes = [vp, vp, vp, vp, i64, f32, f32, f32, f32, f32, i64, f32, up]
    lib.molt_dense_gemm_workspace_bytes.restype = sz
    lib.molt_dense_gemm_workspace_bytes.argtypes = []
    lib.molt_dense_gemm.restype = i32
    lib.molt_dense_gemm.argtypes = [vp, i64, i64, vp, vp, i64, i32, vp, sz, i32, up]
    lib.molt_ce_softmax_grad.restype = i32
    lib.molt_ce_softmax_grad.argtypes = [vp, vp, vp, i64, i64, f32, up]
    lib.molt_mlp_workspace_bytes.restype = sz
    lib.molt_mlp_workspace_bytes.argtypes = [i32, proj, proj, proj, i64, i32]
    lib.molt_mlp_fwd.restype = i32
    lib.molt_mlp_fwd.argtypes = [proj, proj, proj, vp, vp, vp, vp, i64, vp, sz, up]
    lib.molt_mlp_bwd.restype = i32
    lib.molt_mlp_bwd.argtypes = [proj, proj, proj, vp, vp, vp, vp, vp, ctypes.POINTER(vp), i32, i64, vp, sz, up]
    lib.molt_mlp_fwd_t.restype = i32
    lib.molt_mlp_fwd_t.argtypes = [proj, proj, proj, vp, vp, vp, vp, vp, i64, vp, sz, up]
    lib.molt_mlp_bwd_t.restype = i32
    lib.molt_mlp_bwd_t.argtypes = [proj, proj, proj, vp, vp, vp, vp, vp, vp, ctypes.POINTER(vp), i32, i64, vp, sz, up]


def library() -> ctypes.CDLL:
    """Load the shared library once. Raises ``CapabilityError`` when it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not LIBRARY_PATH.exists():
                    raise CapabilityError(
                        f"{LIBRARY_PATH.name} is missing; build it with `python -m molt_b200.build` "
                        "(there is no fallback implementation)"
                    )
                lib = ctypes.CDLL(str(LIBRARY_PATH))
                _declare(lib)
                _lib = lib
    return _lib


def check(code: int) -> None:
    """Map a C status to the exception type the reference raises for the same condition."""
    if code == OK:
        return
    message = library().molt_last_error().decode("utf-8", "replace")
    if code == E_VALUE:
        raise ValueError(message)
    if code == E_CAPABILITY:
        raise CapabilityError(message)
    raise RuntimeError(f"molt_b200 native call failed ({code}): {message}")


def stream_handle(device: Optional[torch.device] = None) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def read_status(device: Optional[torch.device] = None) -> int:
    """Device status word of the bounded waits (0 = clean). Synchronises the current stream."""
    out = ctypes.c_int32(0)
    check(library().molt_read_status(stream_handle(device), ctypes.byref(out)))
    return int(out.value)


def set_option(option: int, value: int) -> None:
    """Process-wide library option (``OPT_*``)."""
    check(library().molt_set_option(int(option), int(value)))


def workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def make_desc(packed: torch.Tensor, absmax: torch.Tensor, n: int, k: int, blocksize: int, nibble_order: int,
              codebook: Sequence[float], absmax2: Optional[torch.Tensor] = None,
              code2: Optional[torch.Tensor] = None, offset: float = 0.0, block2: int = 256) -> NF4Desc:
    desc = NF4Desc()
    desc.packed = packed.data_ptr()
    desc.absmax = absmax.data_ptr()
    nested = absmax.dtype == torch.uint8
    desc.absmax2 = absmax2.data_ptr() if nested else None
    desc.code2 = code2.data_ptr() if nested else None
    desc.offset = float(offset)
    desc.absmax_kind = ABSMAX_NESTED if nested else ABSMAX_F32
    desc.block2 = int(block2)
    desc.blocksize = int(blocksize)
    desc.nibble_order = int(nibble_order)
    desc.n = int(n)
    desc.k = int(k)
    for i in range(16):
        desc.codebook[i] = float(codebook[i])
    return desc
