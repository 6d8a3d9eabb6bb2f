"""Shared plumbing of the NF4 + LoRA linear: argument guards, native calls, and the autograd function
that every public entry point (``scheduled_nf4_lora``, ``StreamedLoRALinear``, the gated-MLP functions)
funnels into.  The arithmetic runs in ``libmolt_b200.so``.
"""
from __future__ import annotations

import ctypes
from typing import Any, Optional, Tuple

import torch

from molt_b200 import _native
from molt_b200.core.errors import CapabilityError

GRAD_SLOT = "_molt_grad_slot"  # attribute naming a preallocated fp32 gradient view (see data_parallel.GradArena)


def weight_desc(packed: torch.Tensor, quant_state: Any) -> _native.NF4Desc:
    """Descriptor for a weight, cached on the quant_state so the hot loop neither re-reads the codebook from
    the device nor synchronises (the reference caches its resolved scales the same way,
    reference methods/nf4_backward.py:151-163)."""
    from molt_b200.methods.quant_state import describe

    cached = getattr(quant_state, "_molt_desc", None)
    key = (packed.data_ptr(), quant_state.absmax.data_ptr())
    if cached is not None and cached[0] == key:
        return cached[1]
    desc = describe(packed, quant_state)
    try:
        quant_state._molt_desc = (key, desc)
    except AttributeError:  # frozen / slotted objects: just do not cache
        pass
    return desc


def weight_desc_for_tokens(packed: torch.Tensor, quant_state: Any, tokens: int) -> _native.NF4Desc:
    """Descriptor to use for a call with this many tokens.  A double-quantised absmax is resolved to fp32 once and the
    result cached on the state, as the reference does (methods/nf4_backward.py:145-164); the tensor-core kernels then
    read it directly instead of resolving it in front of every GEMM.  Up to 128 tokens the GEMV and few-token kernels
    read the 8-bit form themselves (fewer bytes), so those calls keep the state's own descriptor."""
    if tokens <= 128 or not getattr(quant_state, "nested", False):
        return weight_desc(packed, quant_state)
    cached = getattr(quant_state, "_molt_desc_resolved", None)
    key = (packed.data_ptr(), quant_state.absmax.data_ptr())
    if cached is not None and cached[0] == key:
        return cached[1]
    from molt_b200.methods.nf4_backward import resolved_nf4_scales
    from molt_b200.methods.quant_state import QuantState, describe

    fields = dict(absmax=resolved_nf4_scales(quant_state), shape=tuple(quant_state.shape),
                  nibble_order=getattr(quant_state, "nibble_order", "high-first"))
    if getattr(quant_state, "code", None) is not None:
        fields["code"] = quant_state.code
    plain = QuantState(**fields)
    desc = describe(packed, plain)
    try:
        quant_state._molt_desc_resolved = (key, desc, plain)   # `plain` keeps the resolved scales alive
    except AttributeError:
        pass
    return desc


def check_linear_inputs(x: torch.Tensor, packed: torch.Tensor, lora_a: torch.Tensor, lora_b: torch.Tensor,
                        who: str) -> None:
    """Guards of reference methods/nf4_lora.py:36-41, with the same error type and wording stem."""
    if x.device.type != "cuda" or packed.device.type != "cuda":
        raise CapabilityError(f"{who} requires CUDA tensors")
    if packed.requires_grad:
        raise CapabilityError(f"{who} requires frozen NF4 weights")
    if lora_a.dtype != torch.float32 or lora_b.dtype != torch.float32:
        raise CapabilityError(f"{who} requires FP32 adapter masters")
    if x.dtype != torch.bfloat16:
        raise CapabilityError(f"{who} requires bfloat16 activations")
    if lora_a.dim() != 2 or lora_b.dim() != 2 or lora_a.shape[0] != lora_b.shape[1]:
        raise ValueError("LoRA A must be [rank, in_features] and B [out_features, rank]")


SHADOW_SLOT = "_molt_lora_shadow"   # attribute of a LoRA A master: the adapter's LoraShadows (bf16 operands), if any


class LoraShadows:
    """bf16 operands of one adapter for the tensor-core kernels (``molt_lora_shadow``): ``a16 [rp, k]``, ``bs [n, 64]``
    = bf16(scaling * B), ``bt [rp, n]`` = its transpose, so that they are not rebuilt from the fp32 masters in front of every call
    (reference methods/lora_shadow.py:19-141).  Whoever changes the masters refreshes them afterwards (:class:`ShadowTable`);
    ``attach`` makes the fused ops use them (found through the A master)."""

    def __init__(self, lora_a: torch.Tensor, lora_b: torch.Tensor, scaling: float):
        rank, k = (int(v) for v in lora_a.shape)
        n = int(lora_b.shape[0])
        rp = (rank + 15) // 16 * 16
        dev = lora_a.device
        self.lora_a, self.lora_b, self.scaling, self.rank, self.n, self.k = lora_a, lora_b, float(scaling), rank, n, k
        self.a16 = torch.zeros((rp, k), dtype=torch.bfloat16, device=dev)
        self.bs = torch.zeros((n, 64), dtype=torch.bfloat16, device=dev)
        self.bt = torch.zeros((rp, n), dtype=torch.bfloat16, device=dev)
        self.struct = _native.LoraShadow(self.a16.data_ptr(), self.bs.data_ptr(), self.bt.data_ptr())

    def item(self) -> _native.LoraShadowItem:
        return _native.LoraShadowItem(self.lora_a.data_ptr(), self.lora_b.data_ptr(), self.scaling, self.rank, self.n,
                                      self.k, self.a16.data_ptr(), self.bs.data_ptr(), self.bt.data_ptr())

    def attach(self) -> None:
        setattr(self.lora_a, SHADOW_SLOT, self)

    def detach(self) -> None:
        if getattr(self.lora_a, SHADOW_SLOT, None) is self:
            delattr(self.lora_a, SHADOW_SLOT)


class ShadowTable:
    """The item list of many adapters in device memory, built once; ``refresh()`` rebuilds all their shadows in one
    launch on the current stream (call it after the optimizer step)."""

    def __init__(self, shadows):
        self.shadows = list(shadows)
        if not self.shadows:
            raise ValueError("no adapters")
        items = (_native.LoraShadowItem * len(self.shadows))(*[s.item() for s in self.shadows])
        raw = torch.frombuffer(bytearray(bytes(items)), dtype=torch.uint8)
        self.device = self.shadows[0].a16.device
        self.table = raw.to(self.device)
        self.max_n = max(s.n for s in self.shadows)
        self.max_k = max(s.k for s in self.shadows)

    def refresh(self) -> None:
        with torch.cuda.device(self.device):
            _native.check(_native.library().molt_lora_shadow_refresh(self.table.data_ptr(), len(self.shadows), self.max_n,
                                                                     self.max_k, _native.stream_handle(self.device)))


def _shadow_struct(shadow: Optional["LoraShadows"]):
    return ctypes.byref(shadow.struct) if shadow is not None else None


def linear_forward(desc: _native.NF4Desc, x2: torch.Tensor, lora_a: torch.Tensor, lora_b: torch.Tensor,
                   scaling: float, keep_low_rank: bool, path: int = _native.PATH_AUTO,
                   shadow: Optional[LoraShadows] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """y = x . deq(W)^T + s (x A^T) B^T for a 2-D bf16 x.  Returns (y, T) where T = x A^T padded to 64 columns."""
    n, k, m, rank = int(desc.n), int(desc.k), int(x2.shape[0]), int(lora_a.shape[0])
    if x2.shape[1] != k or lora_a.shape[1] != k or lora_b.shape[0] != n:
        raise ValueError("input width and adapter shapes must match the NF4 weight geometry")
    lib = _native.library()
    device = x2.device
    y = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    t = torch.empty((m, 64), dtype=torch.bfloat16, device=device) if keep_low_rank else None
    if m == 0:
        return y, t
    lora_a = lora_a.contiguous()
    lora_b = lora_b.contiguous()
    nbytes = lib.molt_workspace_bytes(_native.OP_LORA_FWD, m, n, k, rank)
    ws = _native.workspace(nbytes, device)
    with torch.cuda.device(device):
        _native.check(lib.molt_nf4_lora_fwd_prepared(
            ctypes.byref(desc), x2.data_ptr(), lora_a.data_ptr(), lora_b.data_ptr(), float(scaling), rank,
            _shadow_struct(shadow), y.data_ptr(), m, _native.ptr(t), ws.data_ptr(), ws.numel(), path,
            _native.stream_handle(device)))
    return y, t


def linear_backward(desc: _native.NF4Desc, x2: Optional[torch.Tensor], dy2: torch.Tensor, lora_a: torch.Tensor,
                    lora_b: torch.Tensor, scaling: float, t: Optional[torch.Tensor], need_dx: bool,
                    need_adapter_grads: bool, grad_a_out: Optional[torch.Tensor] = None,
                    grad_b_out: Optional[torch.Tensor] = None, path: int = _native.PATH_AUTO,
                    shadow: Optional[LoraShadows] = None):
    """dX, dA, dB of the linear.  When ``grad_a_out``/``grad_b_out`` are given the adapter gradients are
    accumulated into them in place (fp32) and returned as None."""
    n, k, m, rank = int(desc.n), int(desc.k), int(dy2.shape[0]), int(lora_a.shape[0])
    lib = _native.library()
    device = dy2.device
    dx = torch.empty((m, k), dtype=torch.bfloat16, device=device) if need_dx else None
    accumulate = 0
    da = db = None
    if need_adapter_grads:
        if grad_a_out is not None and grad_b_out is not None:
            da, db, accumulate = grad_a_out, grad_b_out, 1
        else:
            da = torch.empty((rank, k), dtype=torch.float32, device=device)
            db = torch.empty((n, rank), dtype=torch.float32, device=device)
    if m == 0:
        if need_adapter_grads and not accumulate:
            da.zero_()
            db.zero_()
        return dx, (None if accumulate else da), (None if accumulate else db)
    lora_a = lora_a.contiguous()
    lora_b = lora_b.contiguous()
    nbytes = lib.molt_workspace_bytes(_native.OP_LORA_BWD, m, n, k, rank)
    ws = _native.workspace(nbytes, device)
    with torch.cuda.device(device):
        _native.check(lib.molt_nf4_lora_bwd_prepared(
            ctypes.byref(desc), _native.ptr(x2), dy2.data_ptr(), lora_a.data_ptr(), lora_b.data_ptr(),
            float(scaling), rank, _shadow_struct(shadow), _native.ptr(dx), _native.ptr(da), _native.ptr(db), m,
            _native.ptr(t), accumulate, ws.data_ptr(), ws.numel(), path, _native.stream_handle(device)))
    if accumulate:
        return dx, None, None
    return dx, da, db


class NF4LoRAFunction(torch.autograd.Function):
    """Frozen NF4 base + LoRA with a hand-scheduled backward.

    Same contract as the reference's ``_ScheduledNF4LoRA`` (methods/nf4_lora.py:12-113) and ``_FrozenNF4LoRA``
    (streaming/engine.py:19-48): gradients for x, A and B only; dA/dB come back in fp32.  What is saved for
    backward is x, the packed weight, A, B and the small x A^T product -- never a dense weight.
    """

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, packed_weight: torch.Tensor, lora_a: torch.Tensor, lora_b: torch.Tensor,
                quant_state: Any, scaling: float, desc: Optional[_native.NF4Desc], who: str) -> torch.Tensor:
        check_linear_inputs(x, packed_weight, lora_a, lora_b, who)
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if desc is None:
            desc = weight_desc_for_tokens(packed_weight, quant_state, int(x2.shape[0]))
        needs_backward = any(ctx.needs_input_grad[i] for i in (0, 2, 3))
        ctx.shadow = getattr(lora_a, SHADOW_SLOT, None)
        y, t = linear_forward(desc, x2, lora_a, lora_b, float(scaling), keep_low_rank=needs_backward, shadow=ctx.shadow)
        ctx.desc = desc
        ctx.quant_state = quant_state
        ctx.scaling = float(scaling)
        ctx.input_shape = x.shape
        ctx.slots = (getattr(lora_a, GRAD_SLOT, None), getattr(lora_b, GRAD_SLOT, None))
        ctx.save_for_backward(x2, packed_weight, lora_a, lora_b, t if t is not None else x2.new_empty(0))
        return y.reshape(*x.shape[:-1], y.shape[-1])

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_output: torch.Tensor):
        x2, _packed, lora_a, lora_b, t = ctx.saved_tensors
        dy2 = grad_output.reshape(-1, grad_output.shape[-1])
        if dy2.dtype != torch.bfloat16:
            dy2 = dy2.to(torch.bfloat16)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        need_dx = ctx.needs_input_grad[0]
        need_grads = ctx.needs_input_grad[2] or ctx.needs_input_grad[3]
        slot_a, slot_b = ctx.slots
        dx, da, db = linear_backward(ctx.desc, x2, dy2, lora_a, lora_b, ctx.scaling, t if t.numel() else None,
                                     need_dx, need_grads, slot_a, slot_b, shadow=ctx.shadow)
        if dx is not None:
            dx = dx.reshape(ctx.input_shape)
        return dx, None, da, db, None, None, None, None
