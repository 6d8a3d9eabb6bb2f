"""Data-parallel training of the LoRA adapters: token batches are sharded over ranks, the frozen NF4
weights are replicated, and only the adapter gradients are exchanged.

The reference is single-GPU (its model is pinned to device 0, reference training/qlora.py:343), so this
file has no counterpart there; the invariant it maintains is "sum over ranks of the per-shard adapter
gradients == the full-batch adapter gradients".

``GradArena`` lays every trainable adapter parameter's gradient out in ONE flat fp32 buffer, in registration
order.  The backward kernels accumulate dA/dB straight into their slice (no per-parameter autograd
accumulation, no pack/unpack copy), and ``all_reduce`` hands contiguous, layer-ordered buckets of that same
buffer to the process group (NCCL over NVLink on GPUs, gloo in CPU tests) on a side stream so the exchange
overlaps the remaining backward.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from molt_b200.methods._linear import GRAD_SLOT


class GradArena:
    """One flat fp32 gradient buffer shared by a list of parameters."""

    def __init__(self, params: Iterable[torch.nn.Parameter], bucket_bytes: int = 32 << 20,
                 bucket_starts: Optional[Sequence[int]] = None):
        """``bucket_starts``: indices (into the trainable parameters, ascending, first one 0) at which a new bucket
        begins -- e.g. the first adapter of every decoder layer, so that a layer's gradients can be reduced as soon as
        its backward has run.  Without it buckets are cut by size."""
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("GradArena needs at least one trainable parameter")
        device = self.params[0].device
        offsets = []
        total = 0
        for p in self.params:
            if p.dtype != torch.float32 or p.device != device:
                raise ValueError("GradArena parameters must be float32 on one device")
            offsets.append(total)
            total += (p.numel() + 63) // 64 * 64  # 256-byte aligned slices
        self.flat = torch.zeros(total, dtype=torch.float32, device=device)
        self.offsets = offsets
        self.views: List[torch.Tensor] = []
        for p, off in zip(self.params, offsets):
            view = self.flat[off:off + p.numel()].view_as(p)
            self.views.append(view)
            p.grad = view
            setattr(p, GRAD_SLOT, view)
        self.buckets = self._make_buckets(bucket_bytes) if bucket_starts is None else self._buckets_from(bucket_starts)
        self._comm_stream: Optional[torch.cuda.Stream] = None

    def _buckets_from(self, starts: Sequence[int]) -> List[Tuple[int, int]]:
        """Buckets that begin at the given parameter indices, listed from the last to the first like the size-cut ones."""
        starts = sorted(set(int(i) for i in starts))
        if not starts or starts[0] != 0 or starts[-1] >= len(self.params):
            raise ValueError("bucket_starts must begin with 0 and stay inside the parameter list")
        bounds = self.offsets + [self.flat.numel()]
        edges = starts + [len(self.params)]
        return [(bounds[edges[i]], bounds[edges[i + 1]]) for i in range(len(starts) - 1, -1, -1)]

    def _make_buckets(self, bucket_bytes: int) -> List[Tuple[int, int]]:
        """Contiguous [begin, end) element ranges, cut at parameter boundaries, walked from the LAST
        parameter to the first (the order in which backward produces gradients)."""
        limit = max(1, bucket_bytes // 4)
        bounds = self.offsets + [self.flat.numel()]
        buckets: List[Tuple[int, int]] = []
        end = len(self.params)
        while end > 0:
            begin = end - 1
            while begin > 0 and bounds[end] - bounds[begin - 1] <= limit:
                begin -= 1
            buckets.append((bounds[begin], bounds[end]))
            end = begin
        return buckets

    def rebind(self) -> None:
        """Point every parameter's ``.grad`` at its arena slice again.  ``optimizer.zero_grad()`` with its default
        ``set_to_none=True`` drops ``.grad`` while the kernels keep accumulating into the arena; without this the
        optimiser would silently skip every adapter."""
        for p, view in zip(self.params, self.views):
            if p.grad is not view:
                p.grad = view

    def zero(self) -> None:
        """Clear the arena for the next step (use this, or ``zero_grad(set_to_none=False)``, between steps: the
        backward kernels ADD into the slices)."""
        self.flat.zero_()
        self.rebind()

    def bucket_of_param(self, index: int) -> int:
        off = self.offsets[index]
        for b, (lo, hi) in enumerate(self.buckets):
            if lo <= off < hi:
                return b
        raise IndexError(index)

    def all_reduce_bucket(self, bucket: int, group=None, async_stream: bool = True) -> None:
        """Sum one bucket over the group.  On CUDA the collective is enqueued on a side stream that first
        waits for the current stream (the producer of the gradients)."""
        lo, hi = self.buckets[bucket]
        chunk = self.flat[lo:hi]
        if self.flat.is_cuda and async_stream:
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream(device=self.flat.device)
            self._comm_stream.wait_stream(torch.cuda.current_stream(self.flat.device))
            with torch.cuda.stream(self._comm_stream):
                dist.all_reduce(chunk, op=dist.ReduceOp.SUM, group=group)
        else:
            dist.all_reduce(chunk, op=dist.ReduceOp.SUM, group=group)

    def all_reduce(self, group=None, average: bool = False) -> None:
        """Sum (or average) the whole arena over the group, bucket by bucket, then rejoin the main stream."""
        self.rebind()
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return
        for b in range(len(self.buckets)):
            self.all_reduce_bucket(b, group)
        self.wait()
        if average:
            self.flat.div_(dist.get_world_size(group))

    def wait(self) -> None:
        """Make the current stream wait for the collectives issued so far."""
        if self._comm_stream is not None:
            torch.cuda.current_stream(self.flat.device).wait_stream(self._comm_stream)


class ParamArena:
    """The parameters themselves in one flat fp32 buffer, laid out exactly like a :class:`GradArena` over the same list
    (same offsets), with the two AdamW moments beside it: one fused kernel (``molt_adamw_step``) then steps every
    adapter of the model.  Takes the place of the per-parameter optimizer the reference builds
    (reference training/qlora.py:218-243) and steps (:982-986)."""

    def __init__(self, grads: GradArena, lr: float = 1e-4, betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0):
        self.grads = grads
        self.flat = torch.empty_like(grads.flat)
        self.flat.zero_()
        for p, off in zip(grads.params, grads.offsets):
            view = self.flat[off:off + p.numel()].view_as(p)
            view.copy_(p.data)
            p.data = view                      # the module keeps its Parameter object; its storage is now the arena
        self.exp_avg = torch.zeros_like(self.flat)
        self.exp_avg_sq = torch.zeros_like(self.flat)
        self.lr, self.betas, self.eps, self.weight_decay = float(lr), betas, float(eps), float(weight_decay)
        self.steps = 0

    def step(self, grad_scale: float = 1.0) -> None:
        """One AdamW step over every parameter, on the current stream."""
        import ctypes  # noqa: F401  (the native binding passes raw pointers)

        from molt_b200 import _native

        self.steps += 1
        flat = self.flat
        with torch.cuda.device(flat.device):
            _native.check(_native.library().molt_adamw_step(
                flat.data_ptr(), self.grads.flat.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                flat.numel(), self.lr, self.betas[0], self.betas[1], self.eps, self.weight_decay, self.steps,
                float(grad_scale), _native.stream_handle(flat.device)))


class RankLeftError(RuntimeError):
    """A peer announced that it left, or stopped announcing steps, before a collective was launched."""


class StepGuard:
    """Host-side watchdog in front of the collectives of a step.

    Every rank announces each step it is about to run through the process group's key-value store, and checks that
    every peer has announced the same step before it launches kernels or collectives for it.  A rank that leaves
    (between steps, with nothing in flight) says so; a rank that died silently simply stops announcing.  Either way
    the survivors get :class:`RankLeftError` within ``timeout`` seconds on the host instead of a collective that
    never completes.  (The reference is single-GPU and has no counterpart.)"""

    def __init__(self, store=None, rank: Optional[int] = None, world_size: Optional[int] = None, timeout: float = 30.0,
                 poll: float = 0.02, prefix: str = "molt_step_guard"):
        if store is None:
            from torch.distributed import distributed_c10d

            store = distributed_c10d._get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else int(rank)
        self.world = dist.get_world_size() if world_size is None else int(world_size)
        self.timeout, self.poll, self.prefix = float(timeout), float(poll), prefix

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def announce(self, step: int) -> None:
        self.store.set(self._key(self.rank), str(int(step)))

    def leave(self) -> None:
        """Tell the peers that this rank is gone; call it only between steps."""
        self.store.set(self._key(self.rank), "left")

    def check(self, step: int) -> None:
        """Announce ``step`` and wait until every peer has announced it too."""
        import time

        self.announce(step)
        deadline = time.monotonic() + self.timeout
        pending = [r for r in range(self.world) if r != self.rank]
        while pending:
            still = []
            for r in pending:
                value = None
                try:
                    if self.store.check([self._key(r)]):
                        value = self.store.get(self._key(r)).decode()
                except Exception as exc:  # the store itself is gone (its host rank died)
                    raise RankLeftError(f"lost the rendezvous store while waiting for rank {r}: {exc}") from exc
                if value == "left":
                    raise RankLeftError(f"rank {r} left before step {step}")
                if value is None or int(value) < step:
                    still.append(r)
            pending = still
            if pending:
                if time.monotonic() > deadline:
                    raise RankLeftError(f"ranks {pending} did not reach step {step} within {self.timeout:.1f} s")
                time.sleep(self.poll)


def shard_rows(total_rows: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Row range [begin, end) of ``rank`` when ``total_rows`` tokens are split as evenly as possible."""
    base, extra = divmod(total_rows, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def lora_parameters(model: torch.nn.Module) -> List[torch.nn.Parameter]:
    """Trainable parameters in module registration order (frozen NF4 bases are skipped)."""
    return [p for p in model.parameters() if p.requires_grad]


def check_replicas_equal(tensors: Sequence[torch.Tensor], group=None) -> bool:
    """True when every rank holds bit-identical copies of ``tensors`` (used after an optimiser step)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return True
    ok = True
    for t in tensors:
        lo = t.detach().clone()
        hi = t.detach().clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
        ok = ok and bool(torch.equal(lo, hi))
    return ok
