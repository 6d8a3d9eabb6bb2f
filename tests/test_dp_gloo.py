"""Data-parallel bookkeeping with two CPU ranks over gloo: tokens are sharded, each rank fills its gradient
arena with the adapter gradients of its own shard (computed by the CPU oracle), the arena is all-reduced
bucket by bucket, and the result must equal the full-batch gradients."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import molt_oracle as oracle
from molt_b200.data_parallel import GradArena, check_replicas_equal, shard_rows


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        layers = []
        for layer in range(3):
            n, k, r = 96 + 32 * layer, 64, 8
            w, a, b, x, dy = oracle.seeded_linear_case(n, k, 40, r, seed=100 + layer)
            layers.append((oracle.nf4_dequantize(oracle.nf4_quantize(w, 64)), a, b, x, dy))
        params = []
        for _, a, b, _, _ in layers:
            params += [torch.nn.Parameter(a.clone()), torch.nn.Parameter(b.clone())]
        arena = GradArena(params, bucket_bytes=6000)
        assert len(arena.buckets) > 1
        lo, hi = shard_rows(40, rank, world)
        for i, (w, a, b, x, dy) in enumerate(layers):
            _, da, db = oracle.nf4_lora_backward(x[lo:hi], dy[lo:hi], w, a, b, 2.0)
            arena.views[2 * i].add_(da)
            arena.views[2 * i + 1].add_(db)
        arena.all_reduce()
        worst = 0.0
        for i, (w, a, b, x, dy) in enumerate(layers):
            _, da, db = oracle.nf4_lora_backward(x, dy, w, a, b, 2.0)
            worst = max(worst, oracle.rel_frobenius(params[2 * i].grad, da), oracle.rel_frobenius(params[2 * i + 1].grad, db))
        same = check_replicas_equal([arena.flat])
        results[rank] = (worst, same)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_sharded_gradients_sum_to_full_batch():
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(150)
        assert p.exitcode == 0
    for rank in range(world):
        worst, same = results[rank]
        assert worst < 1e-5   # fp32 reduction-order tolerance
        assert same


def _leaver_worker(rank: int, world: int, port: int, results):
    """Three ranks train in lock step behind a StepGuard; rank 2 leaves between step 1 and step 2 (nothing in flight),
    and the others must get RankLeftError on the host before they launch step 2's collective."""
    import time

    from molt_b200.data_parallel import RankLeftError, StepGuard

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    outcome = "none"
    try:
        guard = StepGuard(timeout=20.0)
        grads = torch.nn.Parameter(torch.zeros(64))
        arena = GradArena([grads], bucket_starts=[0])
        for step in range(3):
            if rank == 2 and step == 2:
                guard.leave()                      # between steps: no kernel or collective of this rank is in flight
                outcome = "left"
                break
            begin = time.monotonic()
            try:
                guard.check(step)
            except RankLeftError as exc:
                outcome = f"detected at step {step} after {time.monotonic() - begin:.2f} s: {exc}"
                break
            arena.zero()
            arena.views[0].add_(float(rank + 1))
            arena.all_reduce()
            assert float(arena.flat[0]) == 6.0     # 1 + 2 + 3
            outcome = f"ran step {step}"
        results[rank] = outcome
    finally:
        # the survivors do not run another collective; tear the group down without a barrier
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_rank_that_leaves_between_steps_is_detected_on_the_host():
    world = 3
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_leaver_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(150)
        assert p.exitcode == 0, "a rank hung or crashed instead of reporting the departure"
    assert results[2] == "left"
    for rank in (0, 1):
        assert results[rank].startswith("detected at step 2"), results[rank]
        assert "rank 2 left" in results[rank]


def _silent_worker(rank: int, world: int, port: int, results):
    """Rank 1 stops announcing steps without saying so (as a crashed process would); rank 0's guard times out."""
    from molt_b200.data_parallel import RankLeftError, StepGuard

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        guard = StepGuard(timeout=1.5)
        guard.check(0)
        if rank == 1:
            results[rank] = "silent"
            return
        try:
            guard.check(1)
            results[rank] = "no error"
        except RankLeftError as exc:
            results[rank] = f"timeout: {exc}"
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_silent_rank_times_out_instead_of_hanging():
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_silent_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
        assert p.exitcode == 0
    assert results[1] == "silent" and results[0].startswith("timeout") and "did not reach step 1" in results[0]


def test_layer_buckets_follow_the_given_starts():
    params = [torch.nn.Parameter(torch.zeros(n)) for n in (10, 70, 64, 5, 130)]
    arena = GradArena(params, bucket_starts=[0, 2, 4])
    # listed from the last layer to the first; slices are padded to 64 elements
    assert arena.buckets == [(arena.offsets[4], arena.flat.numel()), (arena.offsets[2], arena.offsets[4]),
                             (0, arena.offsets[2])]
    assert [arena.bucket_of_param(i) for i in range(5)] == [2, 2, 1, 1, 0]
    with pytest.raises(ValueError):
        GradArena(params, bucket_starts=[1, 3])
