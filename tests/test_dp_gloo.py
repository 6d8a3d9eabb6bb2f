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
