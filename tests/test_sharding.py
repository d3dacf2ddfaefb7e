"""Multi-GPU host logic on CPU: two gloo ranks shard a batch, each runs its shard (through the oracle
here; through its own Session on GPUs), and the concatenated rows equal the full-batch result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sofie_b200 import sharding


def test_shard_bounds_cover_the_batch_exactly():
    for batch in (0, 1, 7, 256, 1000):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.shard_bounds(batch, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(e - b for b, e in spans) == -(-batch // world)
    with pytest.raises(ValueError):
        sharding.shard_bounds(8, 2, 2)


def _worker(rank, world, port, batch, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import run_model
        from sofie_b200 import configs
        m, x = configs.mlp_i8(batch=batch, dims=(64, 48, 16))
        local = run_model.run(m, sharding.shard(x, world, rank))
        full = sharding.gather_rows(local, batch)
        slowest = sharding.max_over_ranks(1.0 + rank)
        if rank == 0:
            ref = run_model.run(m, x)
            out.put((bool(np.array_equal(full.view(np.uint32), ref.view(np.uint32))), slowest))
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_and_reassemble():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 37, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    same, slowest = out.get(timeout=10)
    assert same and slowest == 2.0
