"""World-size-2 test of the data-parallel host logic on CPU (gloo): bucket boundaries cover the flat
gradient buffer exactly once, gradients come out averaged, and per-rank token streams differ."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sys, pathlib
        root = pathlib.Path(__file__).resolve().parent.parent
        sys.path.insert(0, str(root / "photon-mamba2-llm_b200"))
        from pm_b200.dp import GradAllReducer, layer_bounds
        # flat layout: embedding 100 floats (padded to 128), 3 layers of 200 floats each
        offsets, total = [128, 328, 528], 728
        flat = torch.arange(total, dtype=torch.float32) * (rank + 1)
        red = GradAllReducer(flat, offsets)
        covered = torch.zeros(total)
        for l in (2, 1, 0, -1):                      # backward order, embedding last
            a = red.bucket(l)
            covered[a.storage_offset():a.storage_offset() + a.numel()] += 1
            red.on_layer_done(l)
        done = red.finish()
        expect = torch.arange(total, dtype=torch.float32) * (sum(range(1, world + 1)) / world)
        ok = bool(torch.equal(covered, torch.ones(total))) and torch.allclose(flat, expect) and done == [2, 1, 0, -1]
        assert layer_bounds(offsets, total) == [(128, 328), (328, 528), (528, 728)]
        # a second step reuses the reducer
        flat.fill_(float(rank))
        for l in (2, 1, 0, -1):
            red.on_layer_done(l)
        red.finish()
        ok = ok and torch.allclose(flat, torch.full((total,), (world - 1) / 2.0))
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_bucketed_gradient_average_world2():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]


def test_per_rank_token_streams_differ_and_are_reproducible():
    import bench
    a0, _ = bench.make_tokens("c1_single_block_dims_lm", 0, 0, pin=False)
    a0b, _ = bench.make_tokens("c1_single_block_dims_lm", 0, 0, pin=False)
    a1, t1 = bench.make_tokens("c1_single_block_dims_lm", 1, 0, pin=False)
    assert torch.equal(a0, a0b) and not torch.equal(a0, a1)
    assert torch.equal(t1[:, :-1], a1[:, 1:]) and torch.equal(t1[:, -1], a1[:, 0])
