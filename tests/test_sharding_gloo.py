"""CPU: the multi-rank host logic (camel_b200/sharding.py) as two gloo ranks.

The kernels have no CPU form, so each rank's row block of the product is computed here with
numpy; what is under test is the partitioning, the panel-wise all-gather that reassembles C on
every rank, and the max-over-ranks reduction the bench uses for its timings.
"""
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from camel_b200 import sharding


def test_batch_shards_tile_the_batch():
    for batch in (0, 1, 7, 4096, 8191):
        for world in (1, 2, 3, 8):
            parts = [sharding.batch_shard(batch, world, r) for r in range(world)]
            assert parts[0][0] == 0
            for (f0, c0), (f1, _) in zip(parts, parts[1:]):
                assert f0 + c0 == f1
            assert parts[-1][0] + parts[-1][1] == batch
            counts = [c for _, c in parts]
            assert max(counts) - min(counts) <= 1


def test_row_shards_and_panels():
    assert sharding.row_shard(16384, 8, 3) == (3 * 2048, 2048)
    with pytest.raises(ValueError):
        sharding.row_shard(10, 4, 0)
    for rows, panels in ((2048, 4), (10, 4), (3, 4), (0, 4), (7, 1)):
        plan = sharding.panel_plan(rows, panels)
        assert sum(c for _, c in plan) == rows
        at = 0
        for off, cnt in plan:
            assert off == at and cnt > 0
            at += cnt
        assert len(plan) <= panels


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, n, panels, out):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)
        a = rng.uniform(-1, 1, (n, n)).astype(np.float32)
        b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
        row0, rows = sharding.row_shard(n, world, rank)
        c_full = torch.full((n, n), float("nan"), dtype=torch.float32)
        for off, cnt in sharding.panel_plan(rows, panels):
            block = a[row0 + off: row0 + off + cnt].astype(np.float64) @ b.astype(np.float64)
            c_full[row0 + off: row0 + off + cnt] = torch.from_numpy(block.astype(np.float32))
            sharding.gather_panel(dist, c_full, rows, off, cnt, rank, world)
        ref = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
        ok = bool(np.array_equal(c_full.numpy(), ref))
        slowest = sharding.reduce_max(dist, torch, 10.0 + rank, "cpu")
        out.put((rank, ok, slowest))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_sharded_product_is_reassembled_on_every_rank():
    world, n, panels = 2, 96, 4
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, n, panels, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=100) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert [r for r, _, _ in results] == [0, 1]
    assert all(ok for _, ok, _ in results)
    assert all(slowest == 11.0 for _, _, slowest in results)


def test_reduce_max_without_process_group():
    assert sharding.reduce_max(None, torch, 3.5, "cpu") == 3.5


def test_tapered_panel_plan_covers_rows_and_shrinks():
    from camel_b200 import sharding

    for rows in (0, 1, 100, 512, 513, 1024, 2048, 4096, 16384, 2000, 3001):
        plan = sharding.tapered_panel_plan(rows)
        assert sum(c for _, c in plan) == rows
        at = 0
        for off, cnt in plan:
            assert off == at and cnt > 0
            at += cnt
        sizes = [c for _, c in plan]
        assert sizes == sorted(sizes, reverse=True)  # the exposed last gather is the smallest
    assert [c for _, c in sharding.tapered_panel_plan(2048)] == [1024, 512, 256, 256]


def test_banded_rows_partition_every_row_once():
    from camel_b200 import sharding

    for rows_per_rank, world in ((2048, 8), (4096, 4), (1000, 3), (96, 2)):
        plan = sharding.tapered_panel_plan(rows_per_rank, smallest=16, unit=8)
        seen = np.zeros(rows_per_rank * world, np.int32)
        for rank in range(world):
            local = 0
            for off, cnt, g0, band0 in sharding.banded_rows(plan, world, rank):
                assert off == local and g0 == band0 + rank * cnt
                seen[g0:g0 + cnt] += 1
                local += cnt
            assert local == rows_per_rank
        assert np.all(seen == 1)


def _banded_rank_main(rank, world, port, n, out):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(6)
        a = rng.uniform(-1, 1, (n, n)).astype(np.float32)
        b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
        rows = n // world
        plan = sharding.tapered_panel_plan(rows, smallest=8, unit=4)
        c_full = torch.full((n, n), float("nan"), dtype=torch.float32)
        for off, cnt, g0, band0 in sharding.banded_rows(plan, world, rank):
            block = a[g0:g0 + cnt].astype(np.float64) @ b.astype(np.float64)
            c_full[g0:g0 + cnt] = torch.from_numpy(block.astype(np.float32))
            sharding.gather_band(dist, c_full, band0, cnt, rank, world)
        ref = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
        out.put((rank, bool(np.array_equal(c_full.numpy(), ref)), len(plan)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_banded_product_is_reassembled_in_place_on_every_rank():
    world, n = 2, 96
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_banded_rank_main, args=(r, world, port, n, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=100) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
    assert [r[1] for r in results] == [True] * world
    assert results[0][2] >= 3  # several bands
