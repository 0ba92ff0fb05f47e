"""Host-side multi-rank logic on CPU: population sharding, stripe rows, ring halo exchange and sum all-reduce
over gloo with 2 and 3 ranks (the same code drives NCCL on GPUs)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from slime_b200 import sharding


def test_shard_population_partitions_grids_with_their_weight_sets():
    for world in (1, 2, 4, 8):
        shards = [sharding.shard_population(1024, 128, r, world) for r in range(world)]
        assert sum(s.n_grids for s in shards) == 1024 and sum(s.n_sets for s in shards) == 128
        for r, s in enumerate(shards):
            assert s.first_grid == r * 1024 // world and s.first_set == r * 128 // world
            # every local grid's weight set is local
            for b in (s.first_grid, s.first_grid + s.n_grids - 1):
                assert s.first_set <= b // 8 < s.first_set + s.n_sets
    s = sharding.shard_population(64, 1, 3, 4)          # one shared set is replicated
    assert (s.first_grid, s.n_grids, s.first_set, s.n_sets) == (48, 16, 0, 1)
    with pytest.raises(ValueError):
        sharding.shard_population(10, 3, 0, 2)
    with pytest.raises(ValueError):
        sharding.shard_population(12, 3, 0, 2)


def test_stripe_rows():
    assert sharding.stripe_rows(8192, 3, 8) == (3072, 1024)
    with pytest.raises(ValueError):
        sharding.stripe_rows(10, 0, 3)
    with pytest.raises(ValueError):
        sharding.stripe_rows(8, 0, 4)      # 2-row stripes are thinner than the halo


def test_single_rank_ring_wraps_locally():
    ring = sharding.StripeRing()
    n, W = 5, 4
    st = torch.zeros(1, n + 6, W, 64)
    st[:, 3:3 + n] = torch.arange(n, dtype=torch.float32).view(1, n, 1, 1)
    ring.exchange_halos(st, n)
    assert st[0, 0:3, 0, 0].tolist() == [2.0, 3.0, 4.0]       # rows above row 0 on the torus
    assert st[0, n + 3:n + 6, 0, 0].tolist() == [0.0, 1.0, 2.0]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, W, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ring = sharding.StripeRing()
        first, rows = sharding.stripe_rows(n * world, rank, world)
        st = torch.full((1, rows + 6, W, 64), -1.0)
        own = torch.arange(first, first + rows, dtype=torch.float32).view(1, rows, 1, 1).expand(1, rows, W, 64)
        st[:, 3:3 + rows] = own
        ring.exchange_halos(st, rows)
        H = n * world
        want_top = [float((first - 3 + i) % H) for i in range(3)]
        want_bot = [float((first + rows + i) % H) for i in range(3)]
        ok = st[0, 0:3, 0, 0].tolist() == want_top and st[0, rows + 3:rows + 6, W - 1, 63].tolist() == want_bot
        ok = ok and bool((st[:, 3:3 + rows] == own).all())
        sums = torch.full((1, 64), float(rank + 1), dtype=torch.float64)
        ring.allreduce_sums(sums)
        ok = ok and bool((sums == world * (world + 1) / 2).all())
        out[rank] = int(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_ring_halo_exchange_and_allreduce_over_gloo(world):
    port = _free_port()
    ctx = mp.get_context("spawn")
    out = ctx.Array("i", [0] * world)
    procs = [ctx.Process(target=_worker, args=(r, world, port, 4, 5, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert list(out) == [1] * world


def _timeout_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ring = sharding.StripeRing(timeout_s=1.0)
    st = torch.zeros(1, 4 + 6, 3, 64)
    if rank == 0:
        # rank 1 never takes part in this exchange: the wait must end with RingTimeout, not block
        try:
            ring.exchange_halos(st, 4)
            out[0] = 0
        except sharding.RingTimeout as e:
            out[0] = 1 if "halo rows" in str(e) else 0
    else:
        import time
        t0 = time.monotonic()
        while out[0] < 0 and time.monotonic() - t0 < 30:      # stay connected, but silent, until rank 0 has given up
            time.sleep(0.05)
        out[1] = 1
    # the transfers rank 0 posted can never complete: leave without the collective teardown
    os._exit(0)


def test_ring_wait_is_bounded_when_a_neighbour_never_sends():
    port = _free_port()
    ctx = mp.get_context("spawn")
    out = ctx.Array("i", [-1, -1])
    procs = [ctx.Process(target=_timeout_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert list(out) == [1, 1]
