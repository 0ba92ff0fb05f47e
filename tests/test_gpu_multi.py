"""Two-GPU tests (skipped on a single-GPU box): row-stripe decomposition over NCCL against one GPU holding the
whole torus, and a batch-sharded population against the unsharded run."""
import os
import socket

import numpy as np
import pytest

from slime_b200 import inputs
from tests.helpers import rel_l2

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _stripe_worker(rank, world, port, H, W, steps, dtype, out_path, library_ring):
    import torch
    import torch.distributed as dist
    from slime_b200 import capi, sharding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        X0 = inputs.make_state(1, H, W, seed=8, scale=0.45 * H * W)
        w = inputs.make_weight_sets(1, seed=8)
        grid = sharding.StripedGrid(H, W, w, dtype=dtype, device=rank, library_ring=library_ring)
        grid.load(X0[:, grid.first_row:grid.first_row + grid.n_rows])
        grid.step(steps)
        if library_ring:
            grid.handle.ring_wait(60000)      # the bounded host wait of the library's ring
        np.save(out_path % rank, grid.read())
        grid.close()
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("library_ring", [True, False], ids=["library_ring", "python_ring"])
@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_stripes_over_nccl_match_one_gpu(tmp_path, dtype_name, library_ring):
    """Two row stripes on two GPUs against one GPU holding the whole torus: through the ring inside the C library
    (slime_ca_step_ring: ncclSend / ncclRecv / ncclAllReduce on the stream) and through the Python ring."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from slime_b200 import capi
    dtype = capi.F32 if dtype_name == "f32" else capi.BF16
    H, W, steps, world = 64, 48, 3, 2
    X0 = inputs.make_state(1, H, W, seed=8, scale=0.45 * H * W)
    w = inputs.make_weight_sets(1, seed=8)
    with capi.Handle(1, H, W, dtype=dtype) as h:
        h.set_weights(w); h.set_state(X0); h.step(steps)
        ref = h.get_state()
    port = _free_port()
    out = str(tmp_path / "stripe_%d.npy")
    mp.spawn(_stripe_worker, args=(world, port, H, W, steps, dtype, out, library_ring), nprocs=world, join=True)
    got = np.concatenate([np.load(out % r) for r in range(world)], axis=1)
    assert rel_l2(got, ref) < (1e-6 if dtype_name == "f32" else 2e-3)


def test_population_shards_equal_the_unsharded_run():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from slime_b200 import capi, sharding
    n_grids, n_sets, steps = 8, 4, 3
    w = inputs.make_weight_sets(n_sets, seed=21)
    X0 = inputs.make_state(n_grids, 32, 32, seed=21, scale=0.45 * 1024)
    with capi.Handle(n_grids, 32, 32, n_weight_sets=n_sets, dtype=capi.BF16, keep_vprime=True) as h:
        h.set_weights(w); h.set_state(X0); h.step(steps)
        ref, ref_fit = h.get_state(), h.fitness()
    for rank in range(2):
        sh = sharding.shard_population(n_grids, n_sets, rank, 2)
        ws = inputs.make_weight_sets(sh.n_sets, seed=21, first_set=sh.first_set)
        Xs = inputs.make_state(sh.n_grids, 32, 32, seed=21, scale=0.45 * 1024, first_grid=sh.first_grid)
        with capi.Handle(sh.n_grids, 32, 32, n_weight_sets=sh.n_sets, dtype=capi.BF16, device=rank, keep_vprime=True) as h:
            h.set_weights(ws); h.set_state(Xs); h.step(steps)
            got, fit = h.get_state(), h.fitness()
        assert np.array_equal(got, ref[sh.first_grid:sh.first_grid + sh.n_grids])
        np.testing.assert_allclose(fit["fitness"], ref_fit["fitness"][sh.first_grid:sh.first_grid + sh.n_grids], rtol=1e-6)
