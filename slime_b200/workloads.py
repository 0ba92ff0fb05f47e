"""The measured workloads beyond the headline batch, run through the public C ABI; one JSON line each.

  python -m slime_b200.workloads --config 1|3|4|5 [--dtype bf16|f32] [--scale-down K]
  python -m torch.distributed.run --nproc-per-node N -m slime_b200.workloads --config 3|4|5

  1  the CPU-runnable reference model: X[1,128,128,64] fp32, 16 steps
  3  batch-sharded population: 1024 grids, 128 weight sets x 8 grids, 32 steps, then fitness per grid and the
     population step (cull below the median, refill from the best) on each rank's share
  4  one large torus split into row stripes: X[1,8192,8192,64] bf16, 100 steps, halo exchange + mass all-reduce
  5  supervised-input shape: 4096 images 28x28 -> 32x32x64, 24 steps, mean-pool + 64->10 read-out

`--scale-down K` divides the population / image batch / grid edge by K (for quick checks).  Throughput is in CA
cell-updates per second over all ranks, timed on the device (max over ranks) with the state resident.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from . import capi, inputs, sharding


def _dist():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def _timed(fn, world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def config1(args, rank, world, local):
    X0 = inputs.make_state(1, 128, 128, seed=42)
    w = inputs.make_weight_sets(1, seed=42)
    with capi.Handle(1, 128, 128, dtype=capi.F32, device=local, keep_vprime=True) as h:
        h.set_weights(w)
        h.set_state(X0)
        h.step(16)                      # warm
        h.set_state(X0)
        ms = _timed(lambda: h.step(16), 1)
        X1, fit = h.get_state(), h.fitness()
    m = np.abs(X1.reshape(-1, 64).astype(np.float64).sum(0) - 1.0).max()
    return {"config": 1, "workload": "X[1,128,128,64] fp32, 16 steps", "dtype": "f32", "n_gpus": 1, "ms": ms,
            "cell_updates_per_s": 128 * 128 * 16 / (ms * 1e-3), "max_mass_error": float(m),
            "fitness": float(fit["fitness"][0])}


def config3(args, rank, world, local):
    n_grids, n_sets, steps = 1024 // args.scale_down, 128 // args.scale_down, 32
    sh = sharding.shard_population(n_grids, n_sets, rank, world)
    dt = capi.BF16 if args.dtype == "bf16" else capi.F32
    w = inputs.make_weight_sets(sh.n_sets, seed=42, first_set=sh.first_set, bounded=True)
    h = capi.Handle(sh.n_grids, 128, 128, n_weight_sets=sh.n_sets, dtype=dt, device=local, keep_vprime=True)
    h.set_weights(w)
    stage = torch.empty((sh.n_grids, 128, 128, 64), dtype=torch.float32).pin_memory()
    for b0 in range(0, sh.n_grids, 16):          # generate 16 grids at a time: the generator works in fp64
        n = min(16, sh.n_grids - b0)
        stage[b0:b0 + n] = torch.from_numpy(inputs.make_state(n, 128, 128, seed=42, first_grid=sh.first_grid + b0))
    h.set_state_ptr(stage.data_ptr(), capi.F32)
    h.step(2)                            # warm
    h.set_state_ptr(stage.data_ptr(), capi.F32)
    ms = _timed(lambda: h.step(steps), world)
    ms_fit = _timed(lambda: h.fitness(), world)
    fit = h.fitness()
    # the population step that consumes the fitness: cull the sets below the median, refill them from the best
    set_fit = fit["fitness"].astype(np.float64).reshape(sh.n_sets, -1).mean(1)
    thr = float(10.0 * np.nanmedian(set_fit))
    evo = {}

    def population_step():
        evo.update(h.evolve(fitness_threshold=thr, hunger_threshold=2.0, mutation_rate=0.01, mutation_sigma=0.0125,
                            seed=42, generation=1))
    ms_evolve = _timed(population_step, world)
    h.close()
    local_stats = torch.tensor([float(np.nanmean(fit["rank"])), float(np.nanmean(fit["coherence"])),
                                float(np.isfinite(fit["fitness"]).mean())], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(local_stats, op=dist.ReduceOp.SUM)
        local_stats /= world
    return {"config": 3, "workload": f"{n_grids} grids 128x128x64, {n_sets} weight sets, {steps} steps + fitness",
            "dtype": args.dtype, "n_gpus": world, "ms": ms, "ms_fitness": ms_fit, "ms_population_step": ms_evolve,
            "sets_replaced_rank0": int(evo["n_replaced"]),
            "cell_updates_per_s": n_grids * 128 * 128 * steps / (ms * 1e-3),
            "mean_rank": float(local_stats[0]), "mean_coherence": float(local_stats[1]),
            "finite_fraction": float(local_stats[2]), "scaling": "strong (1024 grids split over the ranks)"}


def random_striped_grid(edge, dtype_name, rank, world, local, weights):
    """One edge x edge torus split into `world` row stripes, this rank's stripe filled on the device with a uniform
    state of unit mass per channel (seeded per rank) and adopted as the state; -> (StripedGrid, target masses).

    The state of the full-size torus (4.3e9 elements) is drawn on the device: throughput does not depend on the
    values, and the seeded host generator would need minutes and tens of GB for this size."""
    dt = capi.BF16 if dtype_name == "bf16" else capi.F32
    grid = sharding.StripedGrid(edge, edge, weights, dtype=dt, device=local)
    gen = torch.Generator(device="cuda").manual_seed(42 + rank)
    tdt = torch.bfloat16 if dtype_name == "bf16" else torch.float32
    own = grid.state[:, sharding.HALO:sharding.HALO + grid.n_rows]
    for r0 in range(0, grid.n_rows, 256):
        blk = own[:, r0:r0 + 256]
        blk.copy_(torch.rand(blk.shape, generator=gen, device="cuda", dtype=torch.float32).to(tdt))
    sums = torch.zeros(1, 64, dtype=torch.float64, device="cuda")
    for r0 in range(0, grid.n_rows, 256):
        sums += own[:, r0:r0 + 256].float().sum(dim=(1, 2), dtype=torch.float64)
    grid.ring.allreduce_sums(sums)
    for r0 in range(0, grid.n_rows, 256):
        blk = own[:, r0:r0 + 256]
        blk.copy_((blk.float() / sums.float().view(1, 1, 1, 64)).to(tdt))
    # adopt what is now stored as the state: masses from the stored values, summed over ranks
    grid.handle.set_state_device(own.contiguous().data_ptr(), dt)
    grid.adopt_masses()
    mass = torch.from_numpy(grid.handle.get_mass()).cuda()
    return grid, mass


def striped_mass_error(grid, mass):
    """Largest relative deviation of the torus's per-channel masses from their targets (summed over the ranks)."""
    X = grid.read()
    s = torch.from_numpy(X.reshape(-1, 64).astype(np.float64).sum(0)).cuda()
    grid.ring.allreduce_sums(s)
    return float((s.cpu() - mass.cpu()[0]).abs().div(mass.cpu()[0].abs()).max())


def config4(args, rank, world, local):
    edge, steps = 8192 // args.scale_down, 100
    w = inputs.make_weight_sets(1, seed=42, bounded=True)
    grid, mass = random_striped_grid(edge, args.dtype, rank, world, local, w)
    grid.step(2)
    ms = _timed(lambda: grid.step(steps), world)
    split = grid.handle.step_ring_timed(10)
    err = striped_mass_error(grid, mass)
    grid.close()
    return {"config": 4, "workload": f"X[1,{edge},{edge},64] row stripes, {steps} steps, 3-row halo exchange + 64-value all-reduce per step "
                                     "(ring inside the C library: ncclSend/ncclRecv/ncclAllReduce on the stream)",
            "dtype": args.dtype, "n_gpus": world, "ms": ms, "cell_updates_per_s": edge * edge * steps / (ms * 1e-3),
            "ms_per_step_halo": split[0] / 10, "ms_per_step_kernels": split[1] / 10, "ms_per_step_allreduce": split[2] / 10,
            "max_mass_error": err, "scaling": "strong", "weights": "mass-neutral variant of the specified draws"}


def config5(args, rank, world, local):
    n_img, steps = 4096 // args.scale_down, 24
    per = n_img // world
    dt = capi.BF16 if args.dtype == "bf16" else capi.F32
    L, Wr, br = inputs.make_lift_readout(seed=42)
    w = inputs.make_weight_sets(1, seed=42, bounded=True, mass_profile=L)
    img = inputs.make_images(per, 28, seed=42, first=rank * per)
    with capi.Handle(per, 32, 32, dtype=dt, device=local) as h:
        h.set_weights(w)
        h.lift_images(img, L)
        h.step(2)
        h.lift_images(img, L)
        ms = _timed(lambda: h.step(steps), world)
        logits = h.pool_readout(Wr, br)
    return {"config": 5, "workload": f"{n_img} images 28x28 -> 32x32x64, {steps} steps, mean-pool + 64->10 read-out",
            "dtype": args.dtype, "n_gpus": world, "ms": ms, "cell_updates_per_s": n_img * 32 * 32 * steps / (ms * 1e-3),
            "logits_finite": bool(np.isfinite(logits).all()), "logit0": [float(v) for v in logits[0][:3]],
            "weights": "mass-neutral variant of the specified draws for the lifted state's mass profile (the plain "
                       "draws diverge within 16 steps, in the fp64 CPU oracle too)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, required=True, choices=[1, 3, 4, 5])
    ap.add_argument("--dtype", choices=["bf16", "f32"], default="bf16")
    ap.add_argument("--scale-down", type=int, default=1)
    args = ap.parse_args()
    rank, world, local = _dist()
    out = {1: config1, 3: config3, 4: config4, 5: config5}[args.config](args, rank, world, local)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
