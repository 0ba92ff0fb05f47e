#!/usr/bin/env python
"""Throughput of the Flow-Lenia CA step in cell-updates/s.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype bf16|f32] [--impl ours|reference]

Workload (N=1 and every N, weak scaling: each rank steps its own batch, no data-path collective): the batched
training-shape forward X[64,128,128,64], bf16 storage / fp32 accumulate, 8 heads x 64, 64 CA steps per bench
step, seeded synthetic state (uniform, unit mass per channel) and one seeded weight set (the specified draws with
the output projection made mass-neutral, inputs.mass_neutral: with the plain draws the state grows 1.38x per step
and overflows long before step 64).  One bench "step" is one such 64-step forward, started from the same state
every time.  `value` is timed with the state resident in HBM (restored from a device copy at the start of every
forward); `e2e` copies the state in from pinned host memory and back out through the C ABI inside the timed region.

After that timing the line also gets a `stripe` object: one 8192 x 8192 torus split into N row stripes (strong
scaling), 10 steps through the ring inside the C library (NCCL halo rows + all-reduce of the channel sums), with
the per-step split between halo exchange, kernels and all-reduce, the mass error, and the parity of a small torus
stepped as N stripes against rank 0 holding it whole.

`--impl reference` times the CPU transcription of the same step (the reference has no CPU path and no runnable
GPU step; the transcription is the oracle's fp32 build, all host threads) on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "CA cell-updates/sec"
UNIT = "cell-updates/s"
GRID, BATCH, CA_STEPS = 128, 64, 64
# algorithmic HBM bytes per cell-update of each kernel (bf16 / f32 storage): k1 reads the state (64 values) and
# writes E and V (2 x 512 values); k2 reads E and V and reads + writes the state.
ALG_BYTES = {"k1": {"bf16": 128 + 2048, "f32": 256 + 4096}, "k2": {"bf16": 2048 + 256, "f32": 4096 + 512}}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", 1400.0)), "measured"
    return 6650.0, 1400.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self._halt = index, [], threading.Event()

    def run(self):
        while not self._halt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                f = [x.strip() for x in out.strip().split(",")]
                if len(f) == 6:
                    self.rows.append(f)
            except Exception:
                pass
            self._halt.wait(0.2)

    def stop(self):
        self._halt.set()
        self.join(timeout=6)
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(float(r[0]) for r in self.rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(self.rows)}


def ncu_dram_bytes_per_cell(kernel):
    """DRAM bytes per cell-update of a bf16 kernel, read from the ncu summary committed under profiles/
    (dram__bytes_read.sum + dram__bytes_write.sum of one captured launch over the cells of that launch) -> (bytes per
    cell, file name), or (None, None) if there is no readable summary.  The captures are batches of 8 or 16 grids (a
    quarter to half a GB of E/V per kernel, larger than L2); traffic grows in proportion to the cells, so a full launch
    is this figure times its cells.  k1's figure sits below its algorithmic bytes because part of what it wrote was still
    dirty in the 126 MB L2 when the captured launch ended."""
    import glob
    import re
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", f"{kernel}_bf16_batch*_128x128.txt"))):
        try:
            text = open(path).read()
            cells = int(re.search(r"one launch = ([\d ]+) cells", text).group(1).replace(" ", ""))
            unit = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
            total = 0.0
            for name in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
                m = re.search(r"^" + re.escape(name) + r"\s+([\d.]+)\s+(\w+)", text, re.M)
                total += float(m.group(1)) * unit[m.group(2)]
            return total / cells, os.path.basename(path)
        except (OSError, AttributeError, KeyError, ValueError):
            continue
    return None, None


def bench_config(batch, ca_steps, dtype, world):
    """The `config` object of the bench line: the same for this library's arm and for the reference arm."""
    cells = batch * GRID * GRID
    return {"workload": f"batched training-shape forward X[{batch},{GRID},{GRID},64] per GPU, 8 heads x 64, "
                        f"{ca_steps} CA steps per bench step, renorm every step",
            "weights": "specified draws, output projection made mass-neutral so the trajectory stays finite",
            "l2": "working set per step (E,V intermediates %.1f GB) exceeds the 126 MB L2" %
                  (2 * cells * 512 * (2 if dtype == "bf16" else 4) / 1e9),
            "parallelism": f"batch-sharded x{world}, no data-path collective"}


def cpu_baseline(ca_steps_sample=2, grids=1):
    """The oracle's fp32 multithreaded transcription on a bounded sample: `grids` grids x `ca_steps_sample` steps."""
    from oracle import ca_oracle
    from slime_b200 import inputs
    X = inputs.make_state(grids, GRID, GRID, seed=42)
    w = inputs.make_weight_sets(1, seed=42, bounded=True)
    # all the host threads this process may use, whatever OMP_NUM_THREADS the launcher exported
    cores = ca_oracle.set_threads(ca_oracle.usable_cpus(), real="f32")
    ca_oracle.ca_steps(X[:1, :16, :16].copy(), w, 1, literal=False, real="f32")       # load + warm the library
    t0 = time.perf_counter()
    ca_oracle.ca_steps(X, w, ca_steps_sample, literal=False, real="f32")
    dt = time.perf_counter() - t0
    return {"value": grids * GRID * GRID * ca_steps_sample / dt, "unit": UNIT, "cores": cores, "kind": "port", "seconds": dt,
            "sample": f"{grids} grid(s) of {GRID}x{GRID}x64, {ca_steps_sample} CA steps, fp32, OpenMP on {cores} threads "
                      f"({dt:.1f} s)"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    per_step, secs = [], []
    base = None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline(ca_steps_sample=CA_STEPS, grids=2)      # 2 of the 64 grids, all 64 steps: about 3 s
        if i >= args.warmup:
            per_step.append(base["value"])
            secs.append(base["seconds"])
    v = float(np.mean(per_step))
    base["value"] = v
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": float(np.mean(secs)) * 1e3,       # what a (sampled) step really took
            "ms_per_full_step_extrapolated": BATCH * GRID * GRID * CA_STEPS / v * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            # the workload of this library's arm; each step of this arm times a bounded sample of it (2 of the 64 grids
            # for all 64 CA steps, see cpu_baseline.sample) and the rate is that of the sample
            "config": bench_config(BATCH, CA_STEPS, "bf16", args.gpus),
            "cpu_baseline": base,
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dtype", choices=["bf16", "f32"], default="bf16")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--ca-steps", type=int, default=CA_STEPS)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-stripe", action="store_true", help="skip the row-stripe leg")
    ap.add_argument("--stripe-edge", type=int, default=8192)
    ap.add_argument("--stripe-steps", type=int, default=10)
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from slime_b200 import capi, inputs

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.warmup < 3:
        args.warmup = 3

    B, S = args.batch, args.ca_steps
    dt_code = capi.BF16 if args.dtype == "bf16" else capi.F32
    tdt = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    weights = inputs.make_weight_sets(1, seed=42, bounded=True)
    h = capi.Handle(B, GRID, GRID, n_weight_sets=1, dtype=dt_code, device=local)
    h.set_weights(weights)
    X0 = inputs.make_state(B, GRID, GRID, seed=42, first_grid=rank * B)
    host = torch.from_numpy(X0).to(tdt).pin_memory()
    host_out = torch.empty_like(host).pin_memory()
    dev0 = host.cuda()                       # the forward's start state, resident: restored before every forward
    state_bytes = host.numel() * host.element_size()
    stream = torch.cuda.current_stream().cuda_stream
    cells = B * GRID * GRID

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # ---- device-resident throughput: every forward starts from the same resident state --------------
    def forward():
        h.set_state_device(dev0.data_ptr(), dt_code, stream)     # D2D restore + the masses of the start state
        h.step(S, stream)

    for _ in range(args.warmup):
        forward()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    l0 = h.launch_count
    ms = timed(forward, args.steps)
    launches = h.launch_count - l0
    clocks = sampler.stop() if sampler else None
    value = world * cells * S * args.steps / (ms * 1e-3)
    # what the last timed forward left: finite, and every channel's mass where it started
    X_end = h.get_state(stream)
    m0 = host.float().numpy().reshape(B, -1, 64).astype(np.float64).sum(1)
    m1 = X_end.reshape(B, -1, 64).astype(np.float64).sum(1)
    state_check = {"finite": bool(np.isfinite(X_end).all()), "max_mass_error": float(np.max(np.abs(m1 - m0) / np.abs(m0))),
                   "max_abs_over_start": float(np.abs(X_end).max() / np.abs(X0).max())}

    # ---- per-kernel time of the same step loop (CUDA events between the kernels, on the launch stream) ----
    h.set_state_device(dev0.data_ptr(), dt_code, stream)
    kt = h.step_timed(S, stream)          # ms summed over the S steps: k1, k2, reductions
    dom = "k1" if kt[0] >= kt[1] else "k2"
    dom_ms = max(kt[0], kt[1]) / S
    peak, tensor_peak, peak_kind = measured_peaks()
    achieved = cells * ALG_BYTES[dom][args.dtype] / (dom_ms * 1e-3) / 1e9
    per_cell, per_cell_file = ncu_dram_bytes_per_cell(dom) if args.dtype == "bf16" else (None, None)
    roofline = {"bound": "hbm", "kernel": dom + "_" + args.dtype, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": None if per_cell is None else cells * per_cell, "peak_kind": peak_kind,
                "traffic_source": f"profiles/{per_cell_file} scaled by cells" if per_cell else None,
                "algorithmic_bytes_per_launch": cells * ALG_BYTES[dom][args.dtype],
                "ms_per_launch": dom_ms, "k1_ms": kt[0] / S, "k2_ms": kt[1] / S, "other_ms": kt[2] / S,
                "k1_frac": cells * ALG_BYTES["k1"][args.dtype] / (kt[0] / S * 1e-3) / 1e9 / peak,
                "k2_frac": cells * ALG_BYTES["k2"][args.dtype] / (kt[1] / S * 1e-3) / 1e9 / peak,
                # the projections' 262 144 flop per cell-update over the whole step, against the sustained bf16 peak
                # (the kernels run inside a long step loop): context, not the bound - the step is not tensor-bound
                "tensor": {"achieved": cells * 262144 / ((kt[0] + kt[1] + kt[2]) / S * 1e-3) / 1e12, "peak": tensor_peak,
                           "unit": "TFLOP/s", "frac": cells * 262144 / ((kt[0] + kt[1] + kt[2]) / S * 1e-3) / 1e12 / tensor_peak}}

    # ---- end to end through the C ABI: host state in, 64 steps, host state out -------------------
    def e2e_step():
        h.set_state_ptr(host.data_ptr(), dt_code, stream)
        h.step(S, stream)
        h.get_state_ptr(host_out.data_ptr(), dt_code, stream)

    for _ in range(2):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    e2e = {"value": world * cells * S * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
           "h2d_bytes_per_step": state_bytes, "d2h_bytes_per_step": state_bytes}
    h.close()
    del dev0
    torch.cuda.empty_cache()

    stripe = None if args.no_stripe else stripe_leg(args, rank, world, local, weights, timed)

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
                "config": bench_config(B, S, args.dtype, world),
                "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline,
                "state_after_last_timed_forward": state_check, "stripe": stripe}
        if not args.no_cpu_baseline and world == 1:       # the CPU baseline is timed at N = 1 only
            line["cpu_baseline"] = cpu_baseline(ca_steps_sample=CA_STEPS, grids=8)   # 8 of the 64 grids: 10-15 s
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def stripe_leg(args, rank, world, local, weights, timed):
    """The row-stripe split under the same launch: one torus, N stripes, the ring inside the C library."""
    import torch
    import torch.distributed as dist
    from slime_b200 import capi, inputs, sharding, workloads

    dt_code = capi.BF16 if args.dtype == "bf16" else capi.F32
    edge, steps = args.stripe_edge, args.stripe_steps
    out = {"workload": f"X[1,{edge},{edge},64] {args.dtype} torus as {world} row stripe(s), {steps} steps per timing, 3-row halo "
                       "exchange (ncclSend/ncclRecv) + all-reduce of the 64 channel sums (fp64) every step, enqueued by "
                       "slime_ca_step_ring with no host synchronisation per step", "scaling": "strong"}
    # parity first, on a small torus: N stripes through the ring against rank 0 stepping the whole torus
    H, W, psteps = 64, 48, 3
    X0 = inputs.make_state(1, H, W, seed=8, scale=0.45 * H * W)
    pw = inputs.make_weight_sets(1, seed=8)
    small = sharding.StripedGrid(H, W, pw, dtype=dt_code, device=local)
    small.load(X0[:, small.first_row:small.first_row + small.n_rows])
    small.step(psteps)
    small.handle.ring_wait(60000)
    mine = torch.from_numpy(small.read()).cuda()
    small.close()
    if world > 1:
        parts = [torch.empty_like(mine) for _ in range(world)] if rank == 0 else None
        dist.gather(mine, parts, dst=0)
    else:
        parts = [mine]
    if rank == 0:
        with capi.Handle(1, H, W, dtype=dt_code, device=local) as whole:
            whole.set_weights(pw); whole.set_state(X0); whole.step(psteps)
            ref = whole.get_state()
        got = torch.cat(parts, dim=1).cpu().numpy()
        out["stripe_parity_rel_l2"] = float(np.linalg.norm(got.astype(np.float64) - ref) / np.linalg.norm(ref))
        out["stripe_parity_case"] = f"{H}x{W} torus, {psteps} steps, {world} stripe(s) vs the whole torus on rank 0"
    # the full-size torus
    grid, mass = workloads.random_striped_grid(edge, args.dtype, rank, world, local, weights)
    grid.step(2)
    ms = timed(lambda: grid.step(steps), 1)
    split = grid.handle.step_ring_timed(steps)
    if world > 1:
        t = torch.tensor(split, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        split = [float(v) for v in t.tolist()]
    err = workloads.striped_mass_error(grid, mass)
    grid.close()
    out.update({"cell_updates_per_s": edge * edge * steps / (ms * 1e-3), "ms_per_step": ms / steps,
                "ms_halo": split[0] / steps, "ms_kernels": split[1] / steps, "ms_allreduce": split[2] / steps,
                "max_mass_error": err, "steps_before_mass_check": 2 + 2 * steps})
    return out


if __name__ == "__main__":
    main()
