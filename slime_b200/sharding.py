"""Multi-GPU partitioning of the CA workloads: one process per GPU, torch.distributed for the plumbing.

Two ways the path shards:
  * populations of independent grids (and their weight sets) split into contiguous ranges per rank, with no
    collective on the data path (`shard_population`);
  * one large torus split into row stripes: every step each rank sends its 3 top and 3 bottom own rows to its
    ring neighbours (the step's dependency radius is 3: stencil 1 + softmax denominator 1 + gather 1) and the
    64 per-channel sums are all-reduced for the global mass renormalisation.  On GPUs the ring lives inside the C
    library (slime_ca_step_ring: grouped ncclSend / ncclRecv and ncclAllReduce on the caller's stream, no host
    synchronisation per step) and `StripedGrid` only sets it up; `StripeRing` is the same exchange over any
    torch.distributed backend, which is what the CPU tests drive over gloo, with a deadline on every wait.
    Halo rows land in the receiver's own state buffer first; kernels only ever read local memory.

The reference has no multi-GPU code (one line of intent: BLUEPRINT.md:444-447, device = hash % num_gpus).
"""
from __future__ import annotations

import datetime
import time
from dataclasses import dataclass

import torch
import torch.distributed as dist

HALO = 3    # halo rows of the state on each side of a stripe (must match the C library's stripe mode)


@dataclass(frozen=True)
class PopulationShard:
    first_grid: int
    n_grids: int
    first_set: int
    n_sets: int


def shard_population(n_grids: int, n_sets: int, rank: int, world: int) -> PopulationShard:
    """Contiguous range of grids and of weight sets for `rank`.  Grid b uses set b // (n_grids // n_sets), so the
    split keeps every grid on the rank that holds its weight set."""
    if n_grids % n_sets != 0:
        raise ValueError("n_sets must divide n_grids")
    if n_sets % world != 0:
        if n_sets != 1 or n_grids % world != 0:
            raise ValueError(f"cannot split {n_sets} weight sets / {n_grids} grids over {world} ranks")
        per = n_grids // world          # one shared set: replicate it, split the grids
        return PopulationShard(rank * per, per, 0, 1)
    sets = n_sets // world
    per_set = n_grids // n_sets
    return PopulationShard(rank * sets * per_set, sets * per_set, rank * sets, sets)


def stripe_rows(height: int, rank: int, world: int):
    """(first_row, n_rows) of the row stripe `rank` owns; the height must split evenly and leave >= HALO rows."""
    if height % world != 0:
        raise ValueError(f"{height} rows do not split evenly over {world} ranks")
    n = height // world
    if n < HALO:
        raise ValueError(f"stripes of {n} rows are thinner than the {HALO}-row halo")
    return rank * n, n


class RingTimeout(RuntimeError):
    """A neighbour's halo rows (or the sum reduction) did not arrive within the ring's deadline."""


class StripeRing:
    """Halo exchange and sum reduction for one stripe per rank, ranks forming a ring in y (toroidal wrap).
    Every wait is bounded by `timeout_s`: a neighbour that never sends raises RingTimeout instead of blocking
    the rank for ever."""

    def __init__(self, group=None, timeout_s: float = 60.0):
        self.group = group
        self.timeout_s = float(timeout_s)
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.up = (self.rank - 1) % self.world        # owner of the rows above mine
        self.down = (self.rank + 1) % self.world

    def exchange_halos(self, state: torch.Tensor, n_rows: int) -> None:
        """state: [B][n_rows + 2*HALO][W][64] (any device).  Fills the halo rows from the ring neighbours' own
        rows: top halo <- last HALO own rows of `up`, bottom halo <- first HALO own rows of `down`."""
        top_own = state[:, HALO:2 * HALO]
        bot_own = state[:, n_rows:n_rows + HALO]
        top_halo = state[:, 0:HALO]
        bot_halo = state[:, n_rows + HALO:n_rows + 2 * HALO]
        if self.world == 1:
            top_halo.copy_(bot_own)
            bot_halo.copy_(top_own)
            return
        send_up, send_down = top_own.contiguous(), bot_own.contiguous()
        recv_top, recv_bot = torch.empty_like(send_up), torch.empty_like(send_down)
        ops = [dist.P2POp(dist.isend, send_up, self.up, self.group, tag=1),
               dist.P2POp(dist.isend, send_down, self.down, self.group, tag=2),
               dist.P2POp(dist.irecv, recv_top, self.up, self.group, tag=2),
               dist.P2POp(dist.irecv, recv_bot, self.down, self.group, tag=1)]
        if self.world == 2 and self.rank == 1:      # pair the operations in the same order on both ranks
            ops = [ops[1], ops[0], ops[3], ops[2]]
        self._wait_all(dist.batch_isend_irecv(ops), "halo rows")
        top_halo.copy_(recv_top)
        bot_halo.copy_(recv_bot)

    def _wait_all(self, reqs, what: str) -> None:
        deadline = time.monotonic() + self.timeout_s
        for i, r in enumerate(reqs):
            left = max(deadline - time.monotonic(), 1e-3)
            try:
                ok = r.wait(datetime.timedelta(seconds=left))
            except RuntimeError as e:           # gloo reports an expired wait as a RuntimeError
                if "ime" not in str(e):         # "Timed out" / "timeout"
                    raise
                ok = False
            if ok is False:
                raise RingTimeout(f"rank {self.rank}: {len(reqs) - i} transfer(s) of {what} still pending after "
                                  f"{self.timeout_s:g} s (neighbours {self.up}, {self.down})")

    def allreduce_sums(self, sums: torch.Tensor) -> None:
        """In-place sum over ranks of the [B][64] fp64 per-channel sums."""
        if self.world > 1:
            self._wait_all([dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=self.group, async_op=True)], "channel sums")


class StripedGrid:
    """One large torus [1][H][W][64] stepped as row stripes, one per rank (GPU).

    `library_ring=True` (the default) joins the C library's own NCCL ring: the id made on rank 0 is broadcast over
    `group`, and every step then runs inside slime_ca_step_ring with no host synchronisation.  `library_ring=False`
    drives the same step from Python (StripeRing over torch.distributed around step_partial / step_finish)."""

    def __init__(self, height, width, weights, *, dtype, device, group=None, dt=0.1, library_ring=True):
        from . import capi, devmem
        self.ring = StripeRing(group)
        self.first_row, self.n_rows = stripe_rows(height, self.ring.rank, self.ring.world)
        self.handle = capi.Handle(1, self.n_rows, width, n_weight_sets=1, dtype=dtype, dt=dt, device=device, stripe=True)
        self.handle.set_weights(weights)
        self.state = devmem.state_view(self.handle)
        self.sums = devmem.sums_view(self.handle)
        self.library_ring = bool(library_ring)
        if self.library_ring:
            ring_id = None
            if self.ring.world > 1:
                box = [capi.ring_unique_id() if self.ring.rank == 0 else None]
                dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
                ring_id = box[0]
            self.handle.ring_init(ring_id, self.ring.rank, self.ring.world)

    def load(self, stripe_state) -> None:
        """stripe_state: this rank's own rows [1][n_rows][W][64] (host fp32); target masses are global sums."""
        self.handle.set_state(stripe_state)
        self.adopt_masses()

    def adopt_masses(self) -> None:
        """Make the target masses those of the whole torus (sum over the ranks of what each stripe recorded)."""
        if self.library_ring:
            self.handle.ring_sync_mass()
            torch.cuda.synchronize()
            return
        mass = torch.from_numpy(self.handle.get_mass()).to(self.sums.device)
        self.ring.allreduce_sums(mass)
        self.handle.set_mass(mass.cpu().numpy())

    def step(self, n_steps: int = 1, stream: int = 0) -> None:
        if self.library_ring:
            self.handle.step_ring(n_steps, stream)
            return
        for _ in range(n_steps):
            self.ring.exchange_halos(self.state, self.n_rows)
            self.handle.step_partial(stream)
            self.ring.allreduce_sums(self.sums)
            self.handle.step_finish(stream)

    def read(self):
        return self.handle.get_state()

    def close(self):
        self.handle.close()
