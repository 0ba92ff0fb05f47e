"""Host-side mirror of the reference's pseudopod interfaces over the C ABI.

Names and meanings follow the protocol structs of J0pari/Slime:
  ModelProtocol      forward(input, output), effective_rank(), coherence()        slime/proto/model.cu:5-14
  ComponentProtocol  id, fitness, coherence, hunger, reset(), compute_fitness()  slime/proto/component.cu:5-15
and the planned Organism forward(stimulus, state, output) (BLUEPRINT.md:202).  The C++ adapters with the same
names live in csrc/slime_pseudopod.hpp; this Python class is what the tests and the bench drive.
"""
from __future__ import annotations

import numpy as np

from . import capi


class Pseudopod:
    """A population of CA grids sharing `n_weight_sets` learned update rules, stepped on one GPU."""

    def __init__(self, batch, height, width, weights, *, dtype=capi.F32, dt=0.1, device=0, component_id=0,
                 keep_vprime=True):
        self.id = component_id
        self.fitness = 0.0
        self._coherence = 0.0
        self._rank = 0.0
        self.hunger = 1.0
        self.handle = capi.Handle(batch, height, width, n_weight_sets=weights.n_sets, dtype=dtype, dt=dt,
                                  device=device, keep_vprime=keep_vprime)
        self.handle.set_weights(weights)
        self._steps = 0

    # ModelProtocol ----------------------------------------------------------------------------------
    def forward(self, state: np.ndarray, n_steps: int = 1) -> np.ndarray:
        """input state [B,H,W,64] -> state after n_steps CA steps (the reference's forward(input, output))."""
        self.handle.set_state(state)
        self.handle.step(n_steps)
        self._steps = n_steps
        return self.handle.get_state()

    def effective_rank(self) -> float:
        return float(self._rank)

    def coherence(self) -> float:
        return float(self._coherence)

    # ComponentProtocol ------------------------------------------------------------------------------
    def reset(self):
        self.fitness, self._coherence, self._rank, self.hunger, self._steps = 0.0, 0.0, 0.0, 1.0, 0

    def compute_fitness(self) -> float:
        """effective_rank x coherence over the last two steps, averaged over the population."""
        f = self.handle.fitness()
        self.per_grid = f
        self._rank = float(f["rank"].mean())
        self._coherence = float(f["coherence"].mean())
        self.fitness = float(f["fitness"].mean())
        self.hunger = float(f["hunger"].mean())
        return self.fitness

    def to_dict(self) -> dict:
        return {"id": self.id, "fitness": self.fitness, "coherence": self._coherence,
                "effective_rank": self._rank, "hunger": self.hunger}

    def from_dict(self, d: dict):
        self.id = int(d["id"]); self.fitness = float(d["fitness"]); self._coherence = float(d["coherence"])
        self._rank = float(d["effective_rank"]); self.hunger = float(d["hunger"])

    def close(self):
        self.handle.close()
