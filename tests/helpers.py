"""Shared helpers for the parity tests."""
import hashlib
import os

import numpy as np

from slime_b200 import inputs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
GOLDEN_CASES = ("ragged_5x7", "torus_4x4", "unit_mass_8x8")


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


def load_golden(name):
    """-> (fixture dict, WeightSets regenerated from the stored seed and checked against the stored digest)."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    w = inputs.make_weight_sets(int(z["n_sets"]), seed=int(z["seed"]))
    h = hashlib.sha256()
    for a in w.arrays():
        h.update(np.ascontiguousarray(a, dtype=np.float32).tobytes())
    assert h.hexdigest() == str(z["weights_sha256"]), "weight generator no longer reproduces the fixture's weights"
    return z, w


def channel_mass(X):
    X = np.asarray(X, np.float64)
    return X.reshape(X.shape[0], -1, X.shape[-1]).sum(axis=1)


def bf16_round(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()


def bf16_storage_floor(X0, w, steps, truth):
    """Relative L2 distance from `truth` (the fp64 oracle after `steps` steps) of the same oracle when nothing but the
    state is rounded to bf16 after every step: what bf16 storage of the state alone costs over that many steps,
    whatever the arithmetic in between.  A bf16 kernel can not be expected to come closer than this."""
    from oracle import ca_oracle
    X = bf16_round(X0)
    mass = ca_oracle.channel_mass(X)
    for _ in range(steps):
        X = bf16_round(ca_oracle.ca_steps(X, w, 1, literal=False, mass=mass))
    return rel_l2(X, truth)
