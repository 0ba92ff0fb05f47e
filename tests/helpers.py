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
