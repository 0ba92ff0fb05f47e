"""Generates the golden fixtures in this folder (run from the repo root: python tests/golden/make_golden.py).

The reference (J0pari/Slime) holds no golden vectors for the CA step and cannot be run as a numerical
oracle, so these fixtures come from a second, independently written restatement of the step: plain numpy,
fp64 throughout, stages 5-6 as a literal scatter (every source cell pushes softmax-weighted shares of its
value to its 3x3 neighbours).  They pin the C oracle (oracle/ca_oracle.c) and, through the GPU tests, the
CUDA path.  Nothing here shares code with the C oracle.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from slime_b200 import inputs  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
STATS: list = []          # fraction of growth values off the -1 plateau, per (grid, step, head)
TAPS = [(dy, dx) for dy in (-1, 0, 1) for dx in (-1, 0, 1)]   # t = (dy+1)*3 + (dx+1)


def shift(a, dy, dx):
    """b[y,x] = a[y+dy, x+dx] on the torus (axes 0,1)."""
    return np.roll(a, (-dy, -dx), axis=(0, 1))


def step_numpy(X, w, s, dt=0.1):
    """One step on one grid X[H,W,64] (fp64) with weight set s; returns (X_next_unnormalised, V'[H,W,512])."""
    H, W, _ = X.shape
    Y = np.zeros_like(X)
    vps = []
    for h in range(8):
        P = X @ w.Wp[s, h].astype(np.float64)
        I = X @ w.Wi[s, h].astype(np.float64)
        V = X @ w.Wv[s, h].astype(np.float64)
        U = sum(float(w.K[s, h, t]) * shift(P, dy, dx) for t, (dy, dx) in enumerate(TAPS))
        mu, sg = float(w.mu[s, h]), float(w.sigma[s, h])
        G = 2.0 * np.exp(-((U - mu) ** 2) / (2.0 * sg * sg)) - 1.0
        A = np.clip(G * I, -80.0, 80.0)      # the step's domain limit on the activation (inactive in these fixtures)
        STATS.append(float((G > -0.9).mean()))
        # scatter: source s sends V(s) * softmax over its 9 targets n of A(n)
        nbrA = np.stack([shift(A, dy, dx) for dy, dx in TAPS])          # A at the 9 targets of each source
        e = np.exp(nbrA - nbrA.max(axis=0, keepdims=True))
        share = e / e.sum(axis=0, keepdims=True)                         # [9,H,W,64], sums to 1 per source
        Vp = np.zeros_like(V)
        for t, (dy, dx) in enumerate(TAPS):
            # the share computed at source (y,x) for target (y+dy,x+dx) lands at that target
            Vp += shift(share[t] * V, -dy, -dx)
        vps.append(Vp)
        Y += Vp @ w.Wo[s, h * 64:(h + 1) * 64].astype(np.float64)
    return X + dt * Y, np.concatenate(vps, axis=-1)


def run_numpy(X0, w, n_steps, dt=0.1):
    B = X0.shape[0]
    per_set = B // w.n_sets
    out = np.zeros(X0.shape, np.float64)
    vprev = np.zeros(X0.shape[:3] + (512,), np.float64)
    vlast = np.zeros_like(vprev)
    for b in range(B):
        X = X0[b].astype(np.float64)
        M = X.sum(axis=(0, 1))
        for k in range(n_steps):
            X, vp = step_numpy(X, w, b // per_set, dt)
            X = X.astype(np.float32).astype(np.float64)          # the state is stored fp32
            X = X * (M / X.sum(axis=(0, 1)))
            X = X.astype(np.float32).astype(np.float64)
            if k == n_steps - 2:
                vprev[b] = vp
            if k == n_steps - 1:
                vlast[b] = vp
        out[b] = X
    return out, vprev, vlast


def fitness_numpy(vprev, vlast):
    B = vlast.shape[0]
    rank = np.zeros(B)
    coh = np.zeros(B)
    for b in range(B):
        F = vlast[b].astype(np.float32).astype(np.float64).reshape(-1, 8, 64)
        r = []
        for h in range(8):
            lam = np.clip(np.linalg.eigvalsh(F[:, h].T @ F[:, h]), 0.0, None)
            p = lam / (lam.sum() + 1e-7)
            r.append(np.exp(-(p * np.log(p + 1e-7)).sum()))
        rank[b] = np.mean(r)
        a = vprev[b].astype(np.float32).astype(np.float64).ravel()
        c = vlast[b].astype(np.float32).astype(np.float64).ravel()
        coh[b] = np.corrcoef(a, c)[0, 1]
    return rank, coh


def weights_digest(w) -> str:
    """The fixtures keep the weight seed, not the 0.5 MB per set of weights; this digest pins the generator."""
    h = hashlib.sha256()
    for a in w.arrays():
        h.update(np.ascontiguousarray(a, dtype=np.float32).tobytes())
    return h.hexdigest()


CASES = {
    # name: (B, H, W, n_sets, steps, scale, seed)
    "ragged_5x7": (2, 5, 7, 2, 3, 15.0, 7),       # non-square, odd sizes, two weight sets, bell exercised
    "torus_4x4": (1, 4, 4, 1, 2, 7.0, 11),       # every cell touches the wrap
    "unit_mass_8x8": (1, 8, 8, 1, 2, 1.0, 42),    # the saturated-growth regime of unit-mass states
}


def main():
    for name, (B, H, W, n_sets, steps, scale, seed) in CASES.items():
        X0 = inputs.make_state(B, H, W, seed=seed, scale=scale)
        w = inputs.make_weight_sets(n_sets, seed=seed)
        X1, vprev, vlast = run_numpy(X0, w, steps)
        rank, coh = fitness_numpy(vprev, vlast)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            X0=X0, n_sets=np.int32(n_sets), seed=np.int32(seed), weights_sha256=weights_digest(w),
            steps=np.int32(steps), X1=X1.astype(np.float32), vprev=vprev.astype(np.float32),
            vlast=vlast.astype(np.float32), rank=rank, coherence=coh)
        print(name, "rank", rank, "coherence", coh, "growth off-plateau fraction %.3f" % np.mean(STATS))
        STATS.clear()


if __name__ == "__main__":
    main()
