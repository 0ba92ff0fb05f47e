"""Seeded synthetic inputs for the CA step: states, weight sets, images.

Everything is drawn from a counter-based generator written here (splitmix64 over seed/stream/counter),
so the same call gives the same bits on every machine and the oracle and the CUDA path can be fed
identical arrays.  The reference draws its weights on the GPU with curand
(slime/core/pseudopod.cu:386-444: `curand_init(seed, tid, 0)`, Xavier-like scales); that stream is
GPU-only and order dependent and is deliberately not reproduced.

Shapes and distributions follow the workload list this library is measured on:
  state   X[B,H,W,64] ~ U[0,1), every (grid, channel) divided by its sum over space (mass 1)
  weights per set: Wp, Wi, Wv [8,64,64] ~ N(0, 1/64) in the reference's [head][c_in][d_out] order,
          Wo [512,64] ~ N(0, 1/512), K [8,9] ~ N(0, 1/3) then softmax over the 9 taps,
          mu [8] ~ U(0.1, 0.3), sigma [8] ~ U(0.01, 0.05)
  images  [B,28,28]: each pixel 0 with probability 0.7, else U(0,1)
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

NUM_HEADS = 8      # slime/core/pseudopod.cu:15
HEAD_DIM = 64      # slime/core/pseudopod.cu:16
CHANNELS = 64      # channels of the CA state the step reads and writes
HC = NUM_HEADS * HEAD_DIM

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser on uint64 arrays (wrapping arithmetic)."""
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = x
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def _stream_key(seed: int, stream: int) -> np.uint64:
    k = _splitmix64(np.array([seed & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64))
    k = _splitmix64(k ^ np.uint64(stream & 0xFFFFFFFFFFFFFFFF))
    return k[0]


def uniform(seed: int, stream: int, n: int, offset: int = 0) -> np.ndarray:
    """n doubles in [0,1): element i depends only on (seed, stream, offset+i)."""
    key = _stream_key(seed, stream)
    ctr = np.arange(offset, offset + n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        bits = _splitmix64(key ^ (ctr * np.uint64(0xD1342543DE82EF95) & _M64))
    return (bits >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def normal(seed: int, stream: int, n: int) -> np.ndarray:
    """n standard normals (Box-Muller on pairs of the uniform stream), float64."""
    m = (n + 1) // 2
    u = uniform(seed, stream, 2 * m)
    u1 = 1.0 - u[0::2]          # (0,1]
    u2 = u[1::2]
    r = np.sqrt(-2.0 * np.log(u1))
    out = np.empty(2 * m, dtype=np.float64)
    out[0::2] = r * np.cos(2.0 * np.pi * u2)
    out[1::2] = r * np.sin(2.0 * np.pi * u2)
    return out[:n]


# stream ids: one sub-stream per tensor, so shapes can change without shifting the others
_S_STATE, _S_WP, _S_WI, _S_WV, _S_WO, _S_K, _S_MU, _S_SIGMA = 1, 2, 3, 4, 5, 6, 7, 8
_S_IMG_MASK, _S_IMG_VAL, _S_LIFT, _S_READ_W, _S_READ_B = 9, 10, 11, 12, 13


@dataclass
class WeightSets:
    """n_sets weight sets, host fp32, concatenated over sets (the layout the C-ABI and the oracle take)."""
    Wp: np.ndarray      # [n_sets, 8, 64, 64]
    Wi: np.ndarray
    Wv: np.ndarray
    Wo: np.ndarray      # [n_sets, 512, 64]
    K: np.ndarray       # [n_sets, 8, 9]
    mu: np.ndarray      # [n_sets, 8]
    sigma: np.ndarray   # [n_sets, 8]

    @property
    def n_sets(self) -> int:
        return self.Wp.shape[0]

    def arrays(self):
        return (self.Wp, self.Wi, self.Wv, self.Wo, self.K, self.mu, self.sigma)


def make_state(batch: int, height: int, width: int, seed: int = 42, scale: float = 1.0,
               first_grid: int = 0) -> np.ndarray:
    """X[batch,H,W,64] fp32: U[0,1), each (grid, channel) normalised to unit mass, times `scale`.

    `first_grid` offsets the counter so that a rank holding grids [first_grid, first_grid+batch) of a
    larger population draws exactly the slice the whole population would contain.
    `scale` > 1 (about 3000 for 128x128 grids) moves the stencil output into the bell of the growth
    function; with unit mass the growth saturates at -1 and the nonlinear stages are not exercised.
    """
    per = height * width * CHANNELS
    x = uniform(seed, _S_STATE, batch * per, offset=first_grid * per).reshape(batch, height * width, CHANNELS)
    x = x / x.sum(axis=1, keepdims=True)
    return (x * scale).astype(np.float32).reshape(batch, height, width, CHANNELS)


def make_weight_sets(n_sets: int = 1, seed: int = 42, first_set: int = 0, bounded: bool = False,
                     mass_profile=None) -> WeightSets:
    """Weight set s is drawn from seed + first_set + s, so a population can be generated shard by shard.

    `bounded=True` returns the mass-neutral variant of the same draws (see `mass_neutral`): the one used
    wherever a trajectory has to stay finite over many steps.
    """
    Wp, Wi, Wv, Wo, K, mu, sg = [], [], [], [], [], [], []
    n = NUM_HEADS * CHANNELS * HEAD_DIM
    for s in range(n_sets):
        sd = seed + first_set + s
        Wp.append((normal(sd, _S_WP, n) / 8.0).reshape(NUM_HEADS, CHANNELS, HEAD_DIM))
        Wi.append((normal(sd, _S_WI, n) / 8.0).reshape(NUM_HEADS, CHANNELS, HEAD_DIM))
        Wv.append((normal(sd, _S_WV, n) / 8.0).reshape(NUM_HEADS, CHANNELS, HEAD_DIM))
        Wo.append((normal(sd, _S_WO, HC * CHANNELS) / np.sqrt(512.0)).reshape(HC, CHANNELS))
        k = (normal(sd, _S_K, NUM_HEADS * 9) / np.sqrt(3.0)).reshape(NUM_HEADS, 9)
        k = np.exp(k - k.max(axis=1, keepdims=True))
        K.append(k / k.sum(axis=1, keepdims=True))
        mu.append(0.1 + 0.2 * uniform(sd, _S_MU, NUM_HEADS))
        sg.append(0.01 + 0.04 * uniform(sd, _S_SIGMA, NUM_HEADS))
    f = lambda a: np.ascontiguousarray(np.stack(a).astype(np.float32))
    w = WeightSets(f(Wp), f(Wi), f(Wv), f(Wo), f(K), f(mu), f(sg))
    return mass_neutral(w, mass_profile) if bounded else w


def mass_neutral(w: WeightSets, mass_profile=None) -> WeightSets:
    """The same weight sets with every output projection made mass-neutral for states whose per-channel
    masses are proportional to `mass_profile` ([64], default all ones).

    Why: one step adds dt * Y to the state and the redistribution conserves the value per (head, dim), so the
    per-channel sums move by dt * m^T (sum_h Wv_h Wo_h) for channel masses m.  With the plain draws that is
    about +-0.1 per unit mass and step; the renormalisation then multiplies channel c by 1 / (1 + 0.1 a_c)
    every step, and the channel with the most negative a_c has its zero-mean part amplified by about 1.3-1.4
    per step until the state overflows (around step 50 in fp32 and fp64 alike).  Removing from Wo its
    component along a = m^T Wv (a rank-one change, Wo <- Wo - a (a^T Wo) / (a^T a)) makes the sums
    stationary: the renormalisation scale stays 1 and the remaining growth is the mild one of I + dt * M
    (about 1.08 per step), finite over the 64-, 100- and 24-step workloads.  Everything else (Wp, Wi, Wv, K,
    mu, sigma, and the part of Wo orthogonal to a) keeps the specified distributions.
    """
    m = np.ones(CHANNELS) if mass_profile is None else np.asarray(mass_profile, np.float64).reshape(CHANNELS)
    Wo = np.array(w.Wo, dtype=np.float64)
    for s in range(w.n_sets):
        a = np.einsum("c,hcd->hd", m, w.Wv[s].astype(np.float64)).reshape(HC)
        Wo[s] -= np.outer(a, a @ Wo[s]) / float(a @ a)
    return WeightSets(w.Wp, w.Wi, w.Wv, np.ascontiguousarray(Wo.astype(np.float32)), w.K, w.mu, w.sigma)


def make_images(batch: int, size: int = 28, seed: int = 42, first: int = 0) -> np.ndarray:
    """[batch,size,size] fp32: 70% zeros, 30% U(0,1) (shape and sparsity of handwritten-digit images)."""
    n = batch * size * size
    mask = uniform(seed, _S_IMG_MASK, n, offset=first * size * size) >= 0.7
    val = uniform(seed, _S_IMG_VAL, n, offset=first * size * size)
    return (mask * val).astype(np.float32).reshape(batch, size, size)


def make_lift_readout(seed: int = 42, n_out: int = 10):
    """Lift vector L[64] = 0.5 + |N(0,1)|/2, readout Wr[64,n_out] ~ N(0,1/64), bias br[n_out] ~ N(0,1)/10.

    The lift is kept positive: the step renormalises every channel to its initial mass, which is ill-posed
    (and diverges within a few steps) for a channel whose mass is near zero or of mixed sign.
    """
    L = (0.5 + 0.5 * np.abs(normal(seed, _S_LIFT, CHANNELS))).astype(np.float32)
    Wr = (normal(seed, _S_READ_W, CHANNELS * n_out) / 8.0).astype(np.float32).reshape(CHANNELS, n_out)
    br = (normal(seed, _S_READ_B, n_out) / 10.0).astype(np.float32)
    return L, Wr, br
