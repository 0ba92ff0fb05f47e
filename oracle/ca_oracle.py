"""ctypes loader for the CPU oracle (oracle/ca_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the bench's CPU-baseline legs;
the product package never imports this module.  `real="f64"` is the truth used for parity checks,
`real="f32"` is the multithreaded fp32 transcription that gets timed.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBS: dict = {}

_F = ctypes.POINTER(ctypes.c_float)
_D = ctypes.POINTER(ctypes.c_double)


def build() -> None:
    """Compile both oracle libraries beside the source (gcc + OpenMP)."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)


def _lib(real: str):
    if real not in ("f32", "f64"):
        raise ValueError(real)
    if real not in _LIBS:
        path = os.path.join(_HERE, f"libca_oracle_{real}.so")
        src = os.path.join(_HERE, "ca_oracle.c")
        if not os.path.exists(path) or (os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(path)):
            build()
        lib = ctypes.CDLL(path)
        lib.oracle_ca_steps.restype = ctypes.c_int
        lib.oracle_ca_steps.argtypes = [_F, _D, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        _F, _F, _F, _F, _F, _F, _F, ctypes.c_int,
                                        ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_int, _F, _F]
        lib.oracle_fitness.restype = ctypes.c_int
        lib.oracle_fitness.argtypes = [_F, _F, ctypes.c_int, ctypes.c_int, _F, _F, _F, _F, _F]
        lib.oracle_jacobi_eigenvalues.restype = ctypes.c_int
        lib.oracle_jacobi_eigenvalues.argtypes = [_D, ctypes.c_int, _D]
        lib.oracle_entropy_rank.restype = ctypes.c_double
        lib.oracle_entropy_rank.argtypes = [_D, ctypes.c_int]
        lib.oracle_channel_mass.restype = None
        lib.oracle_channel_mass.argtypes = [_F, ctypes.c_int, ctypes.c_int, ctypes.c_int, _D]
        lib.oracle_lift.restype = None
        lib.oracle_lift.argtypes = [_F, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, _F, _F]
        lib.oracle_pool_readout.restype = None
        lib.oracle_pool_readout.argtypes = [_F, ctypes.c_int, ctypes.c_int, _F, _F, ctypes.c_int, _F]
        lib.oracle_field_from_state.restype = None
        lib.oracle_field_from_state.argtypes = [_F, ctypes.c_int, ctypes.c_int, _F]
        lib.oracle_weights_from_reference_layout.restype = None
        lib.oracle_weights_from_reference_layout.argtypes = [_F] * 10
        lib.oracle_set_activation_clamp.restype = ctypes.c_double
        lib.oracle_set_activation_clamp.argtypes = [ctypes.c_double]
        lib.oracle_genome_hash.restype = ctypes.c_ulonglong
        lib.oracle_genome_hash.argtypes = [_F, ctypes.c_ulonglong]
        lib.oracle_set_threads.restype = ctypes.c_int
        lib.oracle_set_threads.argtypes = [ctypes.c_int]
        lib.oracle_evolve.restype = ctypes.c_int
        lib.oracle_evolve.argtypes = [_F, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float, ctypes.c_float,
                                      ctypes.c_float, ctypes.c_ulonglong, ctypes.c_int, _F, _F, _F, _F,
                                      ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        _LIBS[real] = lib
    return _LIBS[real]


def _f(a):
    return None if a is None else a.ctypes.data_as(_F)


def _c32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def ca_steps(X, weights, n_steps, *, dt=0.1, mass=None, literal=True, renorm=True, want_vprime=False, real="f64"):
    """Run n_steps on X[B,H,W,64]; returns the new state (and V' of the last two steps if asked).

    `weights` is any object with arrays() -> (Wp, Wi, Wv, Wo, K, mu, sigma) concatenated over sets.
    """
    X = _c32(X).copy()
    B, H, W, C = X.shape
    assert C == 64
    arrs = [_c32(a) for a in weights.arrays()]
    n_sets = arrs[0].shape[0]
    vp_prev = vp_last = None
    if want_vprime:
        vp_prev = np.zeros((B, H, W, 512), np.float32)
        vp_last = np.zeros((B, H, W, 512), np.float32)
    m = None
    if mass is not None:
        m = np.ascontiguousarray(mass, dtype=np.float64)
        assert m.shape == (B, 64)
    rc = _lib(real).oracle_ca_steps(
        _f(X), None if m is None else m.ctypes.data_as(_D), B, H, W,
        *[_f(a) for a in arrs], n_sets, int(n_steps), float(dt), int(bool(literal)), int(bool(renorm)),
        _f(vp_prev), _f(vp_last))
    if rc != 0:
        raise RuntimeError(f"oracle_ca_steps failed ({rc})")
    return (X, vp_prev, vp_last) if want_vprime else X


def fitness(vp_prev, vp_last, real="f64"):
    """-> dict(rank[B], coherence[B], fitness[B], hunger[B], head_rank[B,8]) from V' of the last two steps."""
    a, b = _c32(vp_prev), _c32(vp_last)
    B = a.shape[0]
    cells = int(np.prod(a.shape[1:-1]))
    assert a.shape[-1] == 512 and a.shape == b.shape
    out = {k: np.zeros(B, np.float32) for k in ("rank", "coherence", "fitness", "hunger")}
    out["head_rank"] = np.zeros((B, 8), np.float32)
    rc = _lib(real).oracle_fitness(_f(a), _f(b), B, cells, _f(out["rank"]), _f(out["coherence"]),
                                   _f(out["fitness"]), _f(out["hunger"]), _f(out["head_rank"]))
    if rc != 0:
        raise RuntimeError("oracle_fitness failed")
    return out


def jacobi_eigenvalues(A):
    A = np.ascontiguousarray(A, dtype=np.float64).copy()
    n = A.shape[0]
    eig = np.zeros(n, np.float64)
    sweeps = _lib("f64").oracle_jacobi_eigenvalues(A.ctypes.data_as(_D), n, eig.ctypes.data_as(_D))
    return eig, sweeps


def entropy_rank(eig):
    e = np.ascontiguousarray(eig, dtype=np.float64)
    return float(_lib("f64").oracle_entropy_rank(e.ctypes.data_as(_D), e.shape[0]))


def channel_mass(X):
    X = _c32(X)
    B, H, W, _ = X.shape
    m = np.zeros((B, 64), np.float64)
    _lib("f64").oracle_channel_mass(_f(X), B, H, W, m.ctypes.data_as(_D))
    return m


def lift(img, L, pad):
    img = _c32(img)
    B, h, w = img.shape
    X = np.zeros((B, h + 2 * pad, w + 2 * pad, 64), np.float32)
    _lib("f64").oracle_lift(_f(img), B, h, w, pad, _f(_c32(L)), _f(X))
    return X


def pool_readout(X, Wr, br):
    X = _c32(X)
    B = X.shape[0]
    cells = int(np.prod(X.shape[1:-1]))
    Wr = _c32(Wr)
    n_out = Wr.shape[1]
    out = np.zeros((B, n_out), np.float32)
    _lib("f64").oracle_pool_readout(_f(X), B, cells, _f(Wr), _f(None if br is None else _c32(br)), n_out, _f(out))
    return out


def field_from_state(X):
    """field[b, y, x] = mean over channels of X[b, y, x, :]."""
    X = _c32(X)
    out = np.zeros(X.shape[:-1], np.float32)
    _lib("f64").oracle_field_from_state(_f(X), X.shape[0], int(np.prod(X.shape[1:-1])), _f(out))
    return out


def weights_from_reference_layout(perception, interaction, value, mixing, flow):
    """Contract weight arrays (Wp, Wi, Wv, Wo, K) from the reference's bundle layouts
    ([8][512][256], [8][512][256], [8][256][512], [8][8], [8][9])."""
    Wp = np.zeros((8, 64, 64), np.float32); Wi = np.zeros_like(Wp); Wv = np.zeros_like(Wp)
    Wo = np.zeros((512, 64), np.float32); K = np.zeros((8, 9), np.float32)
    _lib("f64").oracle_weights_from_reference_layout(_f(_c32(perception)), _f(_c32(interaction)), _f(_c32(value)),
                                                    _f(_c32(mixing)), _f(_c32(flow)), _f(Wp), _f(Wi), _f(Wv), _f(Wo), _f(K))
    return Wp, Wi, Wv, Wo, K


def evolve(fit, weights, per_set, *, fitness_threshold, hunger_threshold, mutation_rate, mutation_sigma, seed,
           generation):
    """The population step.  fit: [n_grids, 4] = rank, coherence, fitness, hunger per grid; weights: an object with
    arrays() -> (Wp, Wi, Wv, Wo, K, mu, sigma) stacked over sets.  Returns (new arrays tuple, parent, best, n_replaced)."""
    Wp, Wi, Wv, Wo, K, mu, sigma = [np.array(a, dtype=np.float32, order="C", copy=True) for a in weights.arrays()]
    n_sets = Wp.shape[0]
    fit = _c32(fit)
    assert fit.shape == (n_sets * per_set, 4)
    parent = np.zeros(n_sets, np.int32)
    best = ctypes.c_int(-1)
    n = _lib("f64").oracle_evolve(_f(fit), n_sets, per_set, fitness_threshold, hunger_threshold, mutation_rate,
                                  mutation_sigma, seed, generation, _f(Wp), _f(Wi), _f(Wv), _f(Wo),
                                  parent.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), ctypes.byref(best))
    K, mu, sigma = K[parent], mu[parent], sigma[parent]      # taps, mu and sigma are inherited unchanged
    return (Wp, Wi, Wv, Wo, K, mu, sigma), parent, best.value, n


def set_activation_clamp(c, real="f64"):
    """Set the bound on |A| = |G * I| of one build of the oracle (80 by default, as in the CUDA kernels);
    returns the previous bound.  Tests use a huge value to show where the clamp starts to act."""
    return float(_lib(real).oracle_set_activation_clamp(float(c)))


def genome_hash(genome):
    """The reference's 64-bit genome hash over a flat fp32 array (bit patterns, in order)."""
    g = _c32(genome).reshape(-1)
    return int(_lib("f64").oracle_genome_hash(_f(g), g.size))


def usable_cpus():
    """CPUs this process may really use: the affinity mask, capped by the cgroup CPU quota when there is one."""
    import math
    import os
    n = len(os.sched_getaffinity(0))
    try:
        quota, period = open("/sys/fs/cgroup/cpu.max").read().split()
        if quota != "max":
            n = max(1, min(n, math.ceil(int(quota) / int(period))))
    except (OSError, ValueError):
        pass
    return n


def set_threads(n, real="f32"):
    """Set the OpenMP thread count of one build of the oracle; returns the count in force."""
    return int(_lib(real).oracle_set_threads(int(n)))
