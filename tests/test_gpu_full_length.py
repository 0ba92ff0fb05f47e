"""GPU parity at the step counts the workloads specify, through the C ABI, against the fp64 CPU oracle:
the training-shape forward (64 steps), the row-stripe split of one torus (100 steps, two stripes) and the
supervised-input shape (24 steps and the pooled read-out), each in fp32 and in bf16.

Weights: the mass-neutral variant of the specified draws (inputs.mass_neutral).  With the plain draws the
trajectory grows 1.38x per step (tests/test_oracle.py pins that) and nothing can be compared past a few dozen steps.

Tolerances: fp32 1e-5 relative L2, per-channel mass 1e-6, fitness scalars 1e-4.  bf16: 2e-2 relative L2 where
bf16 storage of the state allows it; storing the state in bf16 after every step costs by itself about 1e-2 after
24 steps and up to 3e-2 after 100 (bf16_storage_floor measures it on the same inputs), so the bound is
max(2e-2, 1.5 x that floor); mass 1e-6 on the fp32 read-back, rank 5e-2 relative, coherence 2e-2.
"""
import numpy as np
import pytest

from slime_b200 import inputs
from tests.helpers import bf16_round, bf16_storage_floor, channel_mass, rel_l2

pytestmark = pytest.mark.gpu

TOL_F32, TOL_BF16, TOL_MASS = 1e-5, 2e-2, 1e-6


@pytest.fixture(scope="module")
def gpu():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from slime_b200 import capi, devmem
    capi.lib()
    return capi, devmem


_TRUTH = {}


def truth(key, fn):
    """The oracle's result for one case, computed once for both dtypes."""
    if key not in _TRUTH:
        _TRUTH[key] = fn()
    return _TRUTH[key]


def state_tolerance(dtype_name, X0, w, steps, truth):
    if dtype_name == "f32":
        return TOL_F32
    return max(TOL_BF16, 1.5 * bf16_storage_floor(X0, w, steps, truth))


def check_mass(dtype_name, X0, X1):
    m0 = channel_mass(X0 if dtype_name == "f32" else bf16_round(X0))
    assert np.max(np.abs(channel_mass(X1) - m0) / np.abs(m0)) < TOL_MASS


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_training_shape_forward_64_steps(gpu, dtype_name):
    """Two grids of the 64-grid training batch, all 64 CA steps, then the fitness of the last two steps."""
    from oracle import ca_oracle
    capi, devmem = gpu
    steps = 64
    X0 = inputs.make_state(2, 128, 128, seed=42)
    w = inputs.make_weight_sets(1, seed=42, bounded=True)
    R1, rprev, rlast = truth("forward", lambda: ca_oracle.ca_steps(X0, w, steps, literal=False, want_vprime=True))
    assert np.isfinite(R1).all()
    with capi.Handle(2, 128, 128, dtype=capi.F32 if dtype_name == "f32" else capi.BF16, keep_vprime=True) as h:
        h.set_weights(w)
        h.set_state(X0)
        h.step(steps)
        X1, fit = h.get_state(), h.fitness()
        vlast = devmem.vprime(h, capi.BUF_VPRIME_LAST)
    tol = state_tolerance(dtype_name, X0, w, steps, R1)
    assert np.isfinite(X1).all()
    assert rel_l2(X1, R1) < tol
    assert rel_l2(vlast, rlast) < tol
    check_mass(dtype_name, X0, X1)
    ref = ca_oracle.fitness(rprev, rlast)
    if dtype_name == "f32":
        for k in ("rank", "coherence", "fitness", "hunger"):
            np.testing.assert_allclose(fit[k], ref[k], atol=1e-4)
    else:
        np.testing.assert_allclose(fit["rank"], ref["rank"], rtol=5e-2)
        np.testing.assert_allclose(fit["coherence"], ref["coherence"], atol=2e-2)


def two_stripes(capi, devmem, X0, w, dtype, steps):
    """One torus stepped as two row stripes on one GPU: halo rows copied between the two handles' state buffers,
    the per-channel sums of both added, every step (what the ring does between GPUs)."""
    import torch
    _, H, W, _ = X0.shape
    n = H // 2
    parts = [capi.Handle(1, n, W, stripe=True, dtype=dtype) for _ in range(2)]
    mass = channel_mass(X0 if dtype == capi.F32 else bf16_round(X0))
    for r, p in enumerate(parts):
        p.set_weights(w)
        p.set_state(X0[:, r * n:(r + 1) * n])
        p.set_mass(mass)
    views = [devmem.state_view(p) for p in parts]
    sums = [devmem.sums_view(p) for p in parts]
    for _ in range(steps):
        for r in range(2):
            views[r][:, 0:3] = views[(r - 1) % 2][:, n:n + 3]
            views[r][:, n + 3:n + 6] = views[(r + 1) % 2][:, 3:6]
        torch.cuda.synchronize()
        for p in parts:
            p.step_partial()
        torch.cuda.synchronize()
        total = sums[0] + sums[1]
        for s in sums:
            s.copy_(total)
        for p in parts:
            p.step_finish()
    got = np.concatenate([p.get_state() for p in parts], axis=1)
    for p in parts:
        p.close()
    return got


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_row_stripes_100_steps(gpu, dtype_name):
    """The large-torus workload's step count on a 256 x 128 torus split into two row stripes."""
    from oracle import ca_oracle
    capi, devmem = gpu
    steps, H, W = 100, 256, 128
    X0 = inputs.make_state(1, H, W, seed=42)
    w = inputs.make_weight_sets(1, seed=42, bounded=True)
    R1 = truth("stripes", lambda: ca_oracle.ca_steps(X0, w, steps, literal=False))
    assert np.isfinite(R1).all()
    X1 = two_stripes(capi, devmem, X0, w, capi.F32 if dtype_name == "f32" else capi.BF16, steps)
    assert np.isfinite(X1).all()
    assert rel_l2(X1, R1) < state_tolerance(dtype_name, X0, w, steps, R1)
    check_mass(dtype_name, X0, X1)


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_supervised_shape_24_steps_and_readout(gpu, dtype_name):
    """Eight 28 x 28 images lifted to 32 x 32 x 64, 24 CA steps, mean-pool and the 64 -> 10 read-out.  The weights are
    mass-neutral for the lifted state's mass profile (channel masses proportional to the lift vector)."""
    from oracle import ca_oracle
    capi, devmem = gpu
    steps = 24
    L, Wr, br = inputs.make_lift_readout(seed=42)
    img = inputs.make_images(8, 28, seed=42)
    w = inputs.make_weight_sets(1, seed=42, bounded=True, mass_profile=L)
    X0 = ca_oracle.lift(img, L, 2)
    R1 = ca_oracle.ca_steps(X0, w, steps, literal=False)
    ref_logits = ca_oracle.pool_readout(R1, Wr, br)
    assert np.isfinite(ref_logits).all()
    with capi.Handle(8, 32, 32, dtype=capi.F32 if dtype_name == "f32" else capi.BF16) as h:
        h.set_weights(w)
        h.lift_images(img, L)
        h.step(steps)
        X1 = h.get_state()
        logits = h.pool_readout(Wr, br)
    assert np.isfinite(logits).all()
    assert rel_l2(X1, R1) < state_tolerance(dtype_name, X0, w, steps, R1)
    check_mass(dtype_name, X0, X1)
    np.testing.assert_allclose(logits, ref_logits, atol=1e-5 if dtype_name == "f32" else 5e-3)


def test_activation_beyond_the_clamp_is_the_same_function_everywhere(gpu):
    """With the interaction weights scaled up |G I| passes 80: the oracle, the fp32 kernels and the bf16 kernels all
    clamp the activation there and agree; the oracle with its clamp lifted does not."""
    from oracle import ca_oracle
    capi, devmem = gpu
    X0 = inputs.make_state(2, 16, 32, seed=3, scale=0.45 * 16 * 32)
    w = inputs.make_weight_sets(1, seed=3)
    w.Wi *= 4000.0
    ref = ca_oracle.ca_steps(X0, w, 1, literal=True)
    old = ca_oracle.set_activation_clamp(1e30)
    try:
        free = ca_oracle.ca_steps(X0, w, 1, literal=True)
    finally:
        ca_oracle.set_activation_clamp(old)
    assert rel_l2(free, ref) > 1e-4
    for dtype, tol in ((capi.F32, 1e-5), (capi.BF16, 2e-2)):
        with capi.Handle(2, 16, 32, dtype=dtype) as h:
            h.set_weights(w)
            h.set_state(X0)
            h.step(1)
            got = h.get_state()
        assert np.isfinite(got).all()
        assert rel_l2(got, ref) < tol


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_population_shape_32_steps_and_fitness(gpu, dtype_name):
    """The population workload's shape in small: 4 weight sets x 2 grids of 64 x 64, each set with its own seeded
    weights, all 32 steps, then the fitness of every grid from the last two steps."""
    from oracle import ca_oracle
    capi, devmem = gpu
    steps, n_sets, per = 32, 4, 2
    X0 = inputs.make_state(n_sets * per, 64, 64, seed=42)
    w = inputs.make_weight_sets(n_sets, seed=42, bounded=True)
    R1, rprev, rlast = truth("population", lambda: ca_oracle.ca_steps(X0, w, steps, literal=False, want_vprime=True))
    with capi.Handle(n_sets * per, 64, 64, n_weight_sets=n_sets, dtype=capi.F32 if dtype_name == "f32" else capi.BF16,
                     keep_vprime=True) as h:
        h.set_weights(w)
        h.set_state(X0)
        h.step(steps)
        X1, fit = h.get_state(), h.fitness()
    assert np.isfinite(X1).all()
    assert rel_l2(X1, R1) < state_tolerance(dtype_name, X0, w, steps, R1)
    check_mass(dtype_name, X0, X1)
    ref = ca_oracle.fitness(rprev, rlast)
    if dtype_name == "f32":
        for k in ("rank", "coherence", "fitness", "hunger"):
            np.testing.assert_allclose(fit[k], ref[k], atol=1e-4)
    else:
        np.testing.assert_allclose(fit["rank"], ref["rank"], rtol=5e-2)
        np.testing.assert_allclose(fit["coherence"], ref["coherence"], atol=2e-2)
    assert len(set(np.round(ref["rank"], 3))) > 1          # different weight sets, different ranks: the grouping matters
