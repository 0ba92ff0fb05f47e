"""GPU parity tests of the bf16 tensor-core path (tcgen05 projections), through the C ABI, against the CPU oracle.

Tolerance of this path: 2e-2 relative L2 on the state and on the redistributed value V' against the fp64
oracle run on the same (unrounded) fp32 inputs.  The state moves by about a tenth of its size per step, so
the per-step increment is checked as well (looser: it sits only a few bf16 ulps above the storage rounding).
Mass is conserved to 1e-6 relative on the fp32 read-back (stored bf16 state times the fp32 scale).
"""
import numpy as np
import pytest

from slime_b200 import inputs
from tests.helpers import GOLDEN_CASES, channel_mass, load_golden, rel_l2

pytestmark = pytest.mark.gpu

TOL = 2e-2
TOL_INCREMENT = 0.15
TOL_MASS = 1e-6


@pytest.fixture(scope="module")
def gpu():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from slime_b200 import capi, devmem
    capi.lib()
    return capi, devmem


def bf16_round(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()


def run_bf16(capi, devmem, X0, w, steps):
    B, H, W, _ = X0.shape
    h = capi.Handle(B, H, W, n_weight_sets=w.n_sets, dtype=capi.BF16, keep_vprime=True)
    h.set_weights(w)
    h.set_state(X0)
    h.step(steps)
    X1 = h.get_state()
    out = (X1, devmem.vprime(h, capi.BUF_VPRIME_PREV), devmem.vprime(h, capi.BUF_VPRIME_LAST), h.fitness())
    h.close()
    return out


def check_against(X0, X1, vlast, R1, rlast):
    assert np.isfinite(X1).all()
    assert rel_l2(vlast, rlast) < TOL
    assert rel_l2(X1, R1) < TOL
    if np.linalg.norm(R1 - X0) > 1e-3 * np.linalg.norm(X0):     # a 1-cell grid can not move: its mass is pinned
        assert rel_l2(X1 - X0, R1 - X0) < TOL_INCREMENT
    m0, m1 = channel_mass(bf16_round(X0)), channel_mass(X1)
    assert np.max(np.abs(m1 - m0) / np.abs(m0)) < TOL_MASS


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_fixtures(gpu, name):
    capi, devmem = gpu
    z, w = load_golden(name)
    X1, vprev, vlast, fit = run_bf16(capi, devmem, z["X0"], w, int(z["steps"]))
    check_against(z["X0"], X1, vlast, z["X1"], z["vlast"])
    assert rel_l2(vprev, z["vprev"]) < TOL
    np.testing.assert_allclose(fit["rank"], z["rank"], rtol=5e-2)
    np.testing.assert_allclose(fit["coherence"], z["coherence"], atol=2e-2)


@pytest.mark.parametrize("scale", [1.0, 7000.0], ids=["unit_mass", "bell_exercised"])
def test_training_shape_grids(gpu, scale):
    """128x128 grids with the training-shape generators (a slice of the 64-grid batch), 4 steps."""
    from oracle import ca_oracle
    capi, devmem = gpu
    X0 = inputs.make_state(2, 128, 128, seed=42, scale=scale)
    w = inputs.make_weight_sets(1, seed=42)
    X1, vprev, vlast, fit = run_bf16(capi, devmem, X0, w, 4)
    R1, rprev, rlast = ca_oracle.ca_steps(X0, w, 4, literal=False, want_vprime=True)
    check_against(X0, X1, vlast, R1, rlast)
    ref = ca_oracle.fitness(rprev, rlast)
    np.testing.assert_allclose(fit["rank"], ref["rank"], rtol=5e-2)
    np.testing.assert_allclose(fit["coherence"], ref["coherence"], atol=2e-2)
    assert np.all(fit["rank"] >= 1.0) and np.all(fit["rank"] <= 64.0) and np.all(np.abs(fit["coherence"]) <= 1.0)


@pytest.mark.parametrize("shape,n_sets", [((2, 1, 1), 1), ((1, 3, 17), 1), ((3, 13, 9), 3), ((4, 16, 24), 2), ((2, 40, 33), 1)])
def test_ragged_and_tiny_grids(gpu, shape, n_sets):
    from oracle import ca_oracle
    capi, devmem = gpu
    B, H, W = shape
    X0 = inputs.make_state(B, H, W, seed=5, scale=0.45 * H * W)
    w = inputs.make_weight_sets(n_sets, seed=5)
    X1, vprev, vlast, fit = run_bf16(capi, devmem, X0, w, 2)
    R1, rprev, rlast = ca_oracle.ca_steps(X0, w, 2, literal=True, want_vprime=True)
    check_against(X0, X1, vlast, R1, rlast)


def test_long_run_stays_close_and_deterministic(gpu):
    """16 steps: the accumulated bf16 error stays inside the tolerance, and a repeat run is bit-identical."""
    from oracle import ca_oracle
    capi, devmem = gpu
    X0 = inputs.make_state(2, 64, 64, seed=11, scale=0.45 * 64 * 64)
    w = inputs.make_weight_sets(1, seed=11)
    h = capi.Handle(2, 64, 64, dtype=capi.BF16)
    h.set_weights(w)
    h.set_state(X0); h.step(16); a = h.get_state()
    h.set_state(X0); h.step(16); c = h.get_state()
    h.close()
    assert np.array_equal(a, c)
    R = ca_oracle.ca_steps(X0, w, 16, literal=False)
    assert rel_l2(a, R) < TOL


def test_stripes_match_the_whole_torus(gpu):
    import torch
    capi, devmem = gpu
    H, W, steps = 32, 48, 3
    X0 = inputs.make_state(1, H, W, seed=8, scale=0.45 * H * W)
    w = inputs.make_weight_sets(1, seed=8)
    whole = capi.Handle(1, H, W, dtype=capi.BF16)
    whole.set_weights(w); whole.set_state(X0); whole.step(steps)
    ref = whole.get_state()
    whole.close()
    parts = [capi.Handle(1, H // 2, W, stripe=True, dtype=capi.BF16) for _ in range(2)]
    mass = channel_mass(bf16_round(X0))
    for r, p in enumerate(parts):
        p.set_weights(w)
        p.set_state(X0[:, r * H // 2:(r + 1) * H // 2])
        p.set_mass(mass)
    views = [devmem.state_view(p) for p in parts]
    sums = [devmem.sums_view(p) for p in parts]
    n = H // 2
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
    assert rel_l2(got, ref) < 2e-3


def test_batch_of_64_invariants(gpu):
    """The full training-shape batch X[64,128,128,64]: mass conservation and conservation of the redistributed
    value per (head, dim) against sums computed on the host."""
    capi, devmem = gpu
    B = 64
    X0 = inputs.make_state(B, 128, 128, seed=42)
    w = inputs.make_weight_sets(1, seed=42)
    h = capi.Handle(B, 128, 128, dtype=capi.BF16, keep_vprime=True)
    h.set_weights(w)
    h.set_state(X0)
    h.step(1)
    vlast = devmem.vprime(h, capi.BUF_VPRIME_LAST)
    Xb = bf16_round(X0).reshape(B, -1, 64).astype(np.float64)
    sv = np.einsum("bc,hcd->bhd", Xb.sum(axis=1), bf16_round(w.Wv[0]).astype(np.float64)).reshape(B, 512)
    svp = vlast.reshape(B, -1, 512).astype(np.float64).sum(axis=1)
    np.testing.assert_allclose(svp, sv, rtol=2e-3, atol=2e-3 * np.abs(sv).max())
    h.step(7)
    X1 = h.get_state()
    assert np.isfinite(X1).all()
    m0, m1 = channel_mass(bf16_round(X0)), channel_mass(X1)
    assert np.max(np.abs(m1 - m0) / np.abs(m0)) < TOL_MASS
    h.close()


def test_torus_shift_equivariance_full_size(gpu):
    """A size-independent property at the training shape: rolling every grid on its torus rolls the step's output.
    The stored (un-normalised) state and V' are compared bit for bit - each cell's arithmetic does not depend on
    where the cell sits in a tile - so a wrong apron copy, halo or tile edge anywhere on the 128 x 128 grids shows."""
    import torch
    capi, devmem = gpu
    B, H, W = 16, 128, 128
    X0 = bf16_round(inputs.make_state(B, H, W, seed=13, scale=0.45 * H * W))
    w = inputs.make_weight_sets(2, seed=13)
    dy, dx = 5, -19
    outs = []
    for X in (X0, np.roll(X0, (dy, dx), axis=(1, 2))):
        with capi.Handle(B, H, W, n_weight_sets=2, dtype=capi.BF16, keep_vprime=True) as h:
            h.set_weights(w)
            h.set_state(X)
            h.step(1)
            torch.cuda.synchronize()
            outs.append((devmem.state_view(h).float().cpu().numpy().reshape(B, H, W, 64), devmem.vprime(h, capi.BUF_VPRIME_LAST)))
    assert np.array_equal(np.roll(outs[0][1], (dy, dx), axis=(1, 2)), outs[1][1])
    assert np.array_equal(np.roll(outs[0][0], (dy, dx), axis=(1, 2)), outs[1][0])


def test_two_handles_on_two_host_threads(gpu):
    """Handles are independent: two host threads, each driving its own handle on its own stream on the same GPU,
    get exactly what each handle gives when run alone."""
    import threading
    import torch
    capi, _ = gpu
    w = inputs.make_weight_sets(1, seed=8)
    states = [inputs.make_state(6, 64, 48, seed=30 + i, scale=0.45 * 64 * 48) for i in range(2)]

    def run(i, out, stream):
        with capi.Handle(6, 64, 48, dtype=capi.BF16, keep_vprime=True) as h:
            h.set_weights(w)
            for _ in range(3):
                h.set_state(states[i], stream=stream)
                h.step(5, stream=stream)
                fit = h.fitness(stream=stream)
                out[i] = (h.get_state(stream=stream), fit["fitness"].copy())

    alone = [None, None]
    for i in range(2):
        run(i, alone, 0)
    streams = [torch.cuda.Stream() for _ in range(2)]
    together = [None, None]
    threads = [threading.Thread(target=run, args=(i, together, streams[i].cuda_stream)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for i in range(2):
        assert np.array_equal(alone[i][0], together[i][0])
        assert np.array_equal(alone[i][1], together[i][1])
