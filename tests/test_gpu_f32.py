"""GPU parity tests of the fp32 path, through the C ABI, against the CPU oracle and the golden fixtures.

Tolerances (fp32 path): state and V' within 1e-5 relative L2, per-channel mass within 1e-6 relative,
fitness scalars within 1e-4.
"""
import numpy as np
import pytest

from slime_b200 import inputs
from tests.helpers import GOLDEN_CASES, channel_mass, load_golden, rel_l2

pytestmark = pytest.mark.gpu

TOL_STATE = 1e-5
TOL_MASS = 1e-6
TOL_FIT = 1e-4


@pytest.fixture(scope="module")
def gpu():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from slime_b200 import capi, devmem
    capi.lib()      # raises if the CUDA library is missing: no fallback
    return capi, devmem


def run_gpu(capi, devmem, X0, w, steps, dtype=None, want_vprime=True):
    B, H, W, _ = X0.shape
    h = capi.Handle(B, H, W, n_weight_sets=w.n_sets, dtype=capi.F32 if dtype is None else dtype, keep_vprime=want_vprime)
    h.set_weights(w)
    h.set_state(X0)
    h.step(steps)
    X1 = h.get_state()
    out = (X1,)
    if want_vprime:
        out += (devmem.vprime(h, capi.BUF_VPRIME_PREV), devmem.vprime(h, capi.BUF_VPRIME_LAST), h.fitness())
    h.close()
    return out


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_fixtures(gpu, name):
    capi, devmem = gpu
    z, w = load_golden(name)
    X1, vprev, vlast, fit = run_gpu(capi, devmem, z["X0"], w, int(z["steps"]))
    assert rel_l2(X1, z["X1"]) < TOL_STATE
    assert rel_l2(vlast, z["vlast"]) < TOL_STATE
    assert rel_l2(vprev, z["vprev"]) < TOL_STATE
    m0, m1 = channel_mass(z["X0"]), channel_mass(X1)
    assert np.max(np.abs(m1 - m0) / np.abs(m0)) < TOL_MASS
    np.testing.assert_allclose(fit["rank"], z["rank"], atol=TOL_FIT)
    np.testing.assert_allclose(fit["coherence"], z["coherence"], atol=TOL_FIT)
    np.testing.assert_allclose(fit["fitness"], z["rank"] * z["coherence"], atol=TOL_FIT)
    np.testing.assert_allclose(fit["hunger"], 1 - z["coherence"], atol=TOL_FIT)


@pytest.mark.parametrize("scale", [1.0, 7000.0], ids=["unit_mass", "bell_exercised"])
def test_reference_model_128(gpu, scale):
    """The CPU-runnable reference model: X[1,128,128,64], seed 42, 16 steps.  Unit mass leaves the growth on
    its -1 plateau, so the same shapes are also run with the state scaled into the bell."""
    from oracle import ca_oracle
    capi, devmem = gpu
    X0 = inputs.make_state(1, 128, 128, seed=42, scale=scale)
    w = inputs.make_weight_sets(1, seed=42)
    X1, vprev, vlast, fit = run_gpu(capi, devmem, X0, w, 16)
    R1, rprev, rlast = ca_oracle.ca_steps(X0, w, 16, literal=False, want_vprime=True)
    assert rel_l2(X1, R1) < TOL_STATE
    assert rel_l2(vlast, rlast) < TOL_STATE
    m0, m1 = channel_mass(X0), channel_mass(X1)
    assert np.max(np.abs(m1 - m0) / np.abs(m0)) < TOL_MASS
    ref = ca_oracle.fitness(rprev, rlast)
    for k in ("rank", "coherence", "fitness", "hunger"):
        np.testing.assert_allclose(fit[k], ref[k], atol=TOL_FIT)
    assert 1.0 <= fit["rank"][0] <= 64.0 and abs(fit["coherence"][0]) <= 1.0


@pytest.mark.parametrize("shape,n_sets", [((2, 1, 1), 1), ((1, 3, 17), 1), ((3, 13, 9), 3), ((4, 16, 24), 2), ((1, 2, 2), 1)])
def test_ragged_and_tiny_grids(gpu, shape, n_sets):
    """Sizes that are not multiples of the tile, grids smaller than the stencil (every tap wraps onto the same
    cells), several weight sets."""
    from oracle import ca_oracle
    capi, devmem = gpu
    B, H, W = shape
    X0 = inputs.make_state(B, H, W, seed=5, scale=0.45 * H * W)
    w = inputs.make_weight_sets(n_sets, seed=5)
    X1, vprev, vlast, fit = run_gpu(capi, devmem, X0, w, 3)
    R1, rprev, rlast = ca_oracle.ca_steps(X0, w, 3, literal=True, want_vprime=True)
    assert rel_l2(X1, R1) < TOL_STATE
    assert rel_l2(vlast, rlast) < TOL_STATE
    assert rel_l2(vprev, rprev) < TOL_STATE


def test_batch_invariants_and_determinism(gpu):
    """64 grids of 128x128 (the training-shape batch) in fp32: per-channel mass, conservation of the
    redistributed value per (head, dim), bit-identical repeat runs."""
    capi, devmem = gpu
    B = 64
    X0 = inputs.make_state(B, 128, 128, seed=42, scale=7000.0)
    w = inputs.make_weight_sets(1, seed=42)
    h = capi.Handle(B, 128, 128, keep_vprime=True)
    h.set_weights(w)
    h.set_state(X0)
    h.step(1)
    vlast = devmem.vprime(h, capi.BUF_VPRIME_LAST)
    V = np.einsum("bnc,hcd->bnhd", X0.reshape(B, -1, 64).astype(np.float64), w.Wv[0].astype(np.float64))
    sv = V.sum(axis=1).reshape(B, 512)
    svp = vlast.reshape(B, -1, 512).astype(np.float64).sum(axis=1)
    np.testing.assert_allclose(svp, sv, rtol=1e-4, atol=1e-4 * np.abs(sv).max())
    h.step(3)
    X1 = h.get_state()
    m0, m1 = channel_mass(X0), channel_mass(X1)
    assert np.max(np.abs(m1 - m0) / np.abs(m0)) < TOL_MASS
    h.set_state(X0)
    h.step(4)
    X2 = h.get_state()
    assert np.array_equal(X1, X2), "two runs from the same state differ"
    # grid 0 of the batch equals a batch-of-one run (grids are independent)
    h1 = capi.Handle(1, 128, 128)
    h1.set_weights(w)
    h1.set_state(X0[:1])
    h1.step(4)
    assert np.array_equal(h1.get_state()[0], X1[0])
    h.close(); h1.close()


def test_stripes_match_the_whole_torus(gpu):
    """Row-stripe decomposition: two stripe handles with 3-row halos exchanged by hand and sums added by hand
    give the same states as one handle holding the whole torus."""
    import torch
    capi, devmem = gpu
    H, W, steps = 24, 20, 3
    X0 = inputs.make_state(1, H, W, seed=8, scale=0.45 * H * W)
    w = inputs.make_weight_sets(1, seed=8)
    whole = capi.Handle(1, H, W)
    whole.set_weights(w); whole.set_state(X0); whole.step(steps)
    ref = whole.get_state()
    whole.close()

    parts = [capi.Handle(1, H // 2, W, stripe=True) for _ in range(2)]
    mass = channel_mass(X0)
    for r, p in enumerate(parts):
        p.set_weights(w)
        p.set_state(X0[:, r * H // 2:(r + 1) * H // 2])
        p.set_mass(mass)
    views = [devmem.state_view(p) for p in parts]
    sums = [devmem.sums_view(p) for p in parts]
    n = H // 2
    for _ in range(steps):
        for r in range(2):          # rows [3, 3+n) are own; halos come from the ring neighbours
            up, down = views[(r - 1) % 2], views[(r + 1) % 2]
            views[r][:, 0:3] = up[:, n:n + 3]
            views[r][:, n + 3:n + 6] = down[:, 3:6]
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
    assert rel_l2(got, ref) < 1e-6


def test_lift_and_readout(gpu):
    from oracle import ca_oracle
    capi, devmem = gpu
    B = 8
    img = inputs.make_images(B, 28, seed=4)
    L, Wr, br = inputs.make_lift_readout(seed=4)
    w = inputs.make_weight_sets(1, seed=4)
    h = capi.Handle(B, 32, 32)
    h.set_weights(w)
    h.lift_images(img, L)
    X0 = ca_oracle.lift(img, L, 2)
    np.testing.assert_allclose(h.get_state(), X0, rtol=1e-6, atol=1e-7)
    h.step(4)
    R = ca_oracle.ca_steps(X0, w, 4, literal=False)
    assert rel_l2(h.get_state(), R) < TOL_STATE
    np.testing.assert_allclose(h.pool_readout(Wr, br), ca_oracle.pool_readout(R, Wr, br), rtol=1e-4, atol=1e-5)
    h.close()


def test_planned_host_launcher(gpu):
    """launch_multi_head_ca(ca_state, weights, ca_output, batch, grid): per-head V' with uniform flow kernels."""
    import torch
    from oracle import ca_oracle
    capi, devmem = gpu
    B, G = 2, 16
    X0 = inputs.make_state(B, G, G, seed=6, scale=0.45 * G * G)
    w = inputs.make_weight_sets(1, seed=6)
    w.K[:] = 1.0 / 9.0
    w.mu[:] = 0.2
    w.sigma[:] = 0.03
    _, _, rlast = ca_oracle.ca_steps(X0, w, 1, want_vprime=True)
    st = torch.from_numpy(X0).cuda()
    wt = torch.from_numpy(np.concatenate([w.Wp[0].ravel(), w.Wi[0].ravel(), w.Wv[0].ravel()])).cuda()
    out = torch.zeros(B, 8, G, G, 64, device="cuda")
    capi.lib().launch_multi_head_ca(st.data_ptr(), wt.data_ptr(), out.data_ptr(), B, G)
    got = out.permute(0, 2, 3, 1, 4).reshape(B, G, G, 512).cpu().numpy()
    assert rel_l2(got, rlast) < TOL_STATE


def test_error_behaviour(gpu):
    capi, devmem = gpu
    with pytest.raises(capi.SlimeCAError) as e:
        capi.Handle(0, 8, 8)
    assert e.value.status == 1
    with pytest.raises(capi.SlimeCAError):
        capi.Handle(3, 8, 8, n_weight_sets=2)        # sets must divide the batch
    with pytest.raises(capi.SlimeCAError):
        capi.Handle(1, 8, 8, device=99)
    h = capi.Handle(2, 8, 8, n_weight_sets=2, keep_vprime=True)
    w = inputs.make_weight_sets(2, seed=1)
    with pytest.raises(capi.SlimeCAError) as e:
        h.step(1)                                    # nothing uploaded yet
    assert e.value.status == 4
    h.set_weight_set(0, *[a[0] for a in w.arrays()])
    h.set_state(inputs.make_state(2, 8, 8))
    with pytest.raises(capi.SlimeCAError) as e:
        h.step(1)                                    # weight set 1 still missing
    assert e.value.status == 4
    with pytest.raises(capi.SlimeCAError) as e:
        h.set_weight_set(2, *[a[0] for a in w.arrays()])
    assert e.value.status == 1
    h.set_weights(w)
    h.step(1)
    with pytest.raises(capi.SlimeCAError) as e:
        h.fitness()                                  # needs two steps
    assert e.value.status == 4
    h.step(1)
    f = h.fitness()
    assert np.all(np.isfinite(f["fitness"]))
    with pytest.raises(capi.SlimeCAError):
        h.step(-1)
    assert "negative" in capi.lib().slime_ca_last_error(h._h).decode()
    h.close()
