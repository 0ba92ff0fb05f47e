"""The population step on the device (slime_ca_evolve) against the oracle's, and the device-resident master
weights it works on."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

N_SETS, PER_SET, H, W = 8, 2, 16, 16


def _population(dtype):
    from slime_b200 import capi, inputs
    w = inputs.make_weight_sets(N_SETS, seed=21)
    X0 = inputs.make_state(N_SETS * PER_SET, H, W, seed=21, scale=0.45 * H * W)
    h = capi.Handle(N_SETS * PER_SET, H, W, n_weight_sets=N_SETS, dtype=dtype, keep_vprime=True)
    h.set_weights(w)
    h.set_state(X0)
    return h, w, X0


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_weights_round_trip(dtype_name):
    from slime_b200 import capi
    h, w, _ = _population(capi.F32 if dtype_name == "f32" else capi.BF16)
    with h:
        for s in (0, N_SETS - 1):
            for got, want in zip(h.get_weights(s), w.arrays()):
                assert np.array_equal(got, want[s])


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_evolve_matches_oracle(dtype_name):
    from oracle import ca_oracle
    from slime_b200 import capi, inputs
    dt = capi.F32 if dtype_name == "f32" else capi.BF16
    h, w, X0 = _population(dt)
    with h:
        with pytest.raises(capi.SlimeCAError):            # no fitness yet
            h.evolve(fitness_threshold=1.0, hunger_threshold=1.0, mutation_rate=0.1, mutation_sigma=0.01, seed=1, generation=0)
        h.step(3)
        f = h.fitness()
        fit = np.stack([f["rank"], f["coherence"], f["fitness"], f["hunger"]], axis=1)
        set_fit = fit[:, 2].astype(np.float64).reshape(N_SETS, PER_SET).mean(1).astype(np.float32)
        # threshold between the 3rd and 4th weakest set: three sets are culled
        order = np.sort(set_fit)
        params = dict(fitness_threshold=float(10.0 * 0.5 * (order[2] + order[3])), hunger_threshold=2.0,
                      mutation_rate=0.1, mutation_sigma=0.01, seed=99, generation=5)
        res = h.evolve(**params)
        ref_w, ref_parent, ref_best, ref_n = ca_oracle.evolve(fit, w, PER_SET, **params)
        assert ref_n == 3
        assert res["n_replaced"] == ref_n and res["best"] == ref_best and list(res["parent"]) == list(ref_parent)
        for s in range(N_SETS):
            got = h.get_weights(s)
            for k in range(7):
                if ref_parent[s] == s or k >= 4:
                    assert np.array_equal(got[k], ref_w[k][s])
                else:
                    same = ref_w[k][s] == w.arrays()[k][ref_best]           # values the oracle left alone
                    assert np.array_equal(got[k][same], ref_w[k][s][same])
                    assert np.abs(got[k] - ref_w[k][s]).max() < 1e-6        # perturbed ones: libm vs device math
                    assert 0.05 < 1.0 - same.mean() < 0.15
        # the operand layouts of the replaced sets were rebuilt: stepping equals a fresh handle given the read-back weights
        evolved = [np.stack([h.get_weights(s)[k] for s in range(N_SETS)]) for k in range(7)]
        h.set_state(X0)
        h.step(2)
        a = h.get_state()
    with capi.Handle(N_SETS * PER_SET, H, W, n_weight_sets=N_SETS, dtype=dt) as g:
        g.set_weights(inputs.WeightSets(*evolved))
        g.set_state(X0)
        g.step(2)
        assert np.array_equal(a, g.get_state())


def test_evolve_needs_current_fitness():
    from slime_b200 import capi
    h, _, _ = _population(capi.F32)
    with h:
        h.step(2)
        h.fitness()
        h.step(1)                                           # the fitness on the device is stale now
        with pytest.raises(capi.SlimeCAError):
            h.evolve(fitness_threshold=1.0, hunger_threshold=1.0, mutation_rate=0.1, mutation_sigma=0.01, seed=1, generation=0)
