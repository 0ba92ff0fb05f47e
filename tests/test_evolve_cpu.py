"""The oracle's population step (culling, best, refill with mutated copies): its rules and its statistics."""
import numpy as np

from oracle import ca_oracle
from slime_b200 import inputs

PARAMS = dict(fitness_threshold=10.0, hunger_threshold=0.6, mutation_rate=0.05, mutation_sigma=0.02, seed=7, generation=3)


def _fit(fitness, hunger, per_set):
    n = len(fitness) * per_set
    fit = np.zeros((n, 4), np.float32)
    fit[:, 2] = np.repeat(np.asarray(fitness, np.float32), per_set)
    fit[:, 3] = np.repeat(np.asarray(hunger, np.float32), per_set)
    fit[:, 1] = 1.0 - fit[:, 3]
    return fit


def test_nothing_culled_changes_nothing():
    w = inputs.make_weight_sets(4, seed=1)
    fit = _fit([2.0, 5.0, 3.0, 5.0], [0.1, 0.2, 0.3, 0.4], 2)
    new, parent, best, n = ca_oracle.evolve(fit, w, 2, **PARAMS)
    assert n == 0 and best == 1 and list(parent) == [0, 1, 2, 3]        # first of the tied maxima
    for a, b in zip(new, w.arrays()):
        assert np.array_equal(a, b)


def test_culling_rules_and_refill():
    w = inputs.make_weight_sets(6, seed=2)
    #          low fitness  ok    hungry  NaN          best  ok
    fitness = [0.5,         2.0,  4.0,    float("nan"), 6.0, 1.0]     # culled below 0.1 * 10 = 1.0 (strictly)
    hunger = [0.1,          0.1,  0.7,    0.1,          0.2, 0.6]     # culled above 0.6 (strictly)
    new, parent, best, n = ca_oracle.evolve(_fit(fitness, hunger, 3), w, 3, **PARAMS)
    assert best == 4 and n == 3 and list(parent) == [4, 1, 4, 4, 4, 5]
    old = w.arrays()
    for s in (1, 4, 5):                                   # survivors untouched
        for a, b in zip(new, old):
            assert np.array_equal(a[s], b[s])
    for s in (0, 2, 3):
        for k in (4, 5, 6):                               # taps, mu, sigma inherited unchanged
            assert np.array_equal(new[k][s], old[k][4])
        changed = 0
        total = 0
        deltas = []
        for k in range(4):
            d = new[k][s].astype(np.float64) - old[k][4].astype(np.float64)
            changed += int((d != 0).sum()); total += d.size
            deltas.append(d[d != 0])
        frac = changed / total
        assert abs(frac - 0.05) < 4 * np.sqrt(0.05 * 0.95 / total)
        d = np.concatenate(deltas)
        assert abs(d.mean()) < 4 * 0.02 / np.sqrt(d.size) and abs(d.std() - 0.02) < 0.002
    # the three refills differ from one another (the draw depends on the set index)
    assert not np.array_equal(new[0][0], new[0][2])


def test_no_survivor_changes_nothing():
    w = inputs.make_weight_sets(3, seed=3)
    new, parent, best, n = ca_oracle.evolve(_fit([0.1, 0.2, 0.3], [0.9, 0.9, 0.9], 1), w, 1, **PARAMS)
    assert best == -1 and n == 0 and list(parent) == [0, 1, 2]
    for a, b in zip(new, w.arrays()):
        assert np.array_equal(a, b)


def test_stream_depends_on_seed_and_generation_only():
    w = inputs.make_weight_sets(2, seed=4)
    fit = _fit([0.0, 5.0], [0.0, 0.0], 1)
    a = ca_oracle.evolve(fit, w, 1, **PARAMS)[0][0]
    b = ca_oracle.evolve(fit, w, 1, **PARAMS)[0][0]
    c = ca_oracle.evolve(fit, w, 1, **{**PARAMS, "generation": 4})[0][0]
    d = ca_oracle.evolve(fit, w, 1, **{**PARAMS, "seed": 8})[0][0]
    assert np.array_equal(a, b) and not np.array_equal(a, c) and not np.array_equal(a, d)
    # rate 0 copies the parent exactly; rate 1 perturbs every value
    z = ca_oracle.evolve(fit, w, 1, **{**PARAMS, "mutation_rate": 0.0})[0]
    assert np.array_equal(z[0][0], w.Wp[1]) and np.array_equal(z[3][0], w.Wo[1])
    o = ca_oracle.evolve(fit, w, 1, **{**PARAMS, "mutation_rate": 1.0})[0]
    assert (o[1][0] != w.Wi[1]).mean() > 0.999
