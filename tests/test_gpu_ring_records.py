"""GPU tests of the entry points around the step: the row-stripe ring inside the library (one rank, the stripe
wrapping onto itself; two ranks over NCCL are in test_gpu_multi.py), its bounded host wait, the bounded device wait
and how a caller learns of it, the elite record, occupancy, and the read-out's staging limit."""
import numpy as np
import pytest

from slime_b200 import inputs
from tests.helpers import channel_mass, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from slime_b200 import capi, devmem
    capi.lib()
    return capi, devmem


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_one_rank_ring_equals_the_whole_torus(gpu, dtype_name):
    """slime_ca_step_ring with a ring of one: the stripe's halo rows are its own far rows, so the stripe handle must
    reproduce the torus handle (same kernels, stripe geometry instead of wrap-around indexing)."""
    import torch
    from slime_b200 import sharding
    capi, devmem = gpu
    dtype = capi.F32 if dtype_name == "f32" else capi.BF16
    H, W, steps = 40, 48, 5
    X0 = inputs.make_state(1, H, W, seed=8, scale=0.45 * H * W)
    w = inputs.make_weight_sets(1, seed=8)
    with capi.Handle(1, H, W, dtype=dtype) as h:
        h.set_weights(w); h.set_state(X0); h.step(steps)
        ref = h.get_state()
    grid = sharding.StripedGrid(H, W, w, dtype=dtype, device=0)
    grid.load(X0)
    grid.step(steps)
    torch.cuda.synchronize()
    got = grid.read()
    ms = grid.handle.step_ring_timed(2)
    grid.close()
    assert rel_l2(got, ref) < (1e-6 if dtype_name == "f32" else 2e-3)
    assert len(ms) == 3 and all(m >= 0 for m in ms) and ms[1] > 0


def test_ring_needs_a_stripe_handle_and_a_ring(gpu):
    capi, _ = gpu
    w = inputs.make_weight_sets(1, seed=8)
    with capi.Handle(1, 16, 16, dtype=capi.F32) as h:
        with pytest.raises(capi.SlimeCAError) as e:
            h.ring_init(None, 0, 1)
        assert e.value.status == 4
    with capi.Handle(1, 16, 16, dtype=capi.F32, stripe=True) as h:
        h.set_weights(w); h.set_state(inputs.make_state(1, 16, 16, seed=1))
        with pytest.raises(capi.SlimeCAError) as e:
            h.step_ring(1)
        assert e.value.status == 4 and "no ring attached" in str(e.value)
        with pytest.raises(capi.SlimeCAError):
            h.ring_init(None, 2, 2)                    # rank outside the world


def test_ring_wait_gives_up_at_its_deadline_and_succeeds_with_time(gpu):
    """The bounded host wait: with a tenth of a second of work queued a zero deadline runs out (SLIME_CA_ETIMEOUT, the
    handle stays usable: with one rank there is no communicator to abort), a generous one returns 0."""
    capi, _ = gpu
    H = W = 256
    w = inputs.make_weight_sets(1, seed=8, bounded=True)
    with capi.Handle(1, H, W, dtype=capi.F32, stripe=True) as h:
        h.set_weights(w); h.set_state(inputs.make_state(1, H, W, seed=2))
        h.ring_init(None, 0, 1)
        h.ring_sync_mass()
        h.step_ring(60)
        with pytest.raises(capi.SlimeCAError) as e:
            h.ring_wait(0)
        assert e.value.status == 7
        h.ring_wait(60000)
        h.step_ring(1)
        h.ring_wait(60000)
        assert np.isfinite(h.get_state()).all()


def test_a_bounded_device_wait_runs_out_and_is_reported(gpu):
    """A kernel waits 1 ms on a barrier nobody arrives on, gives up and records its code; the host sees
    SLIME_CA_EDEVICE at the next call - through the copied-back word for a caller that never synchronises, through the
    word itself for one that does - the word is cleared, and the context and the handle keep working."""
    import torch
    capi, _ = gpu
    X0 = inputs.make_state(2, 16, 16, seed=4, scale=0.45 * 256)
    w = inputs.make_weight_sets(1, seed=4)
    with capi.Handle(2, 16, 16, dtype=capi.BF16) as h:
        h.set_weights(w); h.set_state(X0); h.step(2)
        good = h.get_state()
        # device-resident caller: no synchronising call of the library in between
        h.selftest_bounded_wait(1_000_000)
        torch.cuda.synchronize()
        with pytest.raises(capi.SlimeCAError) as e:
            h.step(1)
        assert e.value.status == 5 and "901" in str(e.value) and "load it again" in str(e.value)
        h.set_state(X0); h.step(2)                       # cleared: the same steps give the same state
        assert np.array_equal(h.get_state(), good)
        # synchronising caller
        h.selftest_bounded_wait(1_000_000)
        with pytest.raises(capi.SlimeCAError) as e:
            h.get_state()
        assert e.value.status == 5
        h.set_state(X0); h.step(2)
        assert np.array_equal(h.get_state(), good)
        with pytest.raises(capi.SlimeCAError):
            h.selftest_bounded_wait(10**12)              # limits above 100 ms are refused


def test_elite_record(gpu):
    from oracle import ca_oracle
    capi, _ = gpu
    n_sets, per = 4, 2
    w = inputs.make_weight_sets(n_sets, seed=21)
    X0 = inputs.make_state(n_sets * per, 16, 16, seed=21, scale=0.45 * 256)
    with capi.Handle(n_sets * per, 16, 16, n_weight_sets=n_sets, dtype=capi.F32, keep_vprime=True) as h:
        h.set_weights(w); h.set_state(X0)
        with pytest.raises(capi.SlimeCAError):
            h.elite_record(0, 3)                         # no fitness yet
        h.step(3)
        fit = h.fitness()
        for s in range(n_sets):
            e = h.elite_record(s, 70000 + s)
            sl = slice(s * per, (s + 1) * per)
            assert e["fitness"] == pytest.approx(float(fit["fitness"][sl].mean()), rel=1e-6)
            assert e["coherence"] == pytest.approx(float(fit["coherence"][sl].mean()), rel=1e-6)
            assert e["effective_rank"] == pytest.approx(float(fit["rank"][sl].mean()), rel=1e-6)
            genome = np.concatenate([a[s].reshape(-1) for a in w.arrays()])
            assert genome.size == 131160
            padded = np.concatenate([genome, np.zeros(8, np.float32)])      # the master copy's stride is 131 168
            assert e["genome_hash"] == ca_oracle.genome_hash(padded)
            assert e["parent_ids"] == (s, s) and e["generation"] == (70000 + s) & 0xFFFF
        thr = float(10.0 * np.median(fit["fitness"].reshape(n_sets, per).mean(1)))
        evo = h.evolve(fitness_threshold=thr, hunger_threshold=2.0, mutation_rate=0.01, mutation_sigma=0.0125, seed=42, generation=1)
        assert 0 < evo["n_replaced"] < n_sets
        for s in range(n_sets):
            e = h.elite_record(s, 2)
            assert e["parent_ids"] == (int(evo["parent"][s]), int(evo["parent"][s]))
            got = np.concatenate([a.reshape(-1) for a in h.get_weights(s)] + [np.zeros(8, np.float32)])
            assert e["genome_hash"] == ca_oracle.genome_hash(got)


def test_occupancy_and_readout_limit(gpu):
    capi, _ = gpu
    with capi.Handle(1, 4, 4, dtype=capi.BF16) as h:
        assert h.occupancy == pytest.approx(608 / 2048)          # one 608-thread CTA of the projection kernel per SM
        h.set_weights(inputs.make_weight_sets(1, seed=1)); h.set_state(inputs.make_state(1, 4, 4, seed=1))
        with pytest.raises(capi.SlimeCAError) as e:
            h.pool_readout(np.zeros((64, 1024), np.float32))     # 266 KB of staging into a 64 KB buffer
        assert e.value.status == 1 and "staging" in str(e.value)
        assert h.pool_readout(np.zeros((64, 10), np.float32)).shape == (1, 10)
    with capi.Handle(1, 4, 4, dtype=capi.F32) as h:
        assert 256 / 2048 <= h.occupancy <= 1.0
