"""ctypes binding of the C ABI declared in include/slime_ca.h.

There is no fallback: if libslime_ca.so is missing or a call fails, this raises.  The library is looked up
beside this file (built in-tree by slime_b200.build).
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libslime_ca.so")

F32, BF16 = 0, 1
BUF_STATE, BUF_SCALE, BUF_MASS, BUF_SUMS, BUF_VPRIME_PREV, BUF_VPRIME_LAST = range(6)
STATUS = {0: "OK", 1: "EINVAL", 2: "ECUDA", 3: "ENOMEM", 4: "ESTATE", 5: "EDEVICE", 6: "ECOMM", 7: "ETIMEOUT"}
RING_ID_BYTES = 128

# every symbol include/slime_ca.h declares
SYMBOLS = (
    "slime_ca_create", "slime_ca_destroy", "slime_ca_last_error", "slime_ca_workspace_bytes",
    "slime_ca_set_weights", "slime_ca_set_state", "slime_ca_get_state", "slime_ca_set_state_device",
    "slime_ca_get_state_device", "slime_ca_set_mass", "slime_ca_get_mass", "slime_ca_step",
    "slime_ca_step_partial", "slime_ca_step_finish", "slime_ca_step_timed", "slime_ca_buffer", "slime_ca_fitness",
    "slime_ca_lift_images", "slime_ca_pool_readout", "slime_ca_launch_count", "launch_multi_head_ca",
    "slime_ca_channel_sums_static", "slime_ca_static_error",
    "slime_ca_lift_field_device", "slime_ca_field_from_state_device", "slime_ca_set_weights_reference_layout",
    "slime_ca_get_weights", "slime_ca_evolve", "slime_ca_evolution_record",
    "slime_ca_ring_unique_id", "slime_ca_ring_init", "slime_ca_ring_attach", "slime_ca_ring_detach",
    "slime_ca_ring_sync_mass", "slime_ca_step_ring", "slime_ca_step_ring_timed", "slime_ca_ring_wait",
    "slime_ca_elite_record", "slime_ca_occupancy", "slime_ca_selftest_bounded_wait",
)


class SlimeCAError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"slime_ca status {status} ({STATUS.get(status, '?')}): {text}")
        self.status = status


class Config(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int), ("height", ctypes.c_int), ("width", ctypes.c_int),
                ("n_weight_sets", ctypes.c_int), ("dtype", ctypes.c_int), ("dt", ctypes.c_float),
                ("device", ctypes.c_int), ("stripe", ctypes.c_int), ("keep_vprime", ctypes.c_int)]


class Elite(ctypes.Structure):
    _fields_ = [("fitness", ctypes.c_float), ("coherence", ctypes.c_float), ("effective_rank", ctypes.c_float),
                ("genome_hash", ctypes.c_ulonglong), ("parent_ids", ctypes.c_uint * 2), ("generation", ctypes.c_ushort)]


class EvolveParams(ctypes.Structure):
    _fields_ = [("fitness_threshold", ctypes.c_float), ("hunger_threshold", ctypes.c_float),
                ("mutation_rate", ctypes.c_float), ("mutation_sigma", ctypes.c_float),
                ("seed", ctypes.c_ulonglong), ("generation", ctypes.c_int)]


_lib = None


def lib():
    """The loaded library (raises OSError if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} not found: build it with `python -m slime_b200.build` (needs nvcc)")
        L = ctypes.CDLL(LIB_PATH)
        vp, fp, dp = ctypes.c_void_p, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_double)
        L.slime_ca_create.argtypes = [ctypes.POINTER(Config), ctypes.POINTER(vp)]
        L.slime_ca_destroy.argtypes = [vp]
        L.slime_ca_last_error.argtypes = [vp]
        L.slime_ca_last_error.restype = ctypes.c_char_p
        L.slime_ca_workspace_bytes.argtypes = [vp]
        L.slime_ca_workspace_bytes.restype = ctypes.c_size_t
        L.slime_ca_set_weights.argtypes = [vp, ctypes.c_int] + [fp] * 7
        L.slime_ca_set_state.argtypes = [vp, vp, ctypes.c_int, vp]
        L.slime_ca_get_state.argtypes = [vp, vp, ctypes.c_int, vp]
        L.slime_ca_set_state_device.argtypes = [vp, vp, ctypes.c_int, vp]
        L.slime_ca_get_state_device.argtypes = [vp, vp, ctypes.c_int, vp]
        L.slime_ca_set_mass.argtypes = [vp, dp]
        L.slime_ca_get_mass.argtypes = [vp, dp]
        L.slime_ca_step.argtypes = [vp, ctypes.c_int, vp]
        L.slime_ca_step_partial.argtypes = [vp, vp]
        L.slime_ca_step_finish.argtypes = [vp, vp]
        L.slime_ca_step_timed.argtypes = [vp, ctypes.c_int, vp, fp]
        L.slime_ca_buffer.argtypes = [vp, ctypes.c_int, ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_size_t)]
        L.slime_ca_fitness.argtypes = [vp, fp, fp, fp, fp, vp]
        L.slime_ca_lift_images.argtypes = [vp, fp, ctypes.c_int, ctypes.c_int, fp, vp]
        L.slime_ca_pool_readout.argtypes = [vp, fp, fp, ctypes.c_int, fp, vp]
        L.slime_ca_lift_field_device.argtypes = [vp, vp, fp, vp]
        L.slime_ca_field_from_state_device.argtypes = [vp, vp, vp]
        L.slime_ca_set_weights_reference_layout.argtypes = [vp, ctypes.c_int] + [vp] * 5 + [fp, fp]
        L.slime_ca_get_weights.argtypes = [vp, ctypes.c_int] + [fp] * 7
        ip = ctypes.POINTER(ctypes.c_int)
        L.slime_ca_evolve.argtypes = [vp, ctypes.POINTER(EvolveParams), ip, ip, ip, vp]
        L.slime_ca_evolution_record.argtypes = [vp, ctypes.c_int, ctypes.c_int, ctypes.c_double, vp] + [ctypes.c_int] * 4 + \
                                               [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t), vp]
        L.slime_ca_launch_count.argtypes = [vp]
        L.slime_ca_launch_count.restype = ctypes.c_longlong
        L.slime_ca_ring_unique_id.argtypes = [vp]
        L.slime_ca_ring_init.argtypes = [vp, vp, ctypes.c_int, ctypes.c_int]
        L.slime_ca_ring_attach.argtypes = [vp, vp, ctypes.c_int, ctypes.c_int]
        L.slime_ca_ring_detach.argtypes = [vp]
        L.slime_ca_ring_sync_mass.argtypes = [vp, vp]
        L.slime_ca_step_ring.argtypes = [vp, ctypes.c_int, vp]
        L.slime_ca_step_ring_timed.argtypes = [vp, ctypes.c_int, vp, fp]
        L.slime_ca_ring_wait.argtypes = [vp, vp, ctypes.c_int]
        L.slime_ca_elite_record.argtypes = [vp, ctypes.c_int, ctypes.c_int, ctypes.POINTER(Elite), vp]
        L.slime_ca_occupancy.argtypes = [vp, fp]
        L.slime_ca_selftest_bounded_wait.argtypes = [vp, ctypes.c_ulonglong, vp]
        L.launch_multi_head_ca.argtypes = [vp, vp, vp, ctypes.c_int, ctypes.c_int]
        L.launch_multi_head_ca.restype = None
        L.slime_ca_channel_sums_static.argtypes = [vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, vp, vp]
        L.slime_ca_static_error.argtypes = []
        L.slime_ca_static_error.restype = ctypes.c_char_p
        _lib = L
    return _lib


def _fp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def ring_unique_id() -> bytes:
    """The 128-byte id every rank of a row-stripe ring passes to Handle.ring_init (made on one rank, shipped to
    the others by the caller)."""
    buf = ctypes.create_string_buffer(RING_ID_BYTES)
    rc = lib().slime_ca_ring_unique_id(buf)
    if rc != 0:
        raise SlimeCAError(rc, "slime_ca_ring_unique_id failed (is NCCL loadable?)")
    return buf.raw


class Handle:
    """One CA handle on one GPU (thin, 1:1 over the C ABI)."""

    def __init__(self, batch, height, width, *, n_weight_sets=1, dtype=F32, dt=0.1, device=0, stripe=False,
                 keep_vprime=False):
        self._h = ctypes.c_void_p()
        self.cfg = Config(batch, height, width, n_weight_sets, dtype, dt, device, int(stripe), int(keep_vprime))
        rc = lib().slime_ca_create(ctypes.byref(self.cfg), ctypes.byref(self._h))
        if rc != 0:
            text = lib().slime_ca_last_error(self._h).decode() if self._h else "create failed"
            if self._h:
                lib().slime_ca_destroy(self._h)
                self._h = ctypes.c_void_p()
            raise SlimeCAError(rc, text)

    # -- plumbing ---------------------------------------------------------------------------------
    def _ck(self, rc):
        if rc != 0:
            raise SlimeCAError(rc, lib().slime_ca_last_error(self._h).decode())

    def close(self):
        if getattr(self, "_h", None):
            lib().slime_ca_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def shape(self):
        return (self.cfg.batch, self.cfg.height, self.cfg.width, 64)

    @property
    def workspace_bytes(self):
        return lib().slime_ca_workspace_bytes(self._h)

    @property
    def launch_count(self):
        return lib().slime_ca_launch_count(self._h)

    # -- weights / state ---------------------------------------------------------------------------
    def set_weights(self, weights, first_set=0):
        """weights: object with arrays() -> (Wp, Wi, Wv, Wo, K, mu, sigma) stacked over sets."""
        arrs = [_f32(a) for a in weights.arrays()]
        for s in range(arrs[0].shape[0]):
            self._ck(lib().slime_ca_set_weights(self._h, first_set + s, *[_fp(a[s]) for a in arrs]))

    def set_weight_set(self, index, Wp, Wi, Wv, Wo, K, mu, sigma):
        arrs = [_f32(a) for a in (Wp, Wi, Wv, Wo, K, mu, sigma)]
        self._ck(lib().slime_ca_set_weights(self._h, index, *[_fp(a) for a in arrs]))

    def set_state(self, X, stream=0):
        X = _f32(X)
        if X.shape != self.shape:
            raise ValueError(f"state shape {X.shape} != {self.shape}")
        self._ck(lib().slime_ca_set_state(self._h, X.ctypes.data, F32, stream))

    def get_state(self, stream=0):
        out = np.empty(self.shape, np.float32)
        self._ck(lib().slime_ca_get_state(self._h, out.ctypes.data, F32, stream))
        return out

    def set_state_ptr(self, host_ptr, dtype, stream=0):
        """Host pointer variant (pinned memory, bf16 payloads)."""
        self._ck(lib().slime_ca_set_state(self._h, host_ptr, dtype, stream))

    def get_state_ptr(self, host_ptr, dtype, stream=0):
        self._ck(lib().slime_ca_get_state(self._h, host_ptr, dtype, stream))

    def set_state_device(self, dev_ptr, dtype, stream=0):
        self._ck(lib().slime_ca_set_state_device(self._h, dev_ptr, dtype, stream))

    def get_state_device(self, dev_ptr, dtype, stream=0):
        self._ck(lib().slime_ca_get_state_device(self._h, dev_ptr, dtype, stream))

    def set_mass(self, mass):
        m = np.ascontiguousarray(mass, dtype=np.float64)
        assert m.shape == (self.cfg.batch, 64)
        self._ck(lib().slime_ca_set_mass(self._h, m.ctypes.data_as(ctypes.POINTER(ctypes.c_double))))

    def get_mass(self):
        m = np.empty((self.cfg.batch, 64), np.float64)
        self._ck(lib().slime_ca_get_mass(self._h, m.ctypes.data_as(ctypes.POINTER(ctypes.c_double))))
        return m

    # -- stepping ------------------------------------------------------------------------------------
    def step(self, n_steps=1, stream=0):
        self._ck(lib().slime_ca_step(self._h, int(n_steps), stream))

    def step_partial(self, stream=0):
        self._ck(lib().slime_ca_step_partial(self._h, stream))

    def step_finish(self, stream=0):
        self._ck(lib().slime_ca_step_finish(self._h, stream))

    def step_timed(self, n_steps, stream=0):
        """-> [ms in k1, ms in k2, ms in the reductions] summed over n_steps (synchronises)."""
        ms = np.zeros(3, np.float32)
        self._ck(lib().slime_ca_step_timed(self._h, int(n_steps), stream, _fp(ms)))
        return [float(x) for x in ms]

    # -- row-stripe ring (stripe mode) ------------------------------------------------------------------
    def ring_init(self, ring_id, rank, world):
        """Join the ring: `ring_id` is the 128-byte id rank 0 got from ring_unique_id() (None when world == 1)."""
        buf = None if ring_id is None else ctypes.create_string_buffer(bytes(ring_id), RING_ID_BYTES)
        self._ck(lib().slime_ca_ring_init(self._h, buf, int(rank), int(world)))

    def ring_detach(self):
        self._ck(lib().slime_ca_ring_detach(self._h))

    def ring_sync_mass(self, stream=0):
        self._ck(lib().slime_ca_ring_sync_mass(self._h, stream))

    def step_ring(self, n_steps=1, stream=0):
        self._ck(lib().slime_ca_step_ring(self._h, int(n_steps), stream))

    def step_ring_timed(self, n_steps, stream=0):
        """-> [ms in the halo exchange, ms in the step's kernels, ms in the all-reduce + scale] summed over n_steps."""
        ms = np.zeros(3, np.float32)
        self._ck(lib().slime_ca_step_ring_timed(self._h, int(n_steps), stream, _fp(ms)))
        return [float(x) for x in ms]

    def ring_wait(self, timeout_ms, stream=0):
        self._ck(lib().slime_ca_ring_wait(self._h, stream, int(timeout_ms)))

    # -- records and diagnostics ---------------------------------------------------------------------------
    def elite_record(self, set_index, generation, stream=0):
        e = Elite()
        self._ck(lib().slime_ca_elite_record(self._h, int(set_index), int(generation), ctypes.byref(e), stream))
        return {"fitness": e.fitness, "coherence": e.coherence, "effective_rank": e.effective_rank,
                "genome_hash": int(e.genome_hash), "parent_ids": (int(e.parent_ids[0]), int(e.parent_ids[1])),
                "generation": int(e.generation)}

    @property
    def occupancy(self):
        o = ctypes.c_float(0)
        self._ck(lib().slime_ca_occupancy(self._h, ctypes.byref(o)))
        return float(o.value)

    def selftest_bounded_wait(self, limit_ns=1_000_000, stream=0):
        self._ck(lib().slime_ca_selftest_bounded_wait(self._h, int(limit_ns), stream))

    def buffer(self, which):
        """-> (device address, bytes) of one of the handle's buffers."""
        p, n = ctypes.c_void_p(), ctypes.c_size_t()
        self._ck(lib().slime_ca_buffer(self._h, which, ctypes.byref(p), ctypes.byref(n)))
        return p.value, n.value

    def fitness(self, stream=0):
        B = self.cfg.batch
        out = {k: np.empty(B, np.float32) for k in ("rank", "coherence", "fitness", "hunger")}
        self._ck(lib().slime_ca_fitness(self._h, _fp(out["rank"]), _fp(out["coherence"]), _fp(out["fitness"]),
                                        _fp(out["hunger"]), stream))
        return out

    def lift_images(self, img, L, stream=0):
        img, L = _f32(img), _f32(L)
        assert img.shape[0] == self.cfg.batch and L.shape == (64,)
        self._ck(lib().slime_ca_lift_images(self._h, _fp(img), img.shape[1], img.shape[2], _fp(L), stream))

    def lift_field_device(self, dev_field_ptr, L, stream=0):
        """Lift a device field [batch][height][width] fp32 (raw address) into the state."""
        L = _f32(L)
        assert L.shape == (64,)
        self._ck(lib().slime_ca_lift_field_device(self._h, dev_field_ptr, _fp(L), stream))

    def field_from_state_device(self, dev_field_ptr, stream=0):
        """Mean over channels of the normalised state into a device field [batch][height][width] fp32."""
        self._ck(lib().slime_ca_field_from_state_device(self._h, dev_field_ptr, stream))

    def set_weights_reference_layout(self, perception_ptr, interaction_ptr, value_ptr, mixing_ptr, flow_ptr,
                                     mu=None, sigma=None, set_index=0):
        """Upload a weight set from device arrays in the reference bundle's layouts (raw addresses)."""
        m = None if mu is None else _f32(mu)
        s = None if sigma is None else _f32(sigma)
        self._ck(lib().slime_ca_set_weights_reference_layout(
            self._h, set_index, perception_ptr, interaction_ptr, value_ptr, mixing_ptr, flow_ptr,
            None if m is None else _fp(m), None if s is None else _fp(s)))

    def get_weights(self, set_index=0):
        """(Wp, Wi, Wv, Wo, K, mu, sigma) of one set as held on the device (fp32 master copy)."""
        out = [np.empty((8, 64, 64), np.float32) for _ in range(3)] + [np.empty((512, 64), np.float32),
               np.empty((8, 9), np.float32), np.empty(8, np.float32), np.empty(8, np.float32)]
        self._ck(lib().slime_ca_get_weights(self._h, set_index, *[_fp(a) for a in out]))
        return tuple(out)

    def evolve(self, *, fitness_threshold, hunger_threshold, mutation_rate, mutation_sigma, seed, generation, stream=0):
        """The population step after fitness(): returns dict(parent=[n_sets], best=int, n_replaced=int)."""
        p = EvolveParams(fitness_threshold, hunger_threshold, mutation_rate, mutation_sigma, seed, generation)
        parent = np.empty(self.cfg.n_weight_sets, np.int32)
        best, n = ctypes.c_int(-1), ctypes.c_int(0)
        self._ck(lib().slime_ca_evolve(self._h, ctypes.byref(p), parent.ctypes.data_as(ctypes.POINTER(ctypes.c_int)),
                                       ctypes.byref(best), ctypes.byref(n), stream))
        return {"parent": parent, "best": best.value, "n_replaced": n.value}

    def evolution_record(self, grid_index, generation, elapsed, *, dev_field_ptr=None, active=0, capacity=0, spawned=0,
                         culled=0, stream=0):
        """One line of the reference's evolution.json for one grid (str, newline-terminated)."""
        buf = ctypes.create_string_buffer(16384)
        n = ctypes.c_size_t(0)
        self._ck(lib().slime_ca_evolution_record(self._h, grid_index, generation, elapsed, dev_field_ptr, active, capacity,
                                                 spawned, culled, buf, len(buf), ctypes.byref(n), stream))
        return buf.value.decode()

    def pool_readout(self, Wr, br=None, stream=0):
        Wr = _f32(Wr)
        n_out = Wr.shape[1]
        out = np.empty((self.cfg.batch, n_out), np.float32)
        b = None if br is None else _f32(br)
        self._ck(lib().slime_ca_pool_readout(self._h, _fp(Wr), None if b is None else _fp(b), n_out, _fp(out), stream))
        return out
