"""The allocation-free channel-sum entry point against the handle-based one.

Collected last on purpose (a run that stops at the first failure has then already run every other test).
It serves callers that can not allocate device memory where they need a state's channel masses - the whole
device already belongs to their own pool, or they sit in a loop that can not take cudaMalloc's device-wide
synchronisation - so the library keeps that reduction's scratch in an array built into its image.
"""
import ctypes

import numpy as np
import pytest

from slime_b200 import inputs

pytestmark = pytest.mark.gpu


def test_static_channel_sums_match_the_handle_twice_in_a_row():
    import torch
    from slime_b200 import capi
    lib = capi.lib()
    B, H, W = 6, 40, 56
    X = inputs.make_state(B, H, W, seed=31, scale=3.0)
    with capi.Handle(B, H, W) as h:
        h.set_state(X)                      # existing entry point: set_state records the channel sums as masses
        want = h.get_mass()
    state = torch.from_numpy(X).cuda()
    out = torch.zeros(B, 64, dtype=torch.float64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                   # the second call reuses whatever the first left in the scratch
        out.fill_(-1.0)
        rc = lib.slime_ca_channel_sums_static(state.data_ptr(), capi.F32, B, H * W, out.data_ptr(), stream)
        assert rc == 0, lib.slime_ca_static_error().decode()
        torch.cuda.synchronize()
        np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-12, atol=0)
    # a different, smaller problem right after: stale partials beyond its range must not leak in
    Xs = inputs.make_state(2, 9, 7, seed=32)
    with capi.Handle(2, 9, 7, dtype=capi.BF16) as h:
        h.set_state(Xs)
        want_s = h.get_mass()
    small = torch.from_numpy(Xs).to(torch.bfloat16).cuda()
    out_s = torch.zeros(2, 64, dtype=torch.float64, device="cuda")
    assert lib.slime_ca_channel_sums_static(small.data_ptr(), capi.BF16, 2, 63, out_s.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    np.testing.assert_allclose(out_s.cpu().numpy(), want_s, rtol=1e-12, atol=0)


def test_static_channel_sums_reject_what_does_not_fit():
    import torch
    from slime_b200 import capi
    lib = capi.lib()
    buf = torch.zeros(64, device="cuda")
    out = torch.zeros(64, dtype=torch.float64, device="cuda")
    assert lib.slime_ca_channel_sums_static(buf.data_ptr(), capi.F32, 9000, 256, out.data_ptr(), None) == 1
    assert b"8192" in lib.slime_ca_static_error()
    assert lib.slime_ca_channel_sums_static(None, capi.F32, 1, 1, out.data_ptr(), None) == 1
    assert lib.slime_ca_channel_sums_static(buf.data_ptr(), 7, 1, 1, out.data_ptr(), None) == 1
