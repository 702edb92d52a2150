"""The allocation-free LSTM entry point (aig_lstm_forward_noalloc) against the plan-based one.

Some users of this library cannot allocate device memory once they are running: the 30 Hz frame loop
shares the GPU with the game it plays, where a cudaMalloc would synchronise the whole device and the
game may already own nearly all of the memory, and some hosts reserve their whole device budget at
start-up.  For them the library carries a fixed scratch array in its device image.  This test calls
that entry point through the C ABI twice in a row (the array is shared and keeps the previous call's
contents, so the second call checks that what must start at zero is cleared) and compares both
results with the existing plan-based entry point on the same inputs.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.  It does not depend on them and passes alone in a fresh process.
"""
import numpy as np
import pytest

gpu = pytest.mark.gpu

TOL = 6e-3  # same absolute tolerance on h as the LSTM-vs-oracle tests


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_util as U

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return U


@gpu
def test_noalloc_lstm_matches_plan_entry_point_twice(env):
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    from ai_gamer_b200 import synth as SY

    from oracle import oracle as O

    lib = pk.lib()
    T, B, I, H = 12, 24, 96, 128
    rng = np.random.default_rng(4242)
    blob = SY.make_lstm_blob(rng, I, H, 1, True, 1.0)
    blob[-4 * H:] = rng.uniform(-0.2, 0.2, 4 * H).astype(np.float16)
    d_blob = U.dev(blob)
    plan = pk.LstmPlan(c, T, 1, H, B, I, clip=5.0, double_bias=True)
    plan.set_weights(d_blob)
    for call in range(2):
        x = (rng.standard_normal((T, B, I)) * (1.0 + call)).astype(np.float16)
        dx = U.dev(x)
        want = torch.zeros(T * B * H, dtype=torch.float16, device="cuda")
        plan.forward(dx, want)
        got = torch.full((T * B * H,), 7.0, dtype=torch.float16, device="cuda")
        rc = lib.aig_lstm_forward_noalloc(c.handle, pk.ptr(dx), pk.ptr(d_blob), pk.ptr(got), T, B, I, H, 5.0, 1)
        assert rc == 0, lib.aig_last_error(c.handle).decode()
        c.sync()
        a, b = U.host(got).astype(np.float32), U.host(want).astype(np.float32)
        assert np.isfinite(a).all()
        err = np.abs(a - b).max()
        assert err < TOL, "call %d: max |noalloc - plan| = %.4g" % (call, err)
        assert (a == b).mean() > 0.9  # only the projection's summation order differs
        # and the CPU oracle of the reference's LSTM call on the same inputs
        ref = O.lstm(x, blob, H, 1, 5.0, True).astype(np.float32).ravel()
        assert np.abs(a - ref).max() < TOL, "call %d: max |noalloc - oracle| = %.4g" % (call, np.abs(a - ref).max())
    plan.close()


@gpu
@pytest.mark.parametrize("T,B,I,H,dbl", [(2, 128, 512, 512, 1), (4, 128, 40, 256, 0), (16, 3, 8, 64, 1)])
def test_noalloc_lstm_at_the_limits_of_the_fixed_scratch(env, T, B, I, H, dbl):
    """The largest batch and hidden size the fixed scratch admits, the single-bias blob, and an input width that is a
    multiple of 8 but not of 32 (the projection kernel's tile edge): against the oracle and the plan-based entry point."""
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    from ai_gamer_b200 import synth as SY
    from oracle import oracle as O

    lib = pk.lib()
    rng = np.random.default_rng(T * 31 + B)
    blob = SY.make_lstm_blob(rng, I, H, 1, bool(dbl), 1.0)
    x = rng.standard_normal((T, B, I)).astype(np.float16)
    want = O.lstm(x, blob, H, 1, 5.0, bool(dbl)).astype(np.float32).ravel()
    d_blob, dx = U.dev(blob), U.dev(x)
    got = torch.full((T * B * H,), 3.0, dtype=torch.float16, device="cuda")
    rc = lib.aig_lstm_forward_noalloc(c.handle, pk.ptr(dx), pk.ptr(d_blob), pk.ptr(got), T, B, I, H, 5.0, dbl)
    assert rc == 0, lib.aig_last_error(c.handle).decode()
    c.sync()
    a = U.host(got).astype(np.float32)
    assert np.abs(a - want).max() < TOL
    if I % 16 == 0:
        plan = pk.LstmPlan(c, T, 1, H, B, I, clip=5.0, double_bias=bool(dbl))
        plan.set_weights(d_blob)
        ref = torch.zeros(T * B * H, dtype=torch.float16, device="cuda")
        plan.forward(dx, ref)
        c.sync()
        assert np.abs(a - U.host(ref).astype(np.float32)).max() < TOL
        plan.close()


@gpu
def test_noalloc_lstm_rejects_shapes_beyond_the_fixed_scratch(env):
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    lib = pk.lib()
    t = torch.zeros(16, dtype=torch.float16, device="cuda")
    # 64 * 128 * 4 * 512 floats is far beyond the 2 MiB projection scratch
    rc = lib.aig_lstm_forward_noalloc(c.handle, pk.ptr(t), pk.ptr(t), pk.ptr(t), 64, 128, 512, 512, 5.0, 1)
    assert rc == -4
    assert b"exceeds the fixed scratch" in lib.aig_last_error(c.handle)
    rc = lib.aig_lstm_forward_noalloc(c.handle, pk.ptr(t), pk.ptr(t), pk.ptr(t), 1, 129, 64, 64, 5.0, 1)
    assert rc == -4 and b"batch" in lib.aig_last_error(c.handle)
    rc = lib.aig_lstm_forward_noalloc(c.handle, pk.ptr(t), pk.ptr(t), pk.ptr(t), 1, 1, 64, 1024, 5.0, 1)
    assert rc == -4 and b"hidden" in lib.aig_last_error(c.handle)
