"""The training step's kernels outside the layers' own Backward (Train.cpp:60-109): losses, loss gradient, NaN
check, activation backward passes, bias gradient and the SGD / AdamW updates, three ways where the reference has
the kernel -- the reference's own CudaStuff.cu (compiled as oracle/_ref/libaig_refcuda.so), this library, numpy."""
import ctypes

import numpy as np
import pytest

gpu = pytest.mark.gpu
f16, f32 = np.float16, np.float32


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_util as U

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return U


def _ref(U):
    ref = U.ref_cuda()
    if ref is not None:
        ref.MseLoss2.restype = None
    return ref


@gpu
def test_losses_gradient_and_nan_check(env):
    U = env
    import torch

    c, pk = U.ctx(), U.pkg()
    lib, ref = pk.lib(), _ref(U)
    rng = np.random.default_rng(21)
    batch, n_ctrls, n_but = 40, 16, 14                                    # NN.cpp:12, Train.cpp:70-76
    pred = rng.random((batch, n_ctrls)).astype(f16)
    tgt = np.concatenate([rng.integers(0, 2, (batch, n_but)), rng.standard_normal((batch, 2)) * 0.1], axis=1).astype(f32)
    dp, dt = U.dev(pred), U.dev(tgt)
    b, a = ctypes.c_float(), ctypes.c_float()
    assert lib.aig_mse_loss2(c.handle, pk.ptr(dp), pk.ptr(dt), n_but, n_ctrls, batch, ctypes.byref(b), ctypes.byref(a)) == 0
    d = (pred.astype(np.float64) - tgt) ** 2
    assert abs(b.value - d[:, :n_but].mean()) < 1e-6 * max(1.0, d[:, :n_but].mean())
    assert abs(a.value - d[:, n_but:].mean()) < 1e-6 * max(1.0, d[:, n_but:].mean())
    if ref is not None:
        rb, ra = ctypes.c_float(), ctypes.c_float()
        ref.MseLoss2(U.p(dp), U.p(dt), ctypes.c_int(n_but), ctypes.c_int(n_ctrls), ctypes.c_int(batch), ctypes.byref(rb), ctypes.byref(ra))
        assert abs(rb.value - b.value) < 1e-5 * max(1.0, abs(b.value)) and abs(ra.value - a.value) < 1e-5 * max(1.0, abs(a.value))
    # gradient = prediction - target in half arithmetic
    th = tgt.astype(f16)
    dth, dg = U.dev(th), torch.zeros(batch * n_ctrls, dtype=torch.float16, device="cuda")
    assert lib.aig_loss_gradient(c.handle, pk.ptr(dg), pk.ptr(dp), pk.ptr(dth), batch * n_ctrls) == 0
    c.sync()
    assert np.array_equal(U.host(dg).reshape(batch, n_ctrls), (pred - th).astype(f16))
    if ref is not None:
        rg = torch.zeros_like(dg)
        ref.Gradient(U.p(rg), U.p(dp), U.p(dth), ctypes.c_int(batch * n_ctrls))
        torch.cuda.synchronize()
        assert torch.equal(rg, dg)
    # NaN check
    found = ctypes.c_int(7)
    assert lib.aig_any_nan_half(c.handle, pk.ptr(dp), batch * n_ctrls, ctypes.byref(found)) == 0 and found.value == 0
    bad = pred.copy().ravel()
    bad[333] = np.nan
    assert lib.aig_any_nan_half(c.handle, pk.ptr(U.dev(bad)), bad.size, ctypes.byref(found)) == 0 and found.value == 1


@gpu
def test_activation_backward_passes_match_the_reference_kernels(env):
    U = env
    import torch

    c, pk = U.ctx(), U.pkg()
    lib, ref = pk.lib(), _ref(U)
    rng = np.random.default_rng(22)
    n = 40 * 16 * 37 + 5
    g = (rng.standard_normal(n) * 2).astype(f16)
    x = (rng.standard_normal(n) * 3).astype(f16)
    y_sig = (1.0 / (1.0 + np.exp(-x.astype(f32)))).astype(f16)
    cases = [
        ("swish", lambda dg, dx: lib.aig_swish_backward(c.handle, pk.ptr(dg), pk.ptr(dx), n), x,
         lambda dg, dx: ref.SwishBackward(U.p(dg), U.p(dx), ctypes.c_int(n)),
         lambda: g.astype(f32) * (x.astype(f32) + np.divide(x.astype(f32), 1 + x.astype(f32), out=np.full(n, np.inf, f32), where=(1 + x.astype(f32)) != 0) * (1 - x.astype(f32)))),
        ("leaky", lambda dg, dx: lib.aig_leaky_relu_backward(c.handle, pk.ptr(dg), pk.ptr(dx), n, 0.01), x,
         lambda dg, dx: ref.LeakyReluBackward(U.p(dg), U.p(dx), ctypes.c_int(n), ctypes.c_float(0.01)),
         lambda: g.astype(f32) * np.where(x < 0, f32(f16(0.01)), f32(1))),
        ("sigmoid", lambda dg, dx: lib.aig_sigmoid_backward(c.handle, pk.ptr(dg), pk.ptr(dx), 16, 14, n), y_sig,
         lambda dg, dx: ref.SigmoidBackward(U.p(dg), U.p(dx), ctypes.c_int(16), ctypes.c_int(14), ctypes.c_int(n)),
         lambda: np.where(np.arange(n) % 16 < 14, g.astype(f32) * y_sig.astype(f32) * (1 - y_sig.astype(f32)), g.astype(f32))),
    ]
    for name, ours, data, theirs, numpy_def in cases:
        dg, dx = U.dev(g), U.dev(data)
        assert ours(dg, dx) == 0, name
        c.sync()
        got = U.host(dg)
        want = numpy_def()
        fin = np.isfinite(want) & (np.abs(want) < 6e4)
        assert np.allclose(got.astype(f32)[fin], want[fin], rtol=2e-3, atol=2e-3), name
        if ref is not None:
            rg = U.dev(g)
            theirs(rg, dx)
            torch.cuda.synchronize()
            a, b = U.host(rg), got
            assert np.array_equal(a.view(np.uint16)[fin], b.view(np.uint16)[fin]), name + ": differs from the reference's kernel"


@gpu
def test_bias_gradient_sums_over_the_batch(env):
    U = env
    import torch

    c, pk = U.ctx(), U.pkg()
    rng = np.random.default_rng(23)
    for (batch, ch) in ((40, 16), (7, 300), (128, 1024)):
        g = rng.standard_normal((batch, ch)).astype(f16)
        out = torch.zeros(ch, dtype=torch.float16, device="cuda")
        assert pk.lib().aig_bias_gradient(c.handle, pk.ptr(U.dev(g)), pk.ptr(out), ch, batch) == 0
        c.sync()
        acc = np.zeros(ch, f32)
        for i in range(batch):
            acc += g[i].astype(f32)
        assert np.array_equal(U.host(out), acc.astype(f16))


@gpu
def test_sgd_and_adamw_updates_are_bit_identical_with_the_reference_kernels(env):
    U = env
    import torch

    c, pk = U.ctx(), U.pkg()
    lib, ref = pk.lib(), _ref(U)
    rng = np.random.default_rng(24)
    n = 100_003
    p0 = (rng.standard_normal(n) * 0.1).astype(f32)
    g0 = (rng.standard_normal(n) * np.where(rng.random(n) < 0.01, 500.0, 1.0)).astype(f32)   # a few beyond the clip
    lr, wd = 1e-3, 0.01
    # numpy definitions (fp32 parameters): decoupled decay, clip at 128, AdamW with bias correction
    gc = np.clip(g0, -128, 128)
    want_sgd = p0 * f32(1 - wd) - f32(lr) * gc
    dp, dg = U.dev(p0), U.dev(g0)
    assert lib.aig_sgd_step_f32(c.handle, pk.ptr(dp), pk.ptr(dg), n, lr, wd) == 0
    c.sync()
    assert np.allclose(U.host(dp), want_sgd, rtol=1e-6, atol=1e-7)
    if ref is not None:
        rp = U.dev(p0)
        ref.SGDFloat(U.p(rp), U.p(dg), ctypes.c_int(n), ctypes.c_float(lr), ctypes.c_float(wd))
        torch.cuda.synchronize()
        assert torch.equal(rp, dp), "SGDFloat"
    # three AdamW steps, fp32 and fp16 state
    for half in (False, True):
        dt = f16 if half else f32
        ours = [U.dev(a.astype(dt)) for a in (p0, np.zeros(n), np.zeros(n))]
        theirs = [U.dev(a.astype(dt)) for a in (p0, np.zeros(n), np.zeros(n))]
        m = np.zeros(n, np.float64); v = np.zeros(n, np.float64); w = p0.astype(dt).astype(np.float64)
        for t in (1, 2, 3):
            g = (g0 * f32(1.0 / t)).astype(dt)
            dgt = U.dev(g)
            fn = lib.aig_adamw_step_f16 if half else lib.aig_adamw_step_f32
            assert fn(c.handle, pk.ptr(ours[0]), pk.ptr(dgt), pk.ptr(ours[1]), pk.ptr(ours[2]), n, lr, t, wd) == 0
            c.sync()
            if ref is not None:
                rf = ref.AdamWHalf if half else ref.AdamWFloat
                rf(U.p(theirs[0]), U.p(dgt), U.p(theirs[1]), U.p(theirs[2]), ctypes.c_float(lr), ctypes.c_int(t), ctypes.c_float(wd), ctypes.c_int(n))
                torch.cuda.synchronize()
                for a, b, what in zip(ours, theirs, ("parameters", "first moment", "second moment")):
                    assert torch.equal(a, b), "AdamW %s step %d: %s differ from the reference's kernel" % ("half" if half else "float", t, what)
            gcl = np.clip(g.astype(np.float64), -128, 128)
            m = 0.9 * m + 0.1 * gcl
            v = 0.999 * v + 0.001 * gcl * gcl
            if half:
                m = m.astype(f16).astype(np.float64); v = v.astype(f16).astype(np.float64)
            w = w * (1 - wd) - lr * (m / (1 - 0.9 ** t)) / (np.sqrt(v / (1 - 0.999 ** t)) + 1e-7)
            if half:
                w = w.astype(f16).astype(np.float64)
        if not half:   # (fp16 moments underflow for small gradients and make the step ill-conditioned: the half variant is pinned by the reference's kernel above)
            assert np.allclose(U.host(ours[0]).astype(np.float64), w, rtol=1e-5, atol=1e-5), "AdamW against the numpy definition"
        else:
            assert ref is None or np.isfinite(U.host(ours[0]).astype(np.float64)).mean() > 0.99
    # SGD on half parameters
    ph, gh = p0.astype(f16), g0.astype(f16)
    dph, dgh = U.dev(ph), U.dev(gh)
    assert lib.aig_sgd_step_f16(c.handle, pk.ptr(dph), pk.ptr(dgh), n, lr, wd) == 0
    c.sync()
    if ref is not None:
        rph = U.dev(ph)
        ref.SGDHalf(U.p(rph), U.p(dgh), ctypes.c_int(n), ctypes.c_float(lr), ctypes.c_float(wd))
        torch.cuda.synchronize()
        assert torch.equal(rph, dph), "SGDHalf"
    wantp = (ph * f16(1 - wd)).astype(f32) - f32(lr) * np.clip(gh.astype(f32), -128, 128)
    assert np.allclose(U.host(dph).astype(f32), wantp, rtol=2e-3, atol=1e-4)
