"""FCLayer::Backward and FCLayer::UpdateParameters (FCLayer.cpp:54-70) three ways: this library (aig_fc_backward and
the FCLayer class in training mode), the CPU oracle (double accumulation), and the reference's own FCLayer class on
cuBLAS (oracle/_ref/libaig_reflayers.so, built only where the reference tree is present)."""
import ctypes
import os
import tempfile

import numpy as np
import pytest

from oracle import oracle as O

gpu = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LAYERS = os.path.join(ROOT, "oracle", "_ref", "libaig_reflayers.so")
f16 = np.float16
P = ctypes.c_void_p


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_util as U

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    U.pkg()
    return U


def _case(seed, B, I, N):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((B, I)).astype(f16)
    g = (rng.standard_normal((B, N)) * 0.1).astype(f16)
    W = (rng.standard_normal((I, N)) * np.sqrt(2.0 / I)).astype(f16)
    return x, g, W


def _check(got, want, what, frac_exact=0.99, ulps=2):
    """fp32 accumulation on the tensor cores against the oracle's double accumulation: within `ulps` fp16 ulp at the
    element's magnitude (results formed by cancellation are measured at 1/64 of the tensor's rms), almost all equal."""
    got64, want64 = np.asarray(got, np.float64), np.asarray(want, np.float64)
    rms = float(np.sqrt(np.mean(want64 * want64))) + 1e-30
    scale = np.maximum(np.abs(want64), rms / 64)
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(scale, 2.0 ** -14))) - 10)
    bad = np.abs(got64 - want64) > ulps * ulp * 1.0001
    assert not bad.any(), "%s: %d of %d beyond %d ulp" % (what, bad.sum(), bad.size, ulps)
    exact = float((got64 == want64).mean())
    assert exact >= frac_exact, "%s: only %.4f bit-exact" % (what, exact)


@gpu
@pytest.mark.parametrize("B,I,N", [(64, 1024, 1024), (32, 256, 18), (5, 40, 16), (256, 256, 512), (33, 72, 100)])
def test_fc_backward_against_oracle(env, B, I, N):
    """Weight, bias and input gradients; K extents that are not multiples of 16 (18 outputs, batch 5 / 33) go through
    the zero-padded copies."""
    U = env
    import torch

    c, pk = U.ctx(), U.pkg()
    x, g, W = _case(B * 7 + N, B, I, N)
    want_w, want_b, want_x = O.fc_backward(x, g, W)
    plan = pk.FcBackwardPlan(c, B, I, N)
    dw = torch.full((I * N,), 7.0, dtype=torch.float16, device="cuda")
    db = torch.full((N,), 7.0, dtype=torch.float16, device="cuda")
    dx = torch.full((B * I,), 7.0, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    dX, dG, dW = U.dev(x), U.dev(g), U.dev(W)
    for _ in range(2):                                 # a second call reuses the plan's operand copies
        plan.backward(dX, dG, dW, dw, db, dx)
    c.sync()
    _check(U.host(dw).reshape(I, N), want_w, "grad_w")
    _check(U.host(dx).reshape(B, I), want_x, "grad_x")
    U.assert_close16(U.host(db), want_b, max_ulp=1, what="grad_b", atol=1e-4)
    # outputs may be asked for one at a time
    dx2 = torch.zeros_like(dx)
    plan.backward(None, dG, dW, None, None, dx2)
    c.sync()
    assert torch.equal(dx2, dx)
    plan.close()


def _ref_lib():
    if not os.path.exists(REF_LAYERS):
        pytest.skip("the reference's layer classes were not built (reference tree absent at build time)")
    ref = ctypes.CDLL(REF_LAYERS)
    ref.ref_layer_create.restype = P
    ref.ref_layer_create.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    ref.ref_layer_forward.restype = P
    ref.ref_layer_forward.argtypes = [P, P]
    ref.ref_fc_backward.restype = P
    ref.ref_fc_backward.argtypes = [P, P, ctypes.POINTER(P), ctypes.POINTER(P)]
    ref.ref_layer_update.argtypes = [P, ctypes.c_float]
    ref.ref_layer_load_file.argtypes = [P, ctypes.c_char_p]
    ref.ref_layer_save_file.argtypes = [P, ctypes.c_char_p]
    ref.ref_layer_destroy.argtypes = [P]
    ref.ref_last_error.restype = ctypes.c_char_p
    assert ref.ref_init() == 0, ref.ref_last_error().decode()
    return ref


@gpu
@pytest.mark.parametrize("B,I,N", [(64, 1024, 1024), (32, 256, 16), (256, 256, 512)])
def test_fc_training_steps_against_the_reference_class(env, B, I, N):
    """Three Forward / Backward / UpdateParameters steps of FCLayer in training mode, the reference's class (cuBLAS +
    AdamWHalf) and this library's class side by side from the same payload, inputs and incoming gradients: the input
    gradient, the weight gradient and the updated weights of every step.  The bias is left out of
    the comparison: the reference's BiasGradient adds a cross-channel reduction to the per-channel sums
    (CudaStuff.cu:385-389), which this library does not reproduce."""
    U = env
    import torch

    ref = _ref_lib()
    c, pk, lib = U.ctx(), U.pkg(), U.pkg().lib()
    rng = np.random.default_rng(B + N)
    _, _, W = _case(B + I, B, I, N)
    bias = rng.uniform(-0.5, 0.5, N).astype(f16)
    payload = W.tobytes() + bias.tobytes()
    arr = (ctypes.c_int * 3)(B, I, N)
    lr = 1e-3

    def copy_out(ptr, count):
        t = torch.empty(count, dtype=torch.float16, device="cuda")
        c.call("aig_memcpy", pk.ptr(t), ctypes.c_void_p(ptr), count * 2)
        c.sync()
        return U.host(t)

    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "payload.bin")
        with open(path, "wb") as f:
            f.write(payload)
        torch.cuda.synchronize()
        rl = ref.ref_layer_create(b"FCLayerTrain", arr, 3)
        assert rl, ref.ref_last_error().decode()
        assert ref.ref_layer_load_file(rl, path.encode()) == 0, ref.ref_last_error().decode()
        ol = ctypes.c_void_p()
        assert lib.aig_layer_create(c.handle, b"FCLayerTrain", arr, 3, ctypes.byref(ol)) == 0
        assert lib.aig_layer_load_file(ol, path.encode()) == 0
        plan = pk.FcBackwardPlan(c, B, I, N)           # the class keeps its weight gradient to itself; same kernels
        w_now = W
        for step in range(3):
            x, g, _ = _case(1000 + step, B, I, N)
            dX, dG = U.dev(x), U.dev(g)
            # ---- the reference's class (legacy default stream)
            torch.cuda.synchronize()
            assert ref.ref_layer_forward(rl, pk.ptr(dX)), ref.ref_last_error().decode()
            gw_p, gb_p = P(), P()
            gx_p = ref.ref_fc_backward(rl, pk.ptr(dG), ctypes.byref(gw_p), ctypes.byref(gb_p))
            assert gx_p, ref.ref_last_error().decode()
            torch.cuda.synchronize()
            ref_gx, ref_gw = copy_out(gx_p, B * I).reshape(B, I), copy_out(gw_p.value, I * N).reshape(I, N)
            assert ref.ref_layer_update(rl, lr) == 0, ref.ref_last_error().decode()
            torch.cuda.synchronize()
            # ---- this library's class
            out = ctypes.c_void_p()
            assert lib.aig_layer_forward(ol, pk.ptr(dX), ctypes.byref(out)) == 0
            gx = ctypes.c_void_p()
            assert lib.aig_layer_backward(ol, pk.ptr(dG), ctypes.byref(gx)) == 0 and gx.value
            c.sync()
            got_gx = copy_out(gx.value, B * I).reshape(B, I)
            dgw = torch.zeros(I * N, dtype=torch.float16, device="cuda")
            torch.cuda.synchronize()
            plan.backward(dX, dG, U.dev(w_now), dgw, None, None)
            c.sync()
            got_gw = U.host(dgw).reshape(I, N)
            assert lib.aig_layer_update(ol, lr) == 0
            c.sync()
            # both accumulate in fp32 (CUDA_R_32F compute, FCLayer.cpp:55,57), in different orders
            # (after the first step the two classes hold weights that may differ in a few last bits)
            _check(got_gx, ref_gx, "grad_x vs the reference, step %d" % step, frac_exact=0.999 if step == 0 else 0.99, ulps=1)
            _check(got_gw, ref_gw, "grad_w vs the reference, step %d" % step, frac_exact=0.999, ulps=1)
            want_w, _, want_x = O.fc_backward(x, g, w_now)
            _check(ref_gx, want_x, "the reference's grad_x vs the oracle")
            _check(ref_gw, want_w, "the reference's grad_w vs the oracle")
            # the weights both classes hold after the update
            rp, op = os.path.join(d, "ref.bin"), os.path.join(d, "ours.bin")
            assert ref.ref_layer_save_file(rl, rp.encode()) == 0 and lib.aig_layer_save_file(ol, op.encode()) == 0
            rw = np.frombuffer(open(rp, "rb").read(), f16)[: I * N].reshape(I, N)
            ow = np.frombuffer(open(op, "rb").read(), f16)[: I * N].reshape(I, N)
            same = float((rw == ow).mean())
            assert same >= 0.999, "weights after step %d: only %.5f identical" % (step, same)
            # the few that differ: by one fp16 ulp at the weight's magnitude, or at the step's (lr) for a weight that
            # the update carried to near zero, where an ulp is far below the moments' own rounding
            scale = np.maximum(np.abs(rw.astype(np.float64)), lr)
            ulp = 2.0 ** (np.floor(np.log2(scale)) - 10)
            far = np.abs(rw.astype(np.float64) - ow.astype(np.float64)) > ulp * 1.0001
            assert not far.any(), "step %d: %d weights beyond one ulp" % (step, far.sum())
            assert not np.array_equal(ow, w_now), "the update changed nothing"
            w_now = ow.copy()
        plan.close()
        ref.ref_layer_destroy(rl)
        lib.aig_layer_destroy(ol)
