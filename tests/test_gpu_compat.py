"""The reference's launcher names exported by libaig_b200.so (include/aig_compat.h) against the reference's
own CudaStuff.cu compiled as oracle/_ref/libaig_refcuda.so: same names, same arguments, same results."""
import ctypes

import numpy as np
import pytest

from oracle import oracle as O

gpu = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_util as U

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return U


@gpu
def test_reference_named_launchers(env):
    U = env
    import torch

    lib = U.pkg().lib()
    ref = U.ref_cuda()
    rng = np.random.default_rng(77)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    lib.InitCUDA()
    assert lib.aig_compat_last_status() == 0 and lib.aig_compat_context()
    sides = [("ours", lib)] + ([("reference", ref)] if ref is not None else [])

    def both(fn):
        out = {}
        for name, L in sides:
            torch.cuda.synchronize()      # both libraries launch on the legacy default stream
            out[name] = fn(L)
            torch.cuda.synchronize()
        return out

    # frame preprocessing
    n = 5003
    bgra = rng.integers(0, 256, 4 * n, dtype=np.uint8)
    d_src = U.dev(bgra)

    def pre(L):
        planar = torch.zeros(3 * n, dtype=torch.uint8, device="cuda")
        packed = torch.zeros(3 * n, dtype=torch.uint8, device="cuda")
        half = torch.zeros(3 * n, dtype=torch.float16, device="cuda")
        back = torch.zeros(3 * n, dtype=torch.uint8, device="cuda")
        f32 = torch.zeros(3 * n, dtype=torch.float32, device="cuda")
        assert L.ARGBtoRGBplanar(P(d_src), P(planar), ctypes.c_int(n)) == 0
        assert L.ARGBtoRGB(P(d_src), P(packed), ctypes.c_int(n)) == 0
        L.ConvertAndNormalize(P(half), P(planar), ctypes.c_size_t(3 * n))
        L.UnConvertAndUnNormalize(P(back), P(half), ctypes.c_size_t(3 * n))
        L.ConvertHalfToFloat(P(half), P(f32), ctypes.c_size_t(3 * n))
        return [U.host(t) for t in (planar, packed, half.view(torch.int16), back, f32)]

    r = both(pre)
    want_planar = O.bgra_to_planar(bgra, n)
    assert np.array_equal(r["ours"][0], want_planar)
    assert np.array_equal(r["ours"][1], bgra.reshape(n, 4)[:, :3].reshape(-1))       # packed B,G,R (CudaStuff.cu:52-58)
    assert np.array_equal(r["ours"][2].view(np.uint16), O.convert_normalize(want_planar).view(np.uint16))
    if "reference" in r:
        for a, b in zip(r["ours"], r["reference"]):
            assert np.array_equal(a, b)

    # activations, in place
    m = 4099
    x = np.concatenate([rng.standard_normal(m - 2) * 4, [0.0, -65504.0]]).astype(np.float32).astype(np.float16)

    def acts(L):
        outs = []
        for call in (lambda d: L.SwishForward(P(d), ctypes.c_int(m)), lambda d: L.LeakyReluForward(P(d), ctypes.c_int(m), ctypes.c_float(0.01)),
                     lambda d: L.SigmoidForward(P(d), ctypes.c_int(16), ctypes.c_int(14), ctypes.c_int(m))):
            d = U.dev(x)
            call(d)
            torch.cuda.synchronize()
            outs.append(U.host(d).view(np.uint16))
        return outs

    r = both(acts)
    assert np.array_equal(r["ours"][1], O.leaky_relu(x, 0.01).view(np.uint16))
    if "reference" in r:
        for a, b in zip(r["ours"], r["reference"]):
            assert np.array_equal(a, b)

    # weight initialisation: the distribution of the reference's HeInit (N(0, 2/fanIn)), seeded and repeatable per call index
    w = torch.zeros(1 << 16, dtype=torch.float16, device="cuda")
    lib.HeInit(P(w), ctypes.c_int(w.numel()), ctypes.c_float(50.0))
    torch.cuda.synchronize()
    hw = U.host(w).astype(np.float64)
    assert abs(hw.mean()) < 3e-3 and abs(hw.std() - np.sqrt(2.0 / 50.0)) < 3e-3
