"""GPU parity: preprocessing, conversions, activations, BatchNorm, LayerNorm, spatial attention and
pooling kernels, called through the C ABI, against the CPU oracle -- and, where the reference ships
the kernel itself (CudaStuff.cu), against the reference's own kernel compiled from its source."""
import ctypes

import numpy as np
import pytest

from oracle import oracle as O

gpu = pytest.mark.gpu
RNG = np.random.default_rng(123)


def h(a):
    return np.asarray(a, np.float32).astype(np.float16)


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_util as U

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return U


@gpu
def test_preprocess_bit_exact(env):
    U = env
    import torch

    c = U.ctx()
    for n in (256 * 144, 37 * 5, 1):
        bgra = RNG.integers(0, 256, 4 * n, dtype=np.uint8)
        d_src = U.dev(bgra)
        d_planar = torch.empty(3 * n, dtype=torch.uint8, device="cuda")
        c.call("aig_bgra_to_planar", U.p(d_src), U.p(d_planar), n)
        want_planar = O.bgra_to_planar(bgra, n)
        assert np.array_equal(U.host(d_planar), want_planar)
        d_half = torch.empty(3 * n, dtype=torch.float16, device="cuda")
        c.call("aig_convert_normalize", U.p(d_half), U.p(d_planar), 3 * n)
        want_half = O.convert_normalize(want_planar)
        assert np.array_equal(U.host(d_half).view(np.uint16), want_half.view(np.uint16))
        # fused frames entry point (2 frames)
        if n % 2 == 0:
            d_out = torch.empty(3 * n, dtype=torch.float16, device="cuda")
            c.call("aig_preprocess_bgra", U.p(d_src), U.p(d_out), 2, n // 2)
            want = np.concatenate([O.convert_normalize(O.bgra_to_planar(bgra[:2 * n], n // 2)),
                                   O.convert_normalize(O.bgra_to_planar(bgra[2 * n:], n // 2))])
            assert np.array_equal(U.host(d_out).view(np.uint16), want.view(np.uint16))
        # back to bytes
        d_u8 = torch.empty(3 * n, dtype=torch.uint8, device="cuda")
        c.call("aig_unconvert_unnormalize", U.p(d_u8), U.p(d_half), 3 * n)
        assert np.array_equal(U.host(d_u8), O.unconvert_unnormalize(want_half))
        ref = U.ref_cuda()
        if ref is not None:
            r_planar = torch.zeros(3 * n, dtype=torch.uint8, device="cuda")
            r_half = torch.zeros(3 * n, dtype=torch.float16, device="cuda")
            torch.cuda.synchronize()  # the reference launches on the legacy default stream
            ref.ARGBtoRGBplanar(U.p(d_src), U.p(r_planar), ctypes.c_int(n))
            ref.ConvertAndNormalize(U.p(r_half), U.p(r_planar), ctypes.c_size_t(3 * n))
            torch.cuda.synchronize()
            assert np.array_equal(U.host(r_planar), U.host(d_planar)), "differs from reference ARGBtoRGBplanar"
            assert np.array_equal(U.host(r_half).view(np.uint16), U.host(d_half).view(np.uint16)), \
                "differs from reference ConvertAndNormalize"
    c.sync()


@gpu
def test_conversions_and_layout(env):
    U = env
    import torch

    c = U.ctx()
    x = h(RNG.standard_normal(1000) * 3)
    d = U.dev(x)
    f = torch.empty(1000, dtype=torch.float32, device="cuda")
    c.call("aig_half_to_float", U.p(d), U.p(f), 1000)
    assert np.array_equal(U.host(f), x.astype(np.float32))
    back = torch.empty(1000, dtype=torch.float16, device="cuda")
    c.call("aig_float_to_half", U.p(f), U.p(back), 1000)
    assert np.array_equal(U.host(back), x)
    t = h(RNG.standard_normal((3, 37, 5, 11)))
    dn = U.dev(t)
    dl = torch.empty(3 * 37 * 55, dtype=torch.float16, device="cuda")
    c.call("aig_nchw_to_nhwc", U.p(dn), U.p(dl), 3, 37, 55)
    assert np.array_equal(U.host(dl).reshape(3, 5, 11, 37), U.nhwc(t))
    dn2 = torch.empty_like(dn)
    c.call("aig_nhwc_to_nchw", U.p(dl), U.p(dn2), 3, 37, 55)
    assert np.array_equal(U.host(dn2), t)
    c.sync()


@gpu
@pytest.mark.parametrize("n", [8 * 1024 + 3, 7, 64 * 1024])
def test_activations_vs_oracle_and_reference(env, n):
    U = env
    c = U.ctx()
    x = h(np.concatenate([RNG.standard_normal(n - 4) * 4, [0.0, -0.0, 65504.0, -65504.0]]))
    ref = U.ref_cuda()
    cases = [
        ("swish", lambda d: c.call("aig_swish_forward", U.p(d), n), O.swish, lambda d: ref.SwishForward(U.p(d), ctypes.c_int(n))),
        ("leaky", lambda d: c.call("aig_leaky_relu_forward", U.p(d), n, 0.01), lambda a: O.leaky_relu(a, 0.01),
         lambda d: ref.LeakyReluForward(U.p(d), ctypes.c_int(n), ctypes.c_float(0.01))),
        ("leaky128", lambda d: c.call("aig_leaky_relu_forward", U.p(d), n, 1.0 / 128), lambda a: O.leaky_relu(a, 1.0 / 128),
         lambda d: ref.LeakyReluForward(U.p(d), ctypes.c_int(n), ctypes.c_float(1.0 / 128))),
        ("relu", lambda d: c.call("aig_relu_forward", U.p(d), n), O.relu, None),
        ("sigmoid", lambda d: c.call("aig_sigmoid_forward", U.p(d), 16, 14, n), lambda a: O.sigmoid_head(a, 16, 14),
         lambda d: ref.SigmoidForward(U.p(d), ctypes.c_int(16), ctypes.c_int(14), ctypes.c_int(n))),
        ("tanh", lambda d: c.call("aig_tanh_tail_forward", U.p(d), 18, 16, n), lambda a: O.tanh_tail(a, 18, 16), None),
    ]
    import torch

    for name, ours, oracle_fn, ref_fn in cases:
        d = U.dev(x)
        ours(d)
        c.sync()
        got = U.host(d)
        # expf on the device and in glibc can differ in the last fp32 bit: allow one fp16 ulp vs the CPU oracle
        U.assert_close16(got, oracle_fn(x), max_ulp=1, frac_exact=0.995, what=name + " vs oracle")
        if ref is not None and ref_fn is not None:
            r = U.dev(x)
            torch.cuda.synchronize()
            ref_fn(r)
            torch.cuda.synchronize()
            assert np.array_equal(U.host(r).view(np.uint16), got.view(np.uint16)), name + " differs from the reference kernel"


@gpu
def test_add_and_batchnorm(env):
    U = env
    import torch

    c = U.ctx()
    n = 5000
    a, b = h(RNG.standard_normal(n)), h(RNG.standard_normal(n))
    da, db = U.dev(a), U.dev(b)
    c.call("aig_add_forward", U.p(da), U.p(db), n)
    assert np.array_equal(U.host(da), O.add(a, b))
    from oracle import pipelines as PL

    for (B, C, HW, per_act) in [(3, 6, 20, 0), (2, 16, 8 * 16, 0), (4, 10, 1, 1), (2, 3, 7, 1)]:
        x = h(RNG.standard_normal((B, C, HW)))
        prm = PL.bn_params(RNG, C * HW if per_act else C, trivial=False)
        dx = U.dev(x)
        dy = torch.empty_like(dx)
        dp = [U.dev(q) for q in prm]
        c.call("aig_batchnorm_forward", U.p(dx), U.p(dy), *[U.p(q) for q in dp], B, C, HW, 1e-6, per_act)
        want = O.batchnorm(x, *prm, eps=1e-6, per_activation=bool(per_act))
        U.assert_close16(U.host(dy), want, max_ulp=1, frac_exact=0.98, what="batchnorm", atol=1e-3)
    c.sync()


@gpu
def test_layernorm_reference_axis(env):
    U = env
    import torch

    c = U.ctx()
    ref = U.ref_cuda()
    for (N, C, HW) in [(4, 6, 100), (64, 1024, 1), (2, 3, 640), (3, 70, 64)]:
        x = h(RNG.standard_normal((N, C, HW)) * 2 + 0.3)
        g = RNG.uniform(0.5, 1.5, C).astype(np.float32)
        b = RNG.uniform(-1, 1, C).astype(np.float32)
        dx, dg, db = U.dev(x), U.dev(g), U.dev(b)
        dy = torch.empty_like(dx)
        dm = torch.zeros(C, dtype=torch.float32, device="cuda")
        dv = torch.zeros(C, dtype=torch.float32, device="cuda")
        c.call("aig_layernorm_forward", U.p(dy), U.p(dx), U.p(dg), U.p(db), U.p(dm), U.p(dv), N, C, HW, 1e-7)
        c.sync()
        wy, wm, wv = O.layernorm_ref(x, g, b, N, C, HW, 1e-7)
        np.testing.assert_allclose(U.host(dm), wm, rtol=2e-5, atol=2e-6)
        np.testing.assert_allclose(U.host(dv), wv, rtol=2e-5, atol=1e-7)
        U.assert_close16(U.host(dy), wy, max_ulp=2, frac_exact=0.97, what="layernorm vs oracle", atol=2e-3)
        if ref is not None and HW >= 64:
            # the reference's own kernels, one block per channel (its launcher covers only ceil(C/BS) channels;
            # with fewer than blockDim samples per thread slot it merges empty partitions as 0/0)
            ry = torch.zeros_like(dx)
            rm = torch.zeros(C, dtype=torch.float32, device="cuda")
            rv = torch.zeros(C, dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()
            rc = ref.ref_layernorm_forward_fullgrid(U.p(ry), U.p(dx), U.p(dg), U.p(db), U.p(rm), U.p(rv),
                                                    ctypes.c_int(N), ctypes.c_int(C), ctypes.c_int(HW))
            torch.cuda.synchronize()
            assert rc == 0
            np.testing.assert_allclose(U.host(dm), U.host(rm), rtol=2e-5, atol=2e-6)
            np.testing.assert_allclose(U.host(dv), U.host(rv), rtol=2e-5, atol=1e-7)
            U.assert_close16(U.host(dy), U.host(ry), max_ulp=2, frac_exact=0.97, what="layernorm vs reference kernel", atol=2e-3)
            # and the reference launcher as shipped: its first ceil(C/BS) channels must agree with ours
            sy = torch.zeros_like(dx)
            sm = torch.zeros(C, dtype=torch.float32, device="cuda")
            sv = torch.zeros(C, dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()
            ref.LayerNormForward(U.p(sy), U.p(dx), U.p(dg), U.p(db), U.p(sm), U.p(sv), ctypes.c_int(N), ctypes.c_int(C),
                                 ctypes.c_int(HW))
            torch.cuda.synchronize()
            k = -(-C // 64)
            np.testing.assert_allclose(U.host(dm)[:k], U.host(sm)[:k], rtol=2e-5, atol=2e-6)
            U.assert_close16(U.host(dy)[:, :k], U.host(sy)[:, :k], max_ulp=2, what="layernorm vs reference launcher", atol=2e-3)


@gpu
def test_layernorm_rows(env):
    U = env
    import torch

    c = U.ctx()
    for rows, C in [(64, 1024), (128 * 64, 512), (5, 48), (3, 100), (7, 2048)]:
        x = h(RNG.standard_normal((rows, C)) * 1.5 + 0.2)
        g = RNG.uniform(0.5, 1.5, C).astype(np.float32)
        b = RNG.uniform(-1, 1, C).astype(np.float32)
        dx, dg, db = U.dev(x), U.dev(g), U.dev(b)
        dy = torch.empty_like(dx)
        c.call("aig_layernorm_rows_forward", U.p(dy), U.p(dx), U.p(dg), U.p(db), rows, C, 1e-5)
        c.sync()
        U.assert_close16(U.host(dy), O.layernorm_rows(x, g, b, 1e-5), max_ulp=1, frac_exact=0.98, what="row layernorm", atol=2e-3)


@gpu
def test_spatial_attention_reference_mode(env):
    U = env
    import torch

    c = U.ctx()
    ref = U.ref_cuda()
    for (B, inC, attC, H, W) in [(2, 8, 4, 4, 8), (4, 32, 9, 4, 8), (32, 256, 8, 4, 8)]:
        P = B * H * W
        x = h(RNG.standard_normal(P * inC) * 0.5)
        ws = [h(RNG.standard_normal(attC * inC) * (1.0 / np.sqrt(inC))) for _ in range(3)]
        dx = U.dev(x)
        dw = [U.dev(w) for w in ws]
        bufs = [torch.zeros(P * attC, dtype=torch.float16, device="cuda") for _ in range(3)]
        sc = torch.zeros(P, dtype=torch.float16, device="cuda")
        out = torch.zeros(P * attC, dtype=torch.float16, device="cuda")
        c.call("aig_spatial_attention_forward", U.p(dx), *[U.p(w) for w in dw], *[U.p(b) for b in bufs], U.p(sc), U.p(out),
               B, inC, attC, H, W, 64)
        c.sync()
        want = O.spatial_attention_ref(x, *ws, B, inC, attC, H, W, 64)
        assert np.array_equal(U.host(bufs[0]).reshape(P, attC), want["keyMap"])
        assert np.array_equal(U.host(bufs[1]).reshape(P, attC), want["queryMap"])
        assert np.array_equal(U.host(bufs[2]).reshape(P, attC), want["valueMap"])
        U.assert_close16(U.host(sc), want["scores"], max_ulp=1, frac_exact=0.97, what="attention scores")
        U.assert_close16(U.host(out).reshape(P, attC), want["out"], max_ulp=1, frac_exact=0.97, what="attention out")
        if ref is not None:
            rb = [torch.zeros(P * attC, dtype=torch.float16, device="cuda") for _ in range(3)]
            rs = torch.zeros(P, dtype=torch.float16, device="cuda")
            ro = torch.zeros(P * attC, dtype=torch.float16, device="cuda")
            torch.cuda.synchronize()
            ref.SpatialAttentionForward(U.p(dx), *[U.p(w) for w in dw], *[U.p(b) for b in rb], U.p(rs), U.p(ro),
                                        *[ctypes.c_int(v) for v in (B, inC, attC, H, W)])
            torch.cuda.synchronize()
            for a, b in zip(bufs, rb):
                assert np.array_equal(U.host(a).view(np.uint16), U.host(b).view(np.uint16)), "projection differs from reference"
            assert np.array_equal(U.host(sc).view(np.uint16), U.host(rs).view(np.uint16)), "scores differ from reference"
            assert np.array_equal(U.host(out).view(np.uint16), U.host(ro).view(np.uint16)), "output differs from reference"


@gpu
def test_mask_attention_and_pools(env):
    U = env
    import torch

    c = U.ctx()
    B, C, H, W = 3, 256, 4, 8
    x = h(RNG.standard_normal((B, C, H, W)))
    w1 = h(RNG.standard_normal(C) * 0.1)
    dx = U.dev(U.nhwc(x))
    dy = torch.empty_like(dx)
    c.call("aig_spatial_mask_forward", U.p(dx), U.p(U.dev(w1)), 0.1, U.p(dy), B, H * W, C)
    want = O.spatial_attention_cfg(x, w1, 0.1)
    U.assert_close16(U.host(dy), U.nhwc(want), max_ulp=1, frac_exact=0.98, what="mask attention")
    dp = torch.empty(B * C, dtype=torch.float16, device="cuda")
    c.call("aig_global_avgpool_nhwc", U.p(dy), U.p(dp), B, H * W, C)
    U.assert_close16(U.host(dp).reshape(B, C), O.global_avgpool(U.nchw(U.host(dy))), max_ulp=1, frac_exact=0.98, what="avgpool")
    x3 = h(RNG.random((2, 16, 3, 6, 10)))
    d3 = U.dev(U.nhwc(x3))
    dq = torch.empty(2 * 16 * 4, dtype=torch.float16, device="cuda")
    c.call("aig_adaptive_avgpool3d_ndhwc", U.p(d3), U.p(dq), 2, 3, 6, 10, 16, 2, 2)
    U.assert_close16(U.host(dq).reshape(2, 64), O.adaptive_avgpool3d(x3, 2, 2), max_ulp=1, frac_exact=0.98, what="adaptive pool")
    c.sync()


@gpu
def test_fc_head_one_launch(env):
    """FCLayer + Sigmoid (+ tanh tail) + ConvertHalfToFloat as one launch against the oracle's chain of the three."""
    U = env
    import torch

    c = U.ctx()
    rng = np.random.default_rng(12)
    for rows, in_c, n_out, n_sig in ((16, 512, 18, 16), (3, 256, 16, 14), (1, 1000, 7, 7)):
        x = rng.standard_normal((rows, in_c)).astype(np.float16)
        W = (rng.standard_normal((in_c, n_out)) / np.sqrt(in_c)).astype(np.float16)
        b = rng.uniform(-0.2, 0.2, n_out).astype(np.float16)
        want = O.tanh_tail(O.sigmoid_head(O.fc(x, W, b), n_out, n_sig), n_out, n_sig)
        oh = torch.zeros(rows * n_out, dtype=torch.float16, device="cuda")
        of = torch.zeros(rows * n_out, dtype=torch.float32, device="cuda")
        dx, dW, db = U.dev(x), U.dev(W), U.dev(b)
        c.call("aig_fc_head_forward", U.p(dx), U.p(dW), U.p(db), U.p(oh), U.p(of), rows, in_c, n_out, n_sig)
        c.sync()
        got = U.host(oh).reshape(rows, n_out)
        U.assert_close16(got, want, max_ulp=2, frac_exact=0.9, what="fc head")
        assert np.array_equal(U.host(of).reshape(rows, n_out), got.astype(np.float32))


@gpu
@pytest.mark.parametrize("k", [2, 3, 4])
def test_resize_box_bit_exact(env, k):
    """ConvScale::ScaleInPlace / ScaleToHalf (ConvScale.cpp:41-52) and GrabFrameScale* (NvDisplayCap.h:91-119) as one
    kernel: bit-exact against the oracle on odd sizes, from planar frames and from BGRA pixels, with the reference's
    cross-channel filter and with the per-channel box filter."""
    U = env
    import torch

    c = U.ctx()
    rng = np.random.default_rng(40 + k)
    N, H, W = 3, 37, 53
    planar = rng.integers(0, 256, (N, 3, H, W), dtype=np.uint8)
    bgra = np.zeros((N, H, W, 4), np.uint8)
    bgra[..., 2], bgra[..., 1], bgra[..., 0], bgra[..., 3] = planar[:, 0], planar[:, 1], planar[:, 2], 255
    for cross in (0, 1):
        w8, wh = O.resize_box(planar, k, cross_channel=bool(cross))
        for src, is_bgra in ((planar, 0), (bgra, 1)):
            o8 = torch.zeros(w8.size, dtype=torch.uint8, device="cuda")
            oh = torch.zeros(wh.size, dtype=torch.float16, device="cuda")
            dsrc = U.dev(src)
            c.call("aig_resize_box", U.p(dsrc), is_bgra, U.p(o8), U.p(oh), N, 3, H, W, k, cross)
            c.sync()
            assert np.array_equal(U.host(o8).reshape(w8.shape), w8)
            assert np.array_equal(U.host(oh).reshape(wh.shape).view(np.uint16), wh.view(np.uint16))
