"""GPU parity for the tcgen05 implicit-GEMM kernel (convolution 2-D/3-D and fully connected) and the
first-layer convolutions, through the C ABI, against the CPU oracle on seeded inputs."""
import numpy as np
import pytest

from oracle import oracle as O
from oracle import pipelines as PL

gpu = pytest.mark.gpu
RNG = np.random.default_rng(2024)


def h(a):
    return np.asarray(a, np.float32).astype(np.float16)


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_util as U

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return U


CONV2D = [
    # B, C, H, W, K, k, s, p
    (2, 32, 16, 32, 64, 4, 2, 1),     # 64-byte swizzle, stride 2 (ResConv main conv geometry)
    (2, 64, 8, 16, 64, 3, 1, 1),      # 128-byte swizzle, stride 1
    (3, 32, 18, 20, 64, 2, 2, 0),     # shortcut geometry, ragged row tiles
    (1, 128, 9, 16, 256, 3, 1, 1),    # N tile 256, odd height
    (2, 16, 7, 9, 24, 3, 1, 1),       # 32-byte swizzle, odd extents, out_c not a tile multiple
    (1, 64, 5, 5, 18, 3, 2, 1),       # out_c % 8 != 0 (scalar store path)
    (1, 256, 4, 8, 512, 1, 1, 0),     # two N tiles
    (5, 64, 36, 64, 128, 4, 2, 1),    # several M tiles per CTA
]


@gpu
@pytest.mark.parametrize("B,C,H,W,K,k,s,p", CONV2D)
def test_conv2d_two_step_matches_reference_roundings(env, B, C, H, W, K, k, s, p):
    """ConvLayer::Forward semantics: half(conv) then half(+bias) (ConvLayer.cpp:76-77)."""
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    x = h(RNG.standard_normal((B, C, H, W)))
    w = PL.he_normal(RNG, (K, C, k, k))
    b = h(RNG.uniform(-0.5, 0.5, K))
    want = O.conv2d(x, w, b, s, p)
    plan = pk.ConvPlan(c, B, C, H, W, K, k, s, p, act=pk.ACT_NONE, two_step=True)
    assert plan.out_dims()[1:] == want.shape[2:]
    plan.set_weights(U.dev(w), U.dev(b))
    dx = U.dev(U.nhwc(x))
    dy = torch.zeros(want.size, dtype=torch.float16, device="cuda")
    plan.forward(dx, dy)
    c.sync()
    got = U.nchw(U.host(dy).reshape(B, want.shape[2], want.shape[3], K))
    U.assert_two_step(got, want, b.reshape(1, K, 1, 1), what="conv2d two-step")
    plan.close()


@gpu
@pytest.mark.parametrize("act", [0, 1, 2, 3])
def test_conv2d_fused_bn_act_residual(env, act):
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    B, C, H, W, K = 2, 64, 12, 16, 128
    x = h(RNG.standard_normal((B, C, H, W)))
    w = PL.he_normal(RNG, (K, C, 3, 3))
    b = h(RNG.uniform(-0.2, 0.2, K))
    bn = PL.bn_params(RNG, K, trivial=False)
    res = h(RNG.standard_normal((B, K, H, W)))
    m = O.batchnorm(O.conv2d(x, w, b, 1, 1), *bn)
    want_plain = O.activate(m, act, 0.01)
    want_res = O.activate(O.add(m, res), act, 0.01)
    plan = pk.ConvPlan(c, B, C, H, W, K, 3, 1, 1, act=act, slope=0.01)
    plan.set_weights(U.dev(w), U.dev(b), bn=[U.dev(q) for q in bn], eps=1e-6)
    dx = U.dev(U.nhwc(x))
    dy = torch.zeros(want_plain.size, dtype=torch.float16, device="cuda")
    plan.forward(dx, dy)
    c.sync()
    got = U.nchw(U.host(dy).reshape(B, H, W, K))
    # one rounding here vs four in the layer-by-layer reference chain: a few fp16 ulps (2^-10 each)
    assert U.scaled_err(got, want_plain) < 6e-3
    plan.forward(dx, dy, residual=U.dev(U.nhwc(res)))
    c.sync()
    got = U.nchw(U.host(dy).reshape(B, H, W, K))
    assert U.scaled_err(got, want_res) < 6e-3
    plan.close()


@gpu
def test_conv3d(env):
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    for (B, C, D, H, W, K) in [(1, 32, 4, 8, 16, 64), (2, 64, 3, 6, 10, 128)]:
        x = h(RNG.random((B, C, D, H, W)))
        w = PL.he_normal(RNG, (K, C, 3, 3, 3))
        b = h(RNG.uniform(-0.2, 0.2, K))
        want = O.conv3d(x, w, b, 1, 2, 1, 1)
        plan = pk.ConvPlan(c, B, C, H, W, K, 3, 2, 1, two_step=True, in_d=D, kd=3, sd=1, pd=1)
        assert plan.out_dims() == want.shape[2:]
        plan.set_weights(U.dev(w), U.dev(b))
        dy = torch.zeros(want.size, dtype=torch.float16, device="cuda")
        plan.forward(U.dev(U.nhwc(x)), dy)
        c.sync()
        got = U.nchw(U.host(dy).reshape(B, *want.shape[2:], K))
        U.assert_two_step(got, want, b.reshape(1, K, 1, 1, 1), what="conv3d")
        plan.close()


@gpu
@pytest.mark.parametrize("rows,inC,outC", [(64, 1024, 1024), (1, 256, 18), (200, 512, 2048), (129, 64, 40), (32, 256, 512)])
def test_fc_two_step(env, rows, inC, outC):
    """FCLayer::Forward: half(x.W) then half(+bias) (FCLayer.cpp:50-51)."""
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    x = h(RNG.standard_normal((rows, inC)))
    W = h(RNG.standard_normal((inC, outC)) / np.sqrt(inC))
    b = h(RNG.uniform(-0.5, 0.5, outC))
    want = O.fc(x, W, b)
    plan = pk.FcPlan(c, rows, inC, outC, two_step=True)
    plan.set_weights(U.dev(W), U.dev(b))
    dy = torch.zeros(rows * outC, dtype=torch.float16, device="cuda")
    plan.forward(U.dev(x), dy)
    c.sync()
    U.assert_two_step(U.host(dy).reshape(rows, outC), want, b.reshape(1, outC), what="fc")
    plan.close()


@gpu
def test_fc_fused_per_activation_bn_relu(env):
    """FC -> BatchNorm(per activation) -> ReLU as NN.cpp:45-47 chains them."""
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    rows, inC, outC = 40, 512, 256
    x = h(RNG.standard_normal((rows, inC)))
    W = h(RNG.standard_normal((inC, outC)) / np.sqrt(inC))
    b = h(RNG.uniform(-0.5, 0.5, outC))
    bn = PL.bn_params(RNG, outC, trivial=False)
    want = O.relu(O.batchnorm(O.fc(x, W, b), *bn, per_activation=True))
    plan = pk.FcPlan(c, rows, inC, outC, act=pk.ACT_RELU)
    plan.set_weights(U.dev(W), U.dev(b), bn=[U.dev(q) for q in bn])
    dy = torch.zeros(rows * outC, dtype=torch.float16, device="cuda")
    plan.forward(U.dev(x), dy)
    c.sync()
    assert U.scaled_err(U.host(dy).reshape(rows, outC), want) < 4e-3
    plan.close()


@gpu
def test_first_layer_convs(env):
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    # 2-D, from BGRA bytes (fused preprocessing) and from planar fp16
    # k = 5, 2, 3 run on the tensor-core gather kernel; k = 4 has no instantiation and takes the CUDA-core kernel
    for (B, H, W, K, k, s, p) in [(2, 144, 256, 32, 5, 2, 2), (3, 17, 23, 32, 2, 2, 0), (1, 20, 31, 40, 3, 1, 1),
                                  (2, 18, 22, 32, 4, 2, 1), (1, 33, 47, 18, 5, 2, 2)]:
        frames = PL.make_frames(5, B, H, W)
        w = PL.he_normal(RNG, (K, 3, k, k))
        b = h(RNG.uniform(-0.2, 0.2, K))
        bn = PL.bn_params(RNG, K, trivial=False)
        x = O.preprocess_frames(frames)
        want = O.swish(O.batchnorm(O.conv2d(x, w, b, s, p), *bn))
        plan = pk.Conv0Plan(c, B, H, W, K, k, s, p, act=pk.ACT_SWISH)
        plan.set_weights(U.dev(w), U.dev(b), bn=[U.dev(q) for q in bn])
        dy = torch.zeros(want.size, dtype=torch.float16, device="cuda")
        plan.forward_bgra(U.dev(frames), dy)
        c.sync()
        got = U.nchw(U.host(dy).reshape(B, want.shape[2], want.shape[3], K))
        assert U.scaled_err(got, want) < 4e-3
        dy.zero_()
        plan.forward_nchw(U.dev(x), dy)
        c.sync()
        got2 = U.nchw(U.host(dy).reshape(B, want.shape[2], want.shape[3], K))
        assert np.array_equal(got, got2)
        plan.close()
    # 3-D first layer
    B, D, H, W, K = 1, 4, 12, 20, 32
    x = PL.make_clips(1, B, D, H, W)
    w = PL.he_normal(RNG, (K, 3, 3, 3, 3))
    b = h(RNG.uniform(-0.2, 0.2, K))
    want = O.leaky_relu(O.conv3d(x, w, b, 1, 2, 1, 1), 0.01)
    plan = pk.Conv0Plan(c, B, H, W, K, 3, 2, 1, act=pk.ACT_LEAKY, slope=0.01, in_d=D, kd=3, sd=1, pd=1)
    plan.set_weights(U.dev(w), U.dev(b))
    dy = torch.zeros(want.size, dtype=torch.float16, device="cuda")
    plan.forward_nchw(U.dev(x), dy)
    c.sync()
    got = U.nchw(U.host(dy).reshape(B, *want.shape[2:], K))
    assert U.scaled_err(got, want) < 4e-3
    plan.close()
