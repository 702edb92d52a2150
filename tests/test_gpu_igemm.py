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
                                  (2, 18, 22, 32, 4, 2, 1), (1, 33, 47, 18, 5, 2, 2),
                                  # wide rows, partial 16-pixel blocks at the right edge, k = 3 and k = 2 at stride 2
                                  (2, 40, 300, 32, 5, 2, 2), (1, 31, 200, 32, 3, 2, 1), (1, 32, 256, 32, 2, 2, 0), (3, 21, 131, 32, 5, 2, 2)]:
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
        assert U.scaled_err(got2, want) < 4e-3
        # the two entry points order the K dimension differently (different kernels): equal up to fp32 summation order
        assert np.abs(got.astype(np.float32) - got2.astype(np.float32)).max() <= 2 * np.abs(want).max() * 2.0 ** -10
        plan.close()
    # 3-D first layer: rows shorter than a warp, rows of exactly one warp, an odd width (no column pairs)
    for B, D, H, W, K in [(1, 4, 12, 20, 32), (2, 3, 9, 64, 32), (1, 2, 10, 23, 32)]:
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
        assert U.scaled_err(got, want) < 4e-3, (B, D, H, W)
        plan.close()


def _s2d_host(x_nhwc):
    """numpy restatement of the space-to-depth block layout: [B][H][W][C] -> [B][hb][wb][4][C]."""
    B, H, W, C = x_nhwc.shape
    hb, wb = (H - 2) // 2 + 2, (W - 2) // 2 + 2
    out = np.zeros((B, hb, wb, 4, C), x_nhwc.dtype)
    for y in range(H):
        for x in range(W):
            out[:, (y + 1) >> 1, (x + 1) >> 1, ((y + 1) & 1) * 2 + ((x + 1) & 1)] = x_nhwc[:, y, x]
    return out


@gpu
@pytest.mark.parametrize("B,H,W", [(2, 144, 256), (3, 32, 64), (1, 17, 48), (2, 7, 16), (5, 40, 240)])
def test_first_layer_from_uint8_frames_row_kernel(env, B, H, W):
    """The encoder's own first layer (3 -> 32, 5x5, stride 2, pad 2) on the row-resident kernel: BGRA pixels and
    planar RGB planes of the same frames give the same bytes, both match the oracle, and the space-to-depth
    output is the block rearrangement of the plain one (borders left untouched)."""
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    K = 32
    frames = PL.make_frames(B * 7 + H, B, H, W)                              # [B][H][W][4] = B,G,R,A
    planar = np.ascontiguousarray(frames[..., [2, 1, 0]].transpose(0, 3, 1, 2))   # [B][3][H][W] = R,G,B planes
    w = PL.he_normal(RNG, (K, 3, 5, 5))
    b = h(RNG.uniform(-0.2, 0.2, K))
    bn = PL.bn_params(RNG, K, trivial=False)
    x = O.preprocess_frames(frames)
    assert np.array_equal(x, O.convert_normalize(planar.ravel()).reshape(planar.shape))
    want = O.swish(O.batchnorm(O.conv2d(x, w, b, 2, 2), *bn))
    Ho, Wo = want.shape[2], want.shape[3]
    plan = pk.Conv0Plan(c, B, H, W, K, 5, 2, 2, act=pk.ACT_SWISH)
    plan.set_weights(U.dev(w), U.dev(b), bn=[U.dev(q) for q in bn])
    dy = torch.zeros(want.size, dtype=torch.float16, device="cuda")
    plan.forward_bgra(U.dev(frames), dy)
    c.sync()
    got = U.host(dy).reshape(B, Ho, Wo, K).copy()
    assert U.scaled_err(U.nchw(got), want) < 4e-3
    dy.zero_()
    plan.forward_rgb_planar(U.dev(planar), dy)
    c.sync()
    assert np.array_equal(U.host(dy).reshape(B, Ho, Wo, K), got), "planar RGB and BGRA frames give different results"
    if Ho >= 2 and Wo >= 2:
        pk.lib().aig_conv0_plan_set_output_s2d(plan.handle, 1)
        n = pk.lib().aig_s2d_elems(B, Ho, Wo, K)
        ds = torch.full((n,), 0.0, dtype=torch.float16, device="cuda")
        plan.forward_rgb_planar(U.dev(planar), ds)
        c.sync()
        hb, wb = (Ho - 2) // 2 + 2, (Wo - 2) // 2 + 2
        assert np.array_equal(U.host(ds).reshape(B, hb, wb, 4, K), _s2d_host(got))
    plan.close()


RESDOWN = [
    # B, C, H, W, K
    (2, 32, 24, 32, 64),     # N = 128 in one tile, 32-channel sub-positions
    (3, 64, 18, 32, 128),    # N = 256 in one tile
    (2, 128, 9, 16, 256),    # two N tiles, sparse shortcut schedule, odd height
    (5, 32, 72, 128, 64),    # several M tiles per CTA, resident weights
    (1, 256, 10, 12, 256),   # 1024 space-to-depth channels: the patch streams in channel-block groups
    (4, 256, 9, 16, 256),    # the same with odd height and several M tiles
    (230, 128, 9, 16, 256),  # 81 M tiles on 148 SMs: main and shortcut tiles of an M tile go to different CTAs
]


@gpu
@pytest.mark.parametrize("B,C,H,W,K", RESDOWN)
def test_fused_downsampling_pair(env, B, C, H, W, K):
    """Main k4 s2 p1 conv + BatchNorm + Swish and the k2 s2 p0 shortcut of a residual block in one launch
    over the space-to-depth input, against the two oracle convolutions."""
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    x = h(RNG.standard_normal((B, C, H, W)))
    w0 = PL.he_normal(RNG, (K, C, 4, 4))
    b0 = h(RNG.uniform(-0.2, 0.2, K))
    bn = PL.bn_params(RNG, K, trivial=False)
    ws = PL.he_normal(RNG, (K, C, 2, 2))
    bs = h(RNG.uniform(-0.2, 0.2, K))
    want_main = O.activate(O.batchnorm(O.conv2d(x, w0, b0, 2, 1), *bn), 2, 0.01)
    want_short = O.conv2d(x, ws, bs, 2, 0)
    Ho, Wo = want_main.shape[2:]
    assert want_short.shape == want_main.shape
    plan = pk.ResDownPlan(c, B, C, H, W, K, act=pk.ACT_SWISH)
    assert plan.out_dims() == (1, Ho, Wo)
    keep = [U.dev(a) for a in (w0, b0, ws, bs)] + [U.dev(q) for q in bn]
    plan.set_weights(keep[0], keep[1], keep[4:], keep[2], keep[3], eps=1e-6)
    # space-to-depth input made on the device from the channels-last tensor, checked against the numpy layout
    dx = U.dev(U.nhwc(x))
    n_s2d = pk.lib().aig_s2d_elems(B, H, W, C)
    ds = torch.zeros(n_s2d, dtype=torch.float16, device="cuda")
    c.call("aig_nhwc_to_s2d", U.p(dx), U.p(ds), B, H, W, C)
    c.sync()
    assert np.array_equal(U.host(ds).reshape(-1), _s2d_host(U.nhwc(x)).reshape(-1))
    dm = torch.zeros(want_main.size, dtype=torch.float16, device="cuda")
    dsh = torch.zeros(want_main.size, dtype=torch.float16, device="cuda")
    plan.forward(ds, dm, dsh)
    c.sync()
    got_main = U.nchw(U.host(dm).reshape(B, Ho, Wo, K))
    got_short = U.nchw(U.host(dsh).reshape(B, Ho, Wo, K))
    assert U.scaled_err(got_main, want_main) < 6e-3
    assert U.scaled_err(got_short, want_short) < 3e-3
    # round trip of the layout conversion
    back = torch.zeros_like(dx)
    c.call("aig_s2d_to_nhwc", U.p(ds), U.p(back), B, H, W, C)
    c.sync()
    assert torch.equal(back, dx)
    plan.close()


@gpu
def test_conv_output_in_space_to_depth_layout(env):
    """A stride-1 convolution writing straight into the space-to-depth layout gives the same values as
    its channels-last output rearranged."""
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    for (B, C, H, W, K) in [(2, 64, 12, 16, 64), (3, 128, 9, 16, 128)]:
        x = h(RNG.standard_normal((B, C, H, W)))
        w = PL.he_normal(RNG, (K, C, 3, 3))
        b = h(RNG.uniform(-0.2, 0.2, K))
        res = h(RNG.standard_normal((B, K, H, W)))
        plan = pk.ConvPlan(c, B, C, H, W, K, 3, 1, 1, act=pk.ACT_SWISH)
        dw, db, dx, dr = U.dev(w), U.dev(b), U.dev(U.nhwc(x)), U.dev(U.nhwc(res))
        plan.set_weights(dw, db)
        plain = torch.zeros(B * H * W * K, dtype=torch.float16, device="cuda")
        plan.forward(dx, plain, residual=dr)
        c.sync()
        c.check(pk.lib().aig_conv_plan_set_output_s2d(plan.handle, 1))
        blocks = torch.zeros(pk.lib().aig_s2d_elems(B, H, W, K), dtype=torch.float16, device="cuda")
        plan.forward(dx, blocks, residual=dr)
        c.sync()
        want = _s2d_host(U.host(plain).reshape(B, H, W, K))
        assert np.array_equal(U.host(blocks).reshape(-1), want.reshape(-1))
        plan.close()


@gpu
@pytest.mark.parametrize("B,C,H,W,K", [(2, 32, 24, 32, 64), (3, 64, 18, 32, 128), (4, 128, 18, 32, 256), (5, 256, 9, 16, 256), (37, 64, 10, 12, 128),
                                       (800, 64, 8, 8, 128),    # 157 M tiles: the down-sampling launch runs as CTA pairs, the odd tile's partner past the end
                                       (1210, 128, 6, 6, 256)]) # 152 M tiles of a 256-channel 3x3 convolution: CTA pairs on the stride-1 side
def test_padded_position_layout_between_down_sampling_and_conv1(env, B, C, H, W, K):
    """The fused down-sampling launch writes both outputs in the padded position layout (every image with one extra
    zero row and column) and the 3x3 convolution reads its input and its residual from it: the padding positions
    hold zeros, the real positions hold exactly what the channels-last outputs hold, and the convolution's result
    equals the one computed from the channels-last tensors bit for bit."""
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    x = h(RNG.standard_normal((B, C, H, W)))
    w0, b0 = PL.he_normal(RNG, (K, C, 4, 4)), h(RNG.uniform(-0.2, 0.2, K))
    bn = PL.bn_params(RNG, K, trivial=False)
    ws, bs = PL.he_normal(RNG, (K, C, 2, 2)), h(RNG.uniform(-0.2, 0.2, K))
    w1, b1 = PL.he_normal(RNG, (K, K, 3, 3)), h(RNG.uniform(-0.2, 0.2, K))
    bn1 = PL.bn_params(RNG, K, trivial=False)
    down = pk.ResDownPlan(c, B, C, H, W, K, act=pk.ACT_SWISH)
    _, Ho, Wo = down.out_dims()
    keep = [U.dev(a) for a in (w0, b0, ws, bs, w1, b1)] + [U.dev(q) for q in bn] + [U.dev(q) for q in bn1]
    down.set_weights(keep[0], keep[1], keep[6:10], keep[2], keep[3], eps=1e-6)
    conv = pk.ConvPlan(c, B, K, Ho, Wo, K, 3, 1, 1, act=pk.ACT_SWISH)
    conv.set_weights(keep[4], keep[5], bn=keep[10:14])
    ds = torch.zeros(pk.lib().aig_s2d_elems(B, H, W, C), dtype=torch.float16, device="cuda")
    c.call("aig_nhwc_to_s2d", U.p(U.dev(U.nhwc(x))), U.p(ds), B, H, W, C)
    # channels-last link
    n = B * Ho * Wo * K
    m0, s0, y0 = (torch.zeros(n, dtype=torch.float16, device="cuda") for _ in range(3))
    down.forward(ds, m0, s0)
    conv.forward(m0, y0, residual=s0)
    c.sync()
    # padded link (buffers start as garbage: the launch must write every row itself)
    rows = pk.padded_rows(B, Ho, Wo, 1)
    assert rows % 1024 == 0 and rows >= B * (Ho + 1) * (Wo + 1)
    m1 = torch.full((rows * K,), 7.0, dtype=torch.float16, device="cuda")
    s1 = torch.full((rows * K,), -3.0, dtype=torch.float16, device="cuda")
    y1 = torch.zeros(n, dtype=torch.float16, device="cuda")
    down.set_output_padded(True)
    conv.set_input_padded(True)
    down.forward(ds, m1, s1)
    conv.forward(m1, y1, residual=s1)
    c.sync()
    real = B * (Ho + 1) * (Wo + 1)
    for got, want in ((m1, m0), (s1, s0)):
        g = U.host(got).reshape(rows, K)
        # (rows past the last image belong to the allocation only: the consumer's tensor map ends at `real`)
        g = g[:real].reshape(B, Ho + 1, Wo + 1, K)
        assert not g[:, Ho].any() and not g[:, :, Wo].any(), "padding positions must be zeros"
        assert np.array_equal(g[:, :Ho, :Wo], U.host(want).reshape(B, Ho, Wo, K))
    assert np.array_equal(U.host(y1), U.host(y0)), "conv1 over the padded layout differs from the channels-last result"
    # and against the oracle
    main = O.activate(O.batchnorm(O.conv2d(x, w0, b0, 2, 1), *bn), 2, 0.01)
    short = O.conv2d(x, ws, bs, 2, 0)
    want = O.activate(O.add(O.batchnorm(O.conv2d(main, w1, b1, 1, 1), *bn1), short), 2, 0.01)
    assert U.scaled_err(U.nchw(U.host(y1).reshape(B, Ho, Wo, K)), want) < 8e-3
    # switching back restores the channels-last link
    down.set_output_padded(False)
    conv.set_input_padded(False)
    y2 = torch.zeros(n, dtype=torch.float16, device="cuda")
    down.forward(ds, m0, s0)
    conv.forward(m0, y2, residual=s0)
    c.sync()
    assert torch.equal(y2, y0)
    down.close()
    conv.close()


@gpu
def test_fused_downsampling_refuses_unsupported_channel_counts(env):
    """Channel counts the space-to-depth GEMM cannot tile are refused with a clear status (callers then
    use the two separate convolutions)."""
    U = env
    pk = U.pkg()
    with pytest.raises(pk.AigError, match="in_c"):
        pk.ResDownPlan(U.ctx(), 1, 24, 10, 12, 64)
    with pytest.raises(pk.AigError, match="out_c"):
        pk.ResDownPlan(U.ctx(), 1, 32, 10, 12, 48)
