"""The CPU oracle checked (a) against closed-form / known-answer values for the operators whose
reference arithmetic is fully specified and (b) against PyTorch's CPU fp32/fp64 operators for the
ones the reference delegates to cuDNN/cuBLAS (convolution conventions, BatchNorm, GEMM orientation,
LSTM gate order, attention).  No GPU needed."""
import math
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle as O
from oracle import pipelines as PL

RNG = np.random.default_rng(7)


def h(a):
    return np.asarray(a, np.float32).astype(np.float16)


def close16(a, b, ulps=2.0, atol=1e-4):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    tol = atol + ulps * np.abs(b) * 2.0 ** -10
    bad = np.abs(a - b) > tol
    assert not bad.any(), f"{bad.sum()} mismatches, max abs {np.abs(a - b).max()}"


def test_bgra_planar_known_answer():
    src = np.arange(4 * 6, dtype=np.uint8)
    dst = O.bgra_to_planar(src, 6)
    assert dst[:6].tolist() == [2, 6, 10, 14, 18, 22]  # R
    assert dst[6:12].tolist() == [1, 5, 9, 13, 17, 21]  # G
    assert dst[12:].tolist() == [0, 4, 8, 12, 16, 20]  # B


def test_convert_normalize_all_256_codes():
    u = np.arange(256, dtype=np.uint8)
    got = O.convert_normalize(u)
    want = (u.astype(np.float32) / np.float32(255.0)).astype(np.float16)
    assert got.view(np.uint16).tolist() == want.view(np.uint16).tolist()
    assert got[0] == 0 and got[255] == 1
    # and back: trunc(h*255)
    back = O.unconvert_unnormalize(got)
    assert np.all(np.abs(back.astype(int) - u.astype(int)) <= 1)
    assert back[255] == 255 and back[0] == 0


def test_activations_formulas():
    x = h(np.linspace(-9, 9, 4001))
    xf = x.astype(np.float32)
    sw = O.swish(x)
    close16(sw, xf / (1 + np.exp(-xf.astype(np.float64))), ulps=1.01)
    lr = O.leaky_relu(x, 1.0 / 128)
    assert np.array_equal(lr[xf >= 0], x[xf >= 0])
    assert np.array_equal(lr[xf < 0], (xf[xf < 0] * np.float32(1 / 128)).astype(np.float16))
    # slope is rounded to fp16 first (CudaStuff.cu:403 passes float into a __half parameter)
    lr2 = O.leaky_relu(x, 0.01)
    s16 = np.float32(np.float16(0.01))
    assert np.array_equal(lr2[xf < 0], (xf[xf < 0] * s16).astype(np.float16))
    re = O.relu(h([-1, 0, 2, np.nan]))
    assert re.tolist() == [0, 0, 2, 0]
    sg = O.sigmoid_head(h(np.tile(np.linspace(-4, 4, 16), 3)), 16, 14)
    ref = np.tile(np.linspace(-4, 4, 16), 3).astype(np.float16).astype(np.float64)
    want = 1 / (1 + np.exp(-ref))
    idx = np.arange(48) % 16
    close16(sg[idx < 14], want[idx < 14], ulps=1.01)
    assert np.array_equal(sg[idx >= 14], h(ref)[idx >= 14])  # axes pass through unchanged
    th = O.tanh_tail(h(ref), 16, 14)
    close16(th[idx >= 14], np.tanh(ref[idx >= 14]), ulps=1.01)
    assert np.array_equal(th[idx < 14], h(ref)[idx < 14])


@pytest.mark.parametrize("k,s,p,H,W", [(2, 2, 0, 8, 10), (4, 2, 1, 9, 12), (3, 1, 1, 7, 5), (5, 2, 2, 11, 14)])
def test_conv2d_vs_torch(k, s, p, H, W):
    B, C, K = 2, 5, 7
    x = h(RNG.standard_normal((B, C, H, W)))
    w = h(RNG.standard_normal((K, C, k, k)) * 0.2)
    b = h(RNG.standard_normal(K))
    got = O.conv2d(x, w, b, s, p)
    t = F.conv2d(torch.tensor(x.astype(np.float64)), torch.tensor(w.astype(np.float64)), None, s, p)
    want = t.numpy().astype(np.float16).astype(np.float32) + b.astype(np.float32)[None, :, None, None]
    assert got.shape == t.shape
    close16(got, want.astype(np.float16), ulps=1.01)


def test_conv3d_vs_torch():
    B, C, K, D, H, W = 2, 3, 4, 5, 8, 10
    x = h(RNG.random((B, C, D, H, W)))
    w = h(RNG.standard_normal((K, C, 3, 3, 3)) * 0.2)
    b = h(RNG.standard_normal(K) * 0.1)
    got = O.conv3d(x, w, b, 1, 2, 1, 1)
    t = F.conv3d(torch.tensor(x.astype(np.float64)), torch.tensor(w.astype(np.float64)), None, (1, 2, 2), (1, 1, 1))
    want = t.numpy().astype(np.float16).astype(np.float32) + b.astype(np.float32)[None, :, None, None, None]
    assert got.shape == t.shape == (B, K, 5, 4, 5)
    close16(got, want.astype(np.float16), ulps=1.01)


def test_batchnorm_both_modes_vs_torch():
    B, C, H, W = 3, 6, 4, 5
    x = h(RNG.standard_normal((B, C, H, W)))
    g, be, mu, var = PL.bn_params(RNG, C, trivial=False)
    got = O.batchnorm(x, g, be, mu, var, 1e-6)
    want = F.batch_norm(torch.tensor(x.astype(np.float64)), torch.tensor(mu.astype(np.float64)),
                        torch.tensor(var.astype(np.float64)), torch.tensor(g.astype(np.float64)),
                        torch.tensor(be.astype(np.float64)), False, 0.0, 1e-6).numpy()
    close16(got, want, ulps=1.01)
    # per-activation: one parameter per (c,h,w)
    g2, be2, mu2, var2 = PL.bn_params(RNG, C * H * W, trivial=False)
    got2 = O.batchnorm(x, g2, be2, mu2, var2, 1e-6, per_activation=True)
    xf = x.astype(np.float64).reshape(B, -1)
    want2 = (g2 * (xf - mu2) / np.sqrt(var2 + 1e-6) + be2).reshape(x.shape)
    close16(got2, want2, ulps=1.01)


def test_fc_orientation_and_two_roundings():
    B, I, Oo = 5, 24, 9
    x = h(RNG.standard_normal((B, I)))
    W = h(RNG.standard_normal((I, Oo)) * 0.3)
    b = h(RNG.standard_normal(Oo))
    got = O.fc(x, W, b)
    t = (x.astype(np.float64) @ W.astype(np.float64)).astype(np.float16)
    want = (t.astype(np.float32) + b.astype(np.float32)).astype(np.float16)
    assert np.array_equal(got, want)


def test_fc_backward_orientation():
    """FCLayer.cpp:54-59: grad_w = x^T . g in the weights' [in][out] layout, grad_x = g . W^T, grad_b = column sums."""
    B, I, Oo = 7, 24, 9
    x = h(RNG.standard_normal((B, I)))
    g = h(RNG.standard_normal((B, Oo)) * 0.1)
    W = h(RNG.standard_normal((I, Oo)) * 0.3)
    gw, gb, gx = O.fc_backward(x, g, W)
    x64, g64, W64 = x.astype(np.float64), g.astype(np.float64), W.astype(np.float64)
    assert np.array_equal(gw, (x64.T @ g64).astype(np.float16))
    assert np.array_equal(gx, (g64 @ W64.T).astype(np.float16))
    s = np.zeros(Oo, np.float32)
    for b in range(B):
        s = s + g[b].astype(np.float32)
    assert np.array_equal(gb, s.astype(np.float16))


def test_layernorm_ref_axis_and_rows():
    N, C, HW = 4, 6, 10
    x = h(RNG.standard_normal((N, C, HW)) * 2 + 0.5)
    g = RNG.uniform(0.5, 1.5, C).astype(np.float32)
    b = RNG.uniform(-1, 1, C).astype(np.float32)
    y, mean, var = O.layernorm_ref(x, g, b, N, C, HW, 1e-7)
    xf = x.astype(np.float64)
    mu = xf.transpose(1, 0, 2).reshape(C, -1).mean(1)
    v = xf.transpose(1, 0, 2).reshape(C, -1).var(1)
    np.testing.assert_allclose(mean, mu, rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(var, v, rtol=1e-6)
    want = (xf - mu[None, :, None]) / np.sqrt(v[None, :, None] + 1e-7) * g[None, :, None] + b[None, :, None]
    close16(y, want, ulps=1.5)
    rows = h(RNG.standard_normal((7, 32)))
    g2 = RNG.uniform(0.5, 1.5, 32).astype(np.float32)
    b2 = RNG.uniform(-1, 1, 32).astype(np.float32)
    y2 = O.layernorm_rows(rows, g2, b2, 1e-5)
    want2 = F.layer_norm(torch.tensor(rows.astype(np.float64)), (32,), torch.tensor(g2.astype(np.float64)),
                         torch.tensor(b2.astype(np.float64)), 1e-5).numpy()
    close16(y2, want2, ulps=1.01)


def test_spatial_attention_ref_structure():
    B, inC, attC, H, W, G = 2, 8, 4, 4, 8, 64
    P = B * H * W
    x = h(RNG.standard_normal(P * inC) * 0.5)
    kW = h(RNG.standard_normal(attC * inC) * 0.3)
    qW = h(RNG.standard_normal(attC * inC) * 0.3)
    vW = h(RNG.standard_normal(attC * inC) * 0.3)
    r = O.spatial_attention_ref(x, kW, qW, vW, B, inC, attC, H, W, G)
    X = x.reshape(P, inC)
    # sequential fp16 fma chain, one position checked in numpy
    acc = np.float16(0)
    for c in range(inC):
        acc = np.float16(np.float64(X[3, c]) * np.float64(kW[1 * inC + c]) + np.float64(acc))
    assert r["keyMap"][3, 1] == acc
    # softmax: max per 32-position warp, sum per G-position block
    s = (r["queryMap"].astype(np.float32) * r["keyMap"].astype(np.float32)).sum(1) * np.float32(1 / math.sqrt(inC))
    e = np.concatenate([np.exp(s[i:i + 32] - s[i:i + 32].max()) for i in range(0, P, 32)])
    a = e / e.reshape(-1, G).sum(1).repeat(G)
    close16(r["scores"], a, ulps=2)
    wv = (r["scores"].astype(np.float32)[:, None] * r["valueMap"].astype(np.float32)).astype(np.float16)
    out = (X[:, np.arange(attC) % inC].astype(np.float32) + wv.astype(np.float32)).astype(np.float16)
    assert np.array_equal(r["out"], out)


def test_lstm_vs_torch_gate_order_and_state_carry():
    T, B, I, Hd, L = 6, 3, 8, 8, 2
    rng = np.random.default_rng(11)
    blob = PL.make_lstm_blob(rng, I, Hd, L, True, 1.0)
    # give the recurrent biases something non-zero too
    blob[-4 * Hd:] = h(rng.uniform(-0.2, 0.2, 4 * Hd))
    x = h(rng.standard_normal((T, B, I)))
    y = O.lstm(x, blob, Hd, L, clip=0.0)
    lstm = torch.nn.LSTM(I, Hd, L).double()
    off = 0
    with torch.no_grad():
        for l in range(L):
            inl = I if l == 0 else Hd
            getattr(lstm, f"weight_ih_l{l}").copy_(torch.tensor(blob[off:off + 4 * Hd * inl].astype(np.float64)).view(4 * Hd, inl))
            off += 4 * Hd * inl
            getattr(lstm, f"weight_hh_l{l}").copy_(torch.tensor(blob[off:off + 4 * Hd * Hd].astype(np.float64)).view(4 * Hd, Hd))
            off += 4 * Hd * Hd
        for l in range(L):
            getattr(lstm, f"bias_ih_l{l}").copy_(torch.tensor(blob[off:off + 4 * Hd].astype(np.float64)))
            off += 4 * Hd
            getattr(lstm, f"bias_hh_l{l}").copy_(torch.tensor(blob[off:off + 4 * Hd].astype(np.float64)))
            off += 4 * Hd
        want, _ = lstm(torch.tensor(x.astype(np.float64)))
    assert off == blob.size
    np.testing.assert_allclose(y.astype(np.float64), want.numpy(), atol=4e-3)
    # carried state: two halves with state == one pass
    hs = np.zeros((L, B, Hd), np.float16)
    cs = np.zeros((L, B, Hd), np.float16)
    y1 = O.lstm(x[:3], blob, Hd, L, 0.0, True, hs, cs, True)
    y2 = O.lstm(x[3:], blob, Hd, L, 0.0, True, hs, cs, True)
    assert np.array_equal(np.concatenate([y1, y2]), y)
    # clip: large inputs saturate the cell at +-clip
    big = h(np.full((40, 1, I), 8.0))
    blob2 = blob.copy()
    yc = O.lstm(big, blob2, Hd, L, clip=5.0)
    assert np.isfinite(yc.astype(np.float32)).all() and np.abs(yc.astype(np.float32)).max() <= 1.0


def test_mha_vs_torch_sdpa_and_rope_window():
    B, T, E, Hh = 2, 9, 16, 2
    rng = np.random.default_rng(5)
    x = h(rng.standard_normal((B, T, E)))
    ws = [h(rng.standard_normal((E, E)) * 0.25) for _ in range(4)]
    y = O.mha(x, *ws, Hh)
    xd = torch.tensor(x.astype(np.float64))
    q, k, v = [(xd @ torch.tensor(w.astype(np.float64))).to(torch.float16).double() for w in ws[:3]]
    sp = lambda t: t.view(B, T, Hh, E // Hh).transpose(1, 2)
    ctx = F.scaled_dot_product_attention(sp(q), sp(k), sp(v), is_causal=True).transpose(1, 2).reshape(B, T, E)
    want = ctx.to(torch.float16).double() @ torch.tensor(ws[3].astype(np.float64))
    close16(y, want.numpy(), ulps=2, atol=2e-3)
    # window >= T is the same as unbounded; position offset with RoPE only matters relatively
    assert np.array_equal(O.mha(x, *ws, Hh, 0.0, 0, T), y)
    y_r0 = O.mha(x, *ws, Hh, 10000.0, 0, 0)
    y_r7 = O.mha(x, *ws, Hh, 10000.0, 7, 0)
    assert not np.array_equal(y_r0, y)
    np.testing.assert_allclose(y_r0.astype(np.float32), y_r7.astype(np.float32), atol=2e-2)
    # sliding window 4: last step only sees steps T-4..T-1 -> equals a fresh 4-step run's last step with pos0
    y_w = O.mha(x, *ws, Hh, 10000.0, 0, 4)
    y_tail = O.mha(x[:, T - 4:], *ws, Hh, 10000.0, T - 4, 0)
    assert np.array_equal(y_w[:, -1], y_tail[:, -1])


def test_actions_thresholds():
    p = np.zeros((2, 16), np.float32)
    p[0, :14] = [0.5, 0.50001, 0.49, 1, 0, .7, .2, .9, .1, .6, .4, .51, .5, .8]
    p[0, 14:] = [0.999, -0.999]
    p[1, 14:] = [0.0039, -0.0040]
    a = O.actions(p)
    assert a[0, :14].tolist() == [0, 1, 0, 1, 0, 1, 0, 1, 0, 1, 0, 1, 0, 1]
    assert a[0, 14:].tolist() == [255, -255]
    assert a[1, 14:].tolist() == [0, -1]


def test_cnn_pipeline_small_runs_and_is_deterministic():
    p = PL.make_cnn_params(3, widths=(8, 16, 16), n_out=18, trivial=False)
    fr = PL.make_frames(3, 2, 16, 32)
    f1, l1, o1 = PL.cnn_forward(p, fr)
    f2, l2, o2 = PL.cnn_forward(p, fr)
    assert f1.shape == (2, 16) and o1.shape == (2, 18)
    assert np.array_equal(o1, o2) and np.isfinite(o1.astype(np.float32)).all()
    assert (o1[:, :16] >= 0).all() and (o1[:, :16] <= 1).all() and (np.abs(o1[:, 16:].astype(np.float32)) <= 1).all()


# ----------------------------------------------------------------------------- pinned to the reference
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernels.npz")


def _ulp_diff(a_u16, b_u16):
    """fp16 distance in units of the last place (sign-magnitude bit patterns mapped to a monotone integer line)."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a_u16) - key(b_u16))


def test_oracle_matches_outputs_of_the_reference_kernels():
    """tests/golden/reference_kernels.npz holds outputs of the reference's own CUDA kernels (CudaStuff.cu,
    run on a B200 by tests/golden/make_reference_golden.py).  Byte work and the projections must be
    bit-exact; results that pass through expf / rsqrtf may differ in the last fp16 place."""
    g = np.load(GOLDEN)
    n = g["pre_planar"].size // 3
    planar = O.bgra_to_planar(g["pre_bgra"], n)
    assert np.array_equal(planar, g["pre_planar"])                                   # CudaStuff.cu:63-74
    assert np.array_equal(O.convert_normalize(planar).view(np.uint16), g["pre_half"])  # CudaStuff.cu:150-153, all 256 byte values
    x = g["act_x"].view(np.float16)
    assert np.array_equal(O.leaky_relu(x, 0.01).view(np.uint16), g["act_leaky"])     # CudaStuff.cu:400-405
    for name, got in (("act_swish", O.swish(x)), ("act_sigmoid", O.sigmoid_head(x, 16, 14))):
        d = _ulp_diff(got.view(np.uint16), g[name])
        assert d.max() <= 1 and (d == 0).mean() > 0.995, name
    B, inC, attC, H, W = (int(v) for v in g["sa_dims"])
    sa = O.spatial_attention_ref(g["sa_x"].view(np.float16), g["sa_wk"].view(np.float16), g["sa_wq"].view(np.float16),
                                 g["sa_wv"].view(np.float16), B, inC, attC, H, W, 64)
    for key, name in (("keyMap", "sa_key"), ("queryMap", "sa_query"), ("valueMap", "sa_value")):
        assert np.array_equal(sa[key].reshape(-1).view(np.uint16), g[name]), name      # CudaStuff.cu:673-700
    for key, name in (("scores", "sa_scores"), ("out", "sa_out")):
        d = _ulp_diff(sa[key].reshape(-1).view(np.uint16), g[name])
        assert d.max() <= 1 and (d == 0).mean() > 0.97, name
    N, C, HW = (int(v) for v in g["ln_dims"])
    y, mean, var = O.layernorm_ref(g["ln_x"].view(np.float16), g["ln_gamma"], g["ln_beta"], N, C, HW, 1e-7)
    np.testing.assert_allclose(mean, g["ln_mean"], rtol=2e-5, atol=2e-6)               # CudaStuff.cu:457-515
    np.testing.assert_allclose(var, g["ln_var"], rtol=2e-5, atol=1e-7)
    d = _ulp_diff(y.reshape(-1).view(np.uint16), g["ln_y"].reshape(-1))
    big = np.abs(y.reshape(-1).astype(np.float32)) > 2e-3
    assert d[big].max() <= 2 and (d == 0).mean() > 0.97


def test_resize_box_definition(oracle):
    """The oracle's box-filter resize (ConvScale.cpp:41-52 with a fixed summation order) against a direct numpy
    restatement: fp32 fused multiply-adds in (channel, row, column) order are reproduced here with float64 products
    of fp16-exact operands, which are exact, so every partial sum can be rounded to fp32 explicitly."""
    O = oracle
    rng = np.random.default_rng(4)
    for (N, C, H, W, k, cross) in ((2, 3, 9, 14, 2, False), (1, 3, 10, 11, 3, True), (1, 3, 8, 8, 4, False)):
        src = rng.integers(0, 256, (N, C, H, W), dtype=np.uint8)
        o8, oh = O.resize_box(src, k, cross_channel=cross)
        wk = np.float64(np.float16(np.float32(1.0) / np.float32(k * k)))
        xn = O.convert_normalize(src).astype(np.float64)
        want = np.zeros((N, C, H // k, W // k), np.float16)
        for n in range(N):
            for c in range(C):
                for oy in range(H // k):
                    for ox in range(W // k):
                        acc = np.float32(0.0)
                        for ci in (range(C) if cross else [c]):
                            for dy in range(k):
                                for dx in range(k):
                                    acc = np.float32(np.float64(acc) + xn[n, ci, oy * k + dy, ox * k + dx] * wk)   # one rounding = fmaf
                        want[n, c, oy, ox] = np.float16(acc)
        assert np.array_equal(oh.view(np.uint16), want.view(np.uint16))
        assert np.array_equal(o8, (want.astype(np.float32) * np.float32(255.0)).astype(np.uint8))
        # BGRA source = the same planes read from interleaved pixels
        bgra = np.zeros((N, H, W, 4), np.uint8)
        bgra[..., 2], bgra[..., 1], bgra[..., 0], bgra[..., 3] = src[:, 0], src[:, 1], src[:, 2], 255
        o8b, ohb = O.resize_box(bgra, k, cross_channel=cross, bgra=True)
        assert np.array_equal(o8b, o8) and np.array_equal(ohb.view(np.uint16), oh.view(np.uint16))
