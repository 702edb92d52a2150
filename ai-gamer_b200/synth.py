"""Seeded synthetic parameters and inputs for the benchmark configurations, and checkpoint writers
in the reference's byte layout.  Pure numpy; used by the benchmark, the tests and the oracle
compositions alike so that every side sees the same bytes.  No dataset or checkpoint is involved:
frames, embeddings and weights are drawn from ``numpy.random.default_rng(seed)`` with the stated
distributions."""
import math

import numpy as np

F16 = np.float16


# ----------------------------------------------------------------------------- parameter factories
def he_normal(rng, shape):
    fan_in = int(np.prod(shape[1:]))
    return (rng.standard_normal(shape) * math.sqrt(2.0 / fan_in)).astype(F16)


def xavier_uniform(rng, shape, fan_in, fan_out):
    a = math.sqrt(6.0 / (fan_in + fan_out))
    return rng.uniform(-a, a, shape).astype(F16)


def bn_params(rng, c, trivial=True):
    """(gamma, beta, running_mean, running_var); trivial = gamma 1, beta 0, mean 0, var 1."""
    if trivial:
        return (np.ones(c, np.float32), np.zeros(c, np.float32), np.zeros(c, np.float32), np.ones(c, np.float32))
    return (
        rng.uniform(0.5, 1.5, c).astype(np.float32),
        rng.uniform(-0.5, 0.5, c).astype(np.float32),
        rng.uniform(-0.3, 0.3, c).astype(np.float32),
        rng.uniform(0.5, 2.0, c).astype(np.float32),
    )


def bias_params(rng, c, trivial=True):
    return np.zeros(c, F16) if trivial else rng.uniform(-0.2, 0.2, c).astype(F16)


def make_resconv_params(rng, in_c, out_c, trivial=True):
    """ResConvLayer.cpp:13-21: main k4 s2 p1 -> BN -> act -> k3 s1 p1 -> BN; shortcut k2 s2 p0."""
    return dict(
        c0w=he_normal(rng, (out_c, in_c, 4, 4)), c0b=bias_params(rng, out_c, trivial), bn0=bn_params(rng, out_c, trivial),
        c1w=he_normal(rng, (out_c, out_c, 3, 3)), c1b=bias_params(rng, out_c, trivial), bn1=bn_params(rng, out_c, trivial),
        sw=he_normal(rng, (out_c, in_c, 2, 2)), sb=bias_params(rng, out_c, trivial),
    )


def make_cnn_params(seed=0, widths=(32, 64, 128, 256, 256), n_out=18, k0=5, trivial=True):
    """2-D encoder: Conv 3->w0 k5 s2 p2 + BN + act, ResConv blocks, spatial attention (1x1 conv ->
    sigmoid mask), global average pool, FC -> n_out."""
    rng = np.random.default_rng(seed)
    p = dict(widths=tuple(widths), n_out=n_out, k0=k0)
    p["c0w"] = he_normal(rng, (widths[0], 3, k0, k0))
    p["c0b"] = bias_params(rng, widths[0], trivial)
    p["bn0"] = bn_params(rng, widths[0], trivial)
    p["res"] = [make_resconv_params(rng, widths[i], widths[i + 1], trivial) for i in range(len(widths) - 1)]
    p["sa_w"] = he_normal(rng, (1, widths[-1]))[0]
    p["sa_b"] = 0.0 if trivial else 0.1
    p["fcW"] = he_normal(rng, (n_out, widths[-1])).T.copy()  # stored [in][out] like FCLayer
    p["fcb"] = bias_params(rng, n_out, trivial)
    return p


def _bn_bytes(bn):
    """BatchNorm.cpp:90-117: scale, bias, runningMean, runningVar, savedMean, savedInvVar."""
    g, b, m, v = bn
    z = np.zeros_like(g)
    return b"".join(np.ascontiguousarray(a, np.float32).tobytes() for a in (g, b, m, v, z, z))


def serialize_cnn_checkpoint(p, width, height):
    """Checkpoint bytes in the reference's layout (NN.cpp:113-128 order: int32 w, int32 h, then each
    layer's SaveParameters payload in construction order)."""
    out = [np.array([width, height], np.int32).tobytes()]
    out += [p["c0w"].tobytes(), p["c0b"].tobytes(), _bn_bytes(p["bn0"])]
    for blk in p["res"]:  # ResConvLayer.cpp:55-66: Conv0, BN0, Conv1, BN1, shortcut
        out += [blk["c0w"].tobytes(), blk["c0b"].tobytes(), _bn_bytes(blk["bn0"]), blk["c1w"].tobytes(),
                blk["c1b"].tobytes(), _bn_bytes(blk["bn1"]), blk["sw"].tobytes(), blk["sb"].tobytes()]
    out += [np.ascontiguousarray(p["sa_w"], F16).tobytes(), np.array([p["sa_b"]], np.float32).tobytes()]
    out += [np.ascontiguousarray(p["fcW"], F16).tobytes(), np.ascontiguousarray(p["fcb"], F16).tobytes()]
    return b"".join(out)


def make_frames(seed, batch, height=144, width=256):
    rng = np.random.default_rng(seed + 1000003)
    return rng.integers(0, 256, (batch, height, width, 4), dtype=np.uint8)


def make_fc_ln_params(seed=0, in_c=1024, out_c=1024):
    rng = np.random.default_rng(seed)
    W = (rng.standard_normal((in_c, out_c)) / math.sqrt(in_c)).astype(F16)
    return dict(W=W, b=np.zeros(out_c, F16), gamma=np.ones(out_c, np.float32), beta=np.zeros(out_c, np.float32))


def make_conv3d_params(seed=0, widths=(3, 32, 64, 128), n_out=18, trivial=True):
    rng = np.random.default_rng(seed)
    p = dict(widths=tuple(widths), n_out=n_out, layers=[])
    for i in range(len(widths) - 1):
        p["layers"].append(
            dict(w=he_normal(rng, (widths[i + 1], widths[i], 3, 3, 3)), b=bias_params(rng, widths[i + 1], trivial),
                 bn=bn_params(rng, widths[i + 1], trivial))
        )
    feat = widths[-1] * 4
    p["fcW"] = he_normal(rng, (n_out, feat)).T.copy()
    p["fcb"] = bias_params(rng, n_out, trivial)
    return p


def make_clips(seed, batch, depth=8, height=144, width=256):
    rng = np.random.default_rng(seed + 2000003)
    return rng.random((batch, 3, depth, height, width), dtype=np.float32).astype(F16)


def make_lstm_blob(rng, in_c, hid, layers, double_bias=True, forget_bias=1.0):
    """Blob layout defined in aig_oracle.cpp (orc_lstm): per layer W(i,f,g,o) then R(i,f,g,o);
    then per layer bW(i,f,g,o) [and bR(i,f,g,o)].  Forget-gate bias on the input-bias vector."""
    parts = []
    for l in range(layers):
        inl = in_c if l == 0 else hid
        parts.append(xavier_uniform(rng, (4 * hid * inl,), inl, hid))
        parts.append(xavier_uniform(rng, (4 * hid * hid,), hid, hid))
    for l in range(layers):
        bW = np.zeros(4 * hid, F16)
        bW[hid:2 * hid] = forget_bias
        parts.append(bW)
        if double_bias:
            parts.append(np.zeros(4 * hid, F16))
    return np.concatenate(parts)


def make_seq_params(seed=0, d=512, hid=512, layers=2, heads=8, n_out=18):
    rng = np.random.default_rng(seed)
    p = dict(d=d, hid=hid, layers=layers, heads=heads, n_out=n_out)
    p["lstm"] = make_lstm_blob(rng, d, hid, layers)
    for name in ("wq", "wk", "wv", "wo"):
        p[name] = xavier_uniform(rng, (hid, hid), hid, hid)
    p["ln_g"] = np.ones(hid, np.float32)
    p["ln_b"] = np.zeros(hid, np.float32)
    p["fcW"] = xavier_uniform(rng, (hid, n_out), hid, n_out)
    p["fcb"] = np.zeros(n_out, F16)
    return p


def serialize_seq_params(p):
    """Sequence-head blob in layer order: LSTM blob (LSTMLayer.cpp:139-146), MHA wq,wk,wv,wo
    (MHALayer.cpp:191-210), LayerNorm gamma,beta (LayerNorm.cpp:50-61), FC W,b (FCLayer.cpp:70-81)."""
    parts = [np.ascontiguousarray(p["lstm"], F16).tobytes()]
    parts += [np.ascontiguousarray(p[k], F16).tobytes() for k in ("wq", "wk", "wv", "wo")]
    parts += [np.ascontiguousarray(p["ln_g"], np.float32).tobytes(), np.ascontiguousarray(p["ln_b"], np.float32).tobytes()]
    parts += [np.ascontiguousarray(p["fcW"], F16).tobytes(), np.ascontiguousarray(p["fcb"], F16).tobytes()]
    return b"".join(parts)


def make_agent_params(seed=0, widths=(32, 64, 128, 256, 256), d=512, layers=2, heads=8, n_out=18):
    """Streaming agent = frame encoder + bridge FC (features -> d) + sequence head."""
    rng = np.random.default_rng(seed + 17)
    cnn = make_cnn_params(seed, widths=widths, n_out=n_out)
    seq = make_seq_params(seed + 1, d=d, hid=d, layers=layers, heads=heads, n_out=n_out)
    bw = xavier_uniform(rng, (widths[-1], d), widths[-1], d)
    bb = np.zeros(d, F16)
    return dict(cnn=cnn, seq=seq, bw=bw, bb=bb)


def serialize_agent_params(p, width, height):
    return b"".join([serialize_cnn_checkpoint(p["cnn"], width, height), p["bw"].tobytes(), p["bb"].tobytes(),
                     serialize_seq_params(p["seq"])])


def make_refnn_params(seed, width, height):
    """Parameters of the network the reference itself builds (NN.cpp:33-61) for a width x height input."""
    rng = np.random.default_rng(seed)
    p = dict(width=width, height=height)
    p["c0w"] = he_normal(rng, (32, 3, 2, 2))
    p["c0b"] = bias_params(rng, 32, False)
    p["bn0"] = bn_params(rng, 32, False)
    p["res"] = [make_resconv_params(rng, a, b, False) for a, b in ((32, 64), (64, 128), (128, 256))]
    h, w = height // 2, width // 2
    for _ in range(3):
        h, w = (h + 2 - 4) // 2 + 1, (w + 2 - 4) // 2 + 1
    p["fc"] = []
    dims = [256 * h * w, 1024, 512, 256]
    for i in range(3):
        W = (rng.standard_normal((dims[i], dims[i + 1])) * math.sqrt(2.0 / dims[i])).astype(F16)
        p["fc"].append(dict(W=W, b=bias_params(rng, dims[i + 1], False), bn=bn_params(rng, dims[i + 1], False)))
    p["outW"] = (rng.standard_normal((256, 16)) * math.sqrt(2.0 / 256)).astype(F16)
    p["outb"] = bias_params(rng, 16, False)
    return p


def serialize_refnn_checkpoint(p):
    """The reference's checkpoint file (NN.cpp:113-128): int32 w, h, then each layer's payload."""
    out = [np.array([p["width"], p["height"]], np.int32).tobytes(), p["c0w"].tobytes(), p["c0b"].tobytes(), _bn_bytes(p["bn0"])]
    for blk in p["res"]:
        out += [blk["c0w"].tobytes(), blk["c0b"].tobytes(), _bn_bytes(blk["bn0"]), blk["c1w"].tobytes(), blk["c1b"].tobytes(),
                _bn_bytes(blk["bn1"]), blk["sw"].tobytes(), blk["sb"].tobytes()]
    for L in p["fc"]:
        out += [L["W"].tobytes(), L["b"].tobytes(), _bn_bytes(L["bn"])]
    out += [p["outW"].tobytes(), p["outb"].tobytes()]
    return b"".join(out)


def make_embeddings(seed, T, B, d):
    rng = np.random.default_rng(seed + 3000003)
    return rng.standard_normal((T, B, d)).astype(F16)


def serialize_conv3d_params(p):
    """Clip-encoder blob: per layer the ConvLayer3D payload (w, b; ConvLayer3D.cpp:128-139) and the
    BatchNorm payload, then the FC head (W [in][out], b)."""
    out = []
    for L in p["layers"]:
        out += [L["w"].tobytes(), L["b"].tobytes(), _bn_bytes(L["bn"])]
    out += [np.ascontiguousarray(p["fcW"], F16).tobytes(), np.ascontiguousarray(p["fcb"], F16).tobytes()]
    return b"".join(out)
