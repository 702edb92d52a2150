"""ctypes/numpy front end of the CPU oracle (oracle/aig_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of bench.py, as the checker and the timed CPU baseline.
The product (the CUDA library and its host classes) never imports it.

fp16 tensors are numpy ``float16`` arrays; all arrays are C-contiguous.  Each wrapper names the
reference operator it restates (paths relative to the reference's ``AI gamer/`` directory).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_c_size_t = ctypes.c_size_t
_vp = ctypes.c_void_p


def lib_path():
    return os.path.join(_HERE, "libaig_oracle.so")


def build(force=False):
    """Compile the oracle with the committed Makefile (g++ only, no CUDA)."""
    if force or not os.path.exists(lib_path()) or os.path.getmtime(lib_path()) < os.path.getmtime(
        os.path.join(_HERE, "aig_oracle.cpp")
    ):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libaig_oracle.so"], stdout=subprocess.DEVNULL)
    return lib_path()


def lib():
    global _LIB
    if _LIB is None:
        if not os.path.exists(lib_path()):
            build()
        _LIB = ctypes.CDLL(lib_path())
    return _LIB


def set_threads(n):
    """Threads used by the oracle's OpenMP loops; returns the previous maximum."""
    return lib().orc_set_threads(int(n))


def _p(a):
    return None if a is None else a.ctypes.data_as(_vp)


def _h(a):
    a = np.ascontiguousarray(a, dtype=np.float16)
    return a


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ------------------------------------------------------------------ preprocessing
def bgra_to_planar(src, n):
    """CudaStuff.cu:63-74."""
    src = np.ascontiguousarray(src, dtype=np.uint8)
    dst = np.empty(3 * n, np.uint8)
    lib().orc_bgra_to_planar(_p(src), _p(dst), _c_int(n))
    return dst


def convert_normalize(u8):
    """CudaStuff.cu:150-153."""
    u8 = np.ascontiguousarray(u8, dtype=np.uint8)
    out = np.empty(u8.shape, np.float16)
    lib().orc_convert_normalize(_p(out), _p(u8), _c_size_t(u8.size))
    return out


def unconvert_unnormalize(hf):
    """CudaStuff.cu:158-161."""
    hf = _h(hf)
    out = np.empty(hf.shape, np.uint8)
    lib().orc_unconvert_unnormalize(_p(out), _p(hf), _c_size_t(hf.size))
    return out


def resize_box(src, k, cross_channel=False, bgra=False):
    """ConvScale.cpp:41-52 with the fixed summation order.  src: planar uint8 [N][C][H][W], or BGRA [N][H][W][4];
    returns (uint8, float16) planar [N][C][H//k][W//k]."""
    src = np.ascontiguousarray(src, dtype=np.uint8)
    if bgra:
        N, H, W, _ = src.shape
        C = 3
    else:
        N, C, H, W = src.shape
    o8 = np.empty((N, C, H // k, W // k), np.uint8)
    oh = np.empty((N, C, H // k, W // k), np.float16)
    lib().orc_resize_box(_p(src), _p(o8), _p(oh), *map(_c_int, (N, C, H, W, k, 1 if cross_channel else 0, 1 if bgra else 0)))
    return o8, oh


def half_to_float(hf):
    hf = _h(hf)
    out = np.empty(hf.shape, np.float32)
    lib().orc_half_to_float(_p(hf), _p(out), _c_size_t(hf.size))
    return out


def preprocess_frames(bgra):
    """bgra uint8 [B][H][W][4] -> fp16 NCHW [B][3][H][W] (planar split then /255)."""
    B, H, W, _ = bgra.shape
    out = np.empty((B, 3, H, W), np.float16)
    for b in range(B):
        planar = bgra_to_planar(bgra[b].reshape(-1), H * W)
        out[b] = convert_normalize(planar).reshape(3, H, W)
    return out


# ------------------------------------------------------------------ activations (return new arrays)
def leaky_relu(x, slope):
    """CudaStuff.cu:400-405."""
    y = _h(x).copy()
    lib().orc_leaky_relu(_p(y), _c_int(y.size), _c_float(slope))
    return y


def swish(x):
    """CudaStuff.cu:416-421."""
    y = _h(x).copy()
    lib().orc_swish(_p(y), _c_int(y.size))
    return y


def relu(x):
    """Activate.cpp:10-21."""
    y = _h(x).copy()
    lib().orc_relu(_p(y), _c_int(y.size))
    return y


def sigmoid_head(x, num_ctrls, num_buts):
    """CudaStuff.cu:437-442."""
    y = _h(x).copy()
    lib().orc_sigmoid_head(_p(y), _c_int(num_ctrls), _c_int(num_buts), _c_int(y.size))
    return y


def tanh_tail(x, num_ctrls, num_buts):
    y = _h(x).copy()
    lib().orc_tanh_tail(_p(y), _c_int(num_ctrls), _c_int(num_buts), _c_int(y.size))
    return y


def add(m, r):
    """ResConvLayer.cpp:35."""
    y = _h(m).copy()
    r = _h(r)
    lib().orc_add(_p(y), _p(r), _c_int(y.size))
    return y


ACT_NONE, ACT_RELU, ACT_SWISH, ACT_LEAKY = 0, 1, 2, 3


def activate(x, act, slope=0.01):
    if act == ACT_NONE:
        return x
    if act == ACT_RELU:
        return relu(x)
    if act == ACT_SWISH:
        return swish(x)
    if act == ACT_LEAKY:
        return leaky_relu(x, slope)
    raise ValueError(act)


# ------------------------------------------------------------------ conv / bn / fc
def conv_out(n, k, s, p):
    return (n + 2 * p - k) // s + 1


def conv2d(x, w, b, stride, pad):
    """ConvLayer.cpp:74-79.  x [B][C][H][W], w [K][C][k][k], b [K]."""
    x, w, b = _h(x), _h(w), _h(b)
    B, C, H, W = x.shape
    K, _, k, _ = w.shape
    y = np.empty((B, K, conv_out(H, k, stride, pad), conv_out(W, k, stride, pad)), np.float16)
    lib().orc_conv2d(_p(x), _p(w), _p(b), _p(y), *map(_c_int, (B, C, H, W, K, k, stride, pad)))
    return y


def conv3d(x, w, b, sd, shw, pd, phw):
    """ConvLayer3D.cpp:106-111.  x [B][C][D][H][W], w [K][C][kd][k][k]."""
    x, w, b = _h(x), _h(w), _h(b)
    B, C, D, H, W = x.shape
    K, _, kd, k, _ = w.shape
    y = np.empty(
        (B, K, conv_out(D, kd, sd, pd), conv_out(H, k, shw, phw), conv_out(W, k, shw, phw)), np.float16
    )
    lib().orc_conv3d(_p(x), _p(w), _p(b), _p(y), *map(_c_int, (B, C, D, H, W, K, kd, k, sd, shw, pd, phw)))
    return y


def batchnorm(x, gamma, beta, mean, var, eps=1e-6, per_activation=False):
    """BatchNorm.cpp:55-63.  x [B][C][...]."""
    x = _h(x)
    B, C = x.shape[:2]
    HW = int(np.prod(x.shape[2:])) if x.ndim > 2 else 1
    y = np.empty(x.shape, np.float16)
    lib().orc_batchnorm(
        _p(x), _p(y), _p(_f(gamma)), _p(_f(beta)), _p(_f(mean)), _p(_f(var)),
        _c_int(B), _c_int(C), _c_int(HW), ctypes.c_double(eps), _c_int(1 if per_activation else 0),
    )
    return y


def fc(x, W, b):
    """FCLayer.cpp:48-53.  x [B][in], W [in][out], b [out] or None."""
    x, W = _h(x), _h(W)
    b = None if b is None else _h(b)
    B, inC = x.shape
    outC = W.shape[1]
    y = np.empty((B, outC), np.float16)
    lib().orc_fc(_p(x), _p(W), _p(b), _p(y), _c_int(B), _c_int(inC), _c_int(outC))
    return y


def fc_backward(x, g, W):
    """FCLayer.cpp:54-59.  x [B][in], g [B][out], W [in][out] -> (grad_w [in][out], grad_b [out], grad_x [B][in])."""
    x, g, W = _h(x), _h(g), _h(W)
    B, inC = x.shape
    outC = W.shape[1]
    gw = np.empty((inC, outC), np.float16)
    gb = np.empty(outC, np.float16)
    gx = np.empty((B, inC), np.float16)
    lib().orc_fc_backward(_p(x), _p(g), _p(W), _p(gw), _p(gb), _p(gx), _c_int(B), _c_int(inC), _c_int(outC))
    return gw, gb, gx


# ------------------------------------------------------------------ norms / attention / pools
def layernorm_ref(x, gamma, beta, N, C, HW, eps=1e-7):
    """CudaStuff.cu:457-515 (per channel over N*HW).  Returns (y, mean[C], var[C])."""
    x = _h(x)
    y = np.empty(x.shape, np.float16)
    mean = np.zeros(C, np.float32)
    var = np.zeros(C, np.float32)
    lib().orc_layernorm_ref(
        _p(y), _p(x), _p(_f(gamma)), _p(_f(beta)), _p(mean), _p(var), _c_int(N), _c_int(C), _c_int(HW),
        _c_float(eps),
    )
    return y, mean, var


def layernorm_rows(x, gamma, beta, eps=1e-5):
    x = _h(x)
    C = x.shape[-1]
    rows = x.size // C
    y = np.empty(x.shape, np.float16)
    lib().orc_layernorm_rows(_p(y), _p(x), _p(_f(gamma)), _p(_f(beta)), _c_int(rows), _c_int(C), _c_float(eps))
    return y


def spatial_attention_ref(x, kW, qW, vW, B, inC, attC, H, W, G=64):
    """CudaStuff.cu:673-746, scalar branch.  Returns dict of out/keyMap/queryMap/valueMap/scores."""
    x = _h(x)
    P = B * H * W
    kMap = np.zeros((P, attC), np.float16)
    qMap = np.zeros((P, attC), np.float16)
    vMap = np.zeros((P, attC), np.float16)
    scores = np.zeros(P, np.float16)
    out = np.zeros((P, attC), np.float16)
    lib().orc_spatial_attention_ref(
        _p(x), _p(_h(kW)), _p(_h(qW)), _p(_h(vW)), _p(kMap), _p(qMap), _p(vMap), _p(scores), _p(out),
        *map(_c_int, (B, inC, attC, H, W, G)),
    )
    return dict(out=out, keyMap=kMap, queryMap=qMap, valueMap=vMap, scores=scores)


def spatial_attention_cfg(x, w1, b1):
    x = _h(x)
    B, C = x.shape[:2]
    HW = int(np.prod(x.shape[2:]))
    y = np.empty(x.shape, np.float16)
    lib().orc_spatial_attention_cfg(_p(x), _p(_h(w1)), _c_float(b1), _p(y), _c_int(B), _c_int(C), _c_int(HW))
    return y


def global_avgpool(x):
    x = _h(x)
    B, C = x.shape[:2]
    HW = int(np.prod(x.shape[2:]))
    y = np.empty((B, C), np.float16)
    lib().orc_global_avgpool(_p(x), _p(y), _c_int(B), _c_int(C), _c_int(HW))
    return y


def adaptive_avgpool3d(x, ph, pw):
    x = _h(x)
    B, C, D, H, W = x.shape
    y = np.empty((B, C * ph * pw), np.float16)
    lib().orc_adaptive_avgpool3d(_p(x), _p(y), *map(_c_int, (B, C, D, H, W, ph, pw)))
    return y


# ------------------------------------------------------------------ sequence operators
def lstm_blob_size(inC, hid, layers, double_bias=True):
    n = 0
    for l in range(layers):
        n += 4 * hid * (inC if l == 0 else hid) + 4 * hid * hid
    n += layers * 4 * hid * (2 if double_bias else 1)
    return n


def lstm(x, blob, hid, layers, clip=5.0, double_bias=True, h_state=None, c_state=None, use_state=False):
    """LSTMLayer.cpp:75-104.  x [T][B][in] -> y [T][B][hid]; states [layers][B][hid] updated in place."""
    x, blob = _h(x), _h(blob)
    T, B, inC = x.shape
    assert blob.size == lstm_blob_size(inC, hid, layers, double_bias)
    y = np.empty((T, B, hid), np.float16)
    lib().orc_lstm(
        _p(x), _p(blob), _p(y), *map(_c_int, (T, B, inC, hid, layers)), _c_float(clip),
        _c_int(1 if double_bias else 0), _p(h_state), _p(c_state), _c_int(1 if use_state else 0),
    )
    return y


def mha(x, wq, wk, wv, wo, heads, rope_base=0.0, pos0=0, window=0):
    """MHALayer.cpp:128-146 (as intended by the layer's fields).  x [B][T][E]."""
    x = _h(x)
    B, T, E = x.shape
    y = np.empty((B, T, E), np.float16)
    lib().orc_mha(
        _p(x), _p(_h(wq)), _p(_h(wk)), _p(_h(wv)), _p(_h(wo)), _p(y), *map(_c_int, (B, T, E, heads)),
        _c_float(rope_base), _c_int(pos0), _c_int(window),
    )
    return y


def actions(p, n_ctrls=16, n_buttons=14):
    """Infer.cpp:8-57."""
    p = _f(p).reshape(-1, n_ctrls)
    out = np.empty(p.shape, np.int32)
    lib().orc_actions(_p(p), _p(out), _c_int(p.shape[0]), _c_int(n_ctrls), _c_int(n_buttons))
    return out
