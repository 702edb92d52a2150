"""Oracle compositions for the benchmark configurations.

TEST INFRASTRUCTURE ONLY (see oracle.py).  The compositions restate how the reference chains its
operators (NN.cpp:33-61, ResConvLayer.cpp:28-37) for the operator mixes the benchmark
configurations name.  Parameters and inputs come from the package's seeded generators
(ai-gamer_b200/synth.py), re-exported here for the tests.
"""
import importlib.util
import os
import sys

import numpy as np

from . import oracle as O

_SYNTH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ai-gamer_b200", "synth.py")
if "aig_synth" in sys.modules:
    _synth = sys.modules["aig_synth"]
else:
    _spec = importlib.util.spec_from_file_location("aig_synth", _SYNTH)
    _synth = importlib.util.module_from_spec(_spec)
    sys.modules["aig_synth"] = _synth
    _spec.loader.exec_module(_synth)
for _n in dir(_synth):
    if not _n.startswith("_"):
        globals()[_n] = getattr(_synth, _n)


# ----------------------------------------------------------------------------- oracle compositions
def resconv_forward(x, p, act):
    """ResConvLayer.cpp:28-37 with the block's activation swappable (ReLU in the reference)."""
    r = O.conv2d(x, p["sw"], p["sb"], 2, 0)
    m = O.conv2d(x, p["c0w"], p["c0b"], 2, 1)
    m = O.activate(O.batchnorm(m, *p["bn0"]), act)
    m = O.conv2d(m, p["c1w"], p["c1b"], 1, 1)
    m = O.batchnorm(m, *p["bn1"])
    m = O.add(m, r)
    return O.activate(m, act)


def cnn_forward(p, bgra, act=O.ACT_SWISH, n_sigmoid=16, return_all=False):
    """BGRA frames [B][H][W][4] -> (features [B][C], logits [B][n_out], outputs [B][n_out])."""
    x = O.preprocess_frames(bgra)
    pad0 = p["k0"] // 2
    x = O.conv2d(x, p["c0w"], p["c0b"], 2, pad0)
    x = O.activate(O.batchnorm(x, *p["bn0"]), act)
    stages = [x]
    for blk in p["res"]:
        x = resconv_forward(x, blk, act)
        stages.append(x)
    x = O.spatial_attention_cfg(x, p["sa_w"], p["sa_b"])
    feat = O.global_avgpool(x)
    logits = O.fc(feat, p["fcW"], p["fcb"])
    out = O.tanh_tail(O.sigmoid_head(logits, p["n_out"], n_sigmoid), p["n_out"], n_sigmoid)
    if return_all:
        return feat, logits, out, stages
    return feat, logits, out


# config 1: FC -> row LayerNorm -> Swish
def fc_ln_swish_forward(p, x, eps=1e-5):
    y = O.fc(x, p["W"], p["b"])
    y = O.layernorm_rows(y, p["gamma"], p["beta"], eps)
    return O.swish(y)


# config 3: Conv3D temporal encoder
def conv3d_forward(p, clips, slope=0.01, n_sigmoid=16):
    x = clips
    for L in p["layers"]:
        x = O.conv3d(x, L["w"], L["b"], 1, 2, 1, 1)
        x = O.leaky_relu(O.batchnorm(x, *L["bn"]), slope)
    feat = O.adaptive_avgpool3d(x, 2, 2)
    logits = O.fc(feat, p["fcW"], p["fcb"])
    out = O.tanh_tail(O.sigmoid_head(logits, p["n_out"], n_sigmoid), p["n_out"], n_sigmoid)
    return feat, logits, out


# config 4: sequence head
def seq_forward(p, emb, rope_base=10000.0, window=0, n_sigmoid=16, pos0=0, h_state=None, c_state=None,
                use_state=False):
    """emb [T][B][d] -> logits/outputs [B][T][n_out] (LSTM -> causal MHA + RoPE -> row LN -> FC)."""
    T, B, _ = emb.shape
    y = O.lstm(emb, p["lstm"], p["hid"], p["layers"], 5.0, True, h_state, c_state, use_state)
    ybt = np.ascontiguousarray(y.transpose(1, 0, 2))
    a = O.mha(ybt, p["wq"], p["wk"], p["wv"], p["wo"], p["heads"], rope_base, pos0, window)
    n = O.layernorm_rows(a, p["ln_g"], p["ln_b"], 1e-5)
    logits = O.fc(n.reshape(B * T, -1), p["fcW"], p["fcb"])
    out = O.tanh_tail(O.sigmoid_head(logits, p["n_out"], n_sigmoid), p["n_out"], n_sigmoid)
    return y, a, logits.reshape(B, T, -1), out.reshape(B, T, -1)


def refnn_forward(p, x_nchw):
    """The network NN::NN builds (NN.cpp:33-61) on planar fp16 frames [B][3][H][W]: Conv k2 s2 + BN + ReLU,
    three ResConv blocks (ReLU), three FC + per-activation BN + ReLU, FC(16), Sigmoid on the first 14."""
    x = O.conv2d(x_nchw, p["c0w"], p["c0b"], 2, 0)
    x = O.relu(O.batchnorm(x, *p["bn0"]))
    for blk in p["res"]:
        x = resconv_forward(x, blk, O.ACT_RELU)
    x = x.reshape(x.shape[0], -1)
    for L in p["fc"]:
        x = O.relu(O.batchnorm(O.fc(x, L["W"], L["b"]), *L["bn"], per_activation=True))
    y = O.fc(x, p["outW"], p["outb"])
    return O.sigmoid_head(y, 16, 14)
