"""The reference's own network (NN.cpp:33-61) built from the reference-compatible C++ layer classes
(ConvLayer, BatchNorm, Activate, ResConvLayer, FCLayer, Sigmoid, NN), loading a checkpoint file in the
reference's byte layout, against the oracle composition of the same layers."""
import ctypes
import os
import tempfile

import numpy as np
import pytest

from oracle import oracle as O
from oracle import pipelines as PL

gpu = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_util as U

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return U


@gpu
def test_reference_network_through_layer_classes(env):
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    lib = pk.lib()
    W, H = 64, 32
    p = PL.make_refnn_params(21, W, H)
    rng = np.random.default_rng(3)
    frame = rng.integers(0, 256, (1, H, W, 4), dtype=np.uint8)
    x = O.preprocess_frames(frame)                           # [1][3][H][W], what ConvertAndNormalize hands to NN::Forward
    want = PL.refnn_forward(p, x)                            # [1][16]
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "AIGamer.ckpt")
        with open(path, "wb") as f:
            f.write(PL.serialize_refnn_checkpoint(p))
        nn = ctypes.c_void_p()
        rc = lib.aig_refnn_create(c.handle, 0, 0, path.encode(), ctypes.byref(nn))
        assert rc == 0, lib.aig_layers_last_error().decode()
    w_, h_ = ctypes.c_int(), ctypes.c_int()
    lib.aig_refnn_input_size(nn, ctypes.byref(w_), ctypes.byref(h_))
    assert (w_.value, h_.value) == (W, H)                    # resolution comes from the checkpoint header (NN.cpp:17-20)
    dx = U.dev(x)
    out = ctypes.c_void_p()
    rc = lib.aig_refnn_forward(nn, pk.ptr(dx), ctypes.byref(out))
    assert rc == 0, lib.aig_layers_last_error().decode()
    got = torch.empty(16, dtype=torch.float16, device="cuda")
    c.call("aig_memcpy", pk.ptr(got), out, 32)
    c.sync()
    got = U.host(got).astype(np.float32)
    # every layer here reproduces the reference's rounding points; what remains is fp32 vs double
    # accumulation through 14 layers: a few fp16 ulps, far inside the 2e-2 relative tolerance
    assert U.rel_err(got, want[0].astype(np.float32), 0.05).max() < 5e-3
    a_got, a_want = O.actions(got, 16, 14), O.actions(want[0].astype(np.float32), 16, 14)
    clear = np.abs(want[0, :14].astype(np.float32) - 0.5) > 2e-3
    assert (a_got[0, :14] == a_want[0, :14])[clear].all()
    # a second forward reuses the layer-owned buffers and gives the same result
    rc = lib.aig_refnn_forward(nn, pk.ptr(dx), ctypes.byref(out))
    got2 = torch.empty(16, dtype=torch.float16, device="cuda")
    c.call("aig_memcpy", pk.ptr(got2), out, 32)
    c.sync()
    assert np.array_equal(U.host(got2).astype(np.float32), got)
    lib.aig_refnn_destroy(nn)


@gpu
def test_missing_checkpoint_and_truncated_checkpoint(env):
    U = env
    c = U.ctx()
    pk = U.pkg()
    lib = pk.lib()
    p = PL.make_refnn_params(22, 64, 32)
    blob = PL.serialize_refnn_checkpoint(p)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "short.ckpt")
        with open(path, "wb") as f:
            f.write(blob[: len(blob) // 2])
        nn = ctypes.c_void_p()
        rc = lib.aig_refnn_create(c.handle, 0, 0, path.encode(), ctypes.byref(nn))
        assert rc != 0 and b"truncated" in lib.aig_layers_last_error()


class _LayerObj:
    """One object of a reference-compatible layer class, driven through the aig_layer_* C hooks."""

    def __init__(self, U, kind, iargs):
        self.U, self.pk = U, U.pkg()
        self.lib, self.c = self.pk.lib(), U.ctx()
        arr = (ctypes.c_int * len(iargs))(*iargs)
        self.h = ctypes.c_void_p()
        rc = self.lib.aig_layer_create(self.c.handle, kind.encode(), arr, len(iargs), ctypes.byref(self.h))
        assert rc == 0, self.lib.aig_layers_last_error().decode()

    def load(self, payload, d):
        path = os.path.join(d, "payload.bin")
        with open(path, "wb") as f:
            f.write(payload)
        rc = self.lib.aig_layer_load_file(self.h, path.encode())
        assert rc == 0, self.lib.aig_layers_last_error().decode()

    def save(self, d):
        path = os.path.join(d, "saved.bin")
        rc = self.lib.aig_layer_save_file(self.h, path.encode())
        assert rc == 0, self.lib.aig_layers_last_error().decode()
        with open(path, "rb") as f:
            return f.read()

    def forward(self, x, count):
        """Layer::Forward on a host array; returns `count` halves from the pointer the layer hands back."""
        import torch

        dx = self.U.dev(np.ascontiguousarray(x, np.float16))
        out = ctypes.c_void_p()
        rc = self.lib.aig_layer_forward(self.h, self.pk.ptr(dx), ctypes.byref(out))
        assert rc == 0, self.lib.aig_layers_last_error().decode()
        got = torch.empty(count, dtype=torch.float16, device="cuda")
        self.c.call("aig_memcpy", self.pk.ptr(got), out, count * 2)
        self.c.sync()
        return self.U.host(got), (out.value == dx.data_ptr())

    def close(self):
        self.lib.aig_layer_destroy(self.h)


def _b(*arrays):
    return b"".join(np.ascontiguousarray(a).tobytes() for a in arrays)


@gpu
def test_layer_classes_not_reached_by_the_reference_network(env):
    """LayerNorm, SpatialAttentionLayer, LSTMLayer (both constructor forms), MultiHeadAttentionLayer,
    ConvLayer3D, Swish, LeakyReLU and Dropout: constructed with the reference's argument lists, parameters
    loaded from a payload in the reference's byte layout, Forward against the oracle, and SaveParameters
    writing back the very bytes that were loaded."""
    U = env
    import math

    from ai_gamer_b200 import synth as SY

    rng = np.random.default_rng(77)
    f16 = np.float16
    with tempfile.TemporaryDirectory() as d:
        # ---- ConvLayer3D (ConvLayer3D.h:8): batch, inC, outC, kD, kHW, sD, sHW, pD, pHW, width, height, depth
        B, C, K, D, H, W = 2, 16, 32, 4, 8, 16
        L = _LayerObj(U, "ConvLayer3D", [B, C, K, 3, 3, 1, 2, 1, 1, W, H, D])
        w, b = SY.he_normal(rng, (K, C, 3, 3, 3)), rng.uniform(-0.2, 0.2, K).astype(f16)
        payload = _b(w, b)
        L.load(payload, d)
        x = rng.standard_normal((B, C, D, H, W)).astype(f16)
        want = O.conv3d(x, w, b, 1, 2, 1, 1)
        got, _ = L.forward(x, want.size)
        U.assert_two_step(got.reshape(want.shape), want, b.astype(np.float64)[None, :, None, None, None], "ConvLayer3D")
        assert L.save(d) == payload
        L.close()
        # ---- LayerNorm (LayerNorm.h:6): batch, channels, height, width; statistics per channel over N*H*W
        N, C, H, W = 4, 8, 4, 4
        L = _LayerObj(U, "LayerNorm", [N, C, H, W])
        g, be = rng.uniform(0.5, 1.5, C).astype(np.float32), rng.uniform(-0.5, 0.5, C).astype(np.float32)
        payload = _b(g, be)
        L.load(payload, d)
        x = rng.standard_normal((N, C, H, W)).astype(f16)
        want, _, _ = O.layernorm_ref(x, g, be, N, C, H * W)
        got, _ = L.forward(x, want.size)
        U.assert_close16(got.reshape(want.shape), want, max_ulp=2, what="LayerNorm")
        assert L.save(d) == payload
        L.close()
        # ---- SpatialAttentionLayer (SpatialAttentionLayer.h:7): attC, batch, channels, height, width
        A, B, C, H, W = 4, 2, 8, 4, 8
        L = _LayerObj(U, "SpatialAttentionLayer", [A, B, C, H, W])
        kq = lambda: (rng.standard_normal(C * 9) * 0.3).astype(f16)
        kW, qW, vW = kq(), kq(), (rng.standard_normal(C * A) * 0.3).astype(f16)
        payload = _b(kW, qW, vW)
        L.load(payload, d)
        x = rng.standard_normal((B, C, H, W)).astype(f16)
        want = O.spatial_attention_ref(x, kW, qW, vW, B, C, A, H, W, 64)["out"]
        got, _ = L.forward(x, want.size)
        U.assert_close16(got.reshape(want.shape), want, max_ulp=1, what="SpatialAttentionLayer")
        assert L.save(d) == payload
        L.close()
        # ---- LSTMLayer (LSTMLayer.h:8): seqLength, numLayers, hiddenSize, batchSize, inC
        T, NL, HID, B, I = 8, 2, 64, 4, 32
        L = _LayerObj(U, "LSTMLayer", [T, NL, HID, B, I])
        blob = SY.make_lstm_blob(rng, I, HID, NL, True, 1.0)
        blob[-4 * HID:] = rng.uniform(-0.2, 0.2, 4 * HID).astype(f16)
        assert L.lib.aig_layer_param_bytes(L.h) == blob.nbytes
        L.load(_b(blob), d)
        x = rng.standard_normal((T, B, I)).astype(f16)
        want = O.lstm(x, blob, HID, NL, 5.0, True)[-1]                      # LSTMLayer.cpp:103: the last step's rows
        got, _ = L.forward(x, want.size)
        assert np.abs(got.reshape(want.shape).astype(np.float32) - want.astype(np.float32)).max() < 6e-3
        assert L.save(d) == _b(blob)
        L.close()
        # ---- LSTMLayer, cuDNN-8 form (LSTMLayerv8.h:10): batch, seq, inCHW, outC, numLayers; returns hy
        L = _LayerObj(U, "LSTMLayerV8", [B, T, I, HID, NL])
        blob1 = SY.make_lstm_blob(rng, I, HID, NL, False, 1.0)
        assert L.lib.aig_layer_param_bytes(L.h) == blob1.nbytes
        L.load(_b(blob1), d)
        hs, cs = np.zeros((NL, B, HID), f16), np.zeros((NL, B, HID), f16)
        O.lstm(x, blob1, HID, NL, 0.0, False, hs, cs, False)
        got, _ = L.forward(np.ascontiguousarray(x.transpose(1, 0, 2)), hs.size)
        assert np.abs(got.reshape(hs.shape).astype(np.float32) - hs.astype(np.float32)).max() < 6e-3
        assert L.save(d) == _b(blob1)
        L.close()
        # ---- MultiHeadAttentionLayer (MHALayer.h:9): batch, seq, embed, heads
        B, T, E, NH = 2, 16, 128, 2
        L = _LayerObj(U, "MultiHeadAttentionLayer", [B, T, E, NH])
        ws = [SY.xavier_uniform(rng, (E, E), E, E) for _ in range(4)]
        payload = _b(*ws)
        L.load(payload, d)
        x = rng.standard_normal((B, T, E)).astype(f16)
        want = O.mha(x, *ws, NH, 0.0)
        got, _ = L.forward(x, want.size)
        assert U.scaled_err(got.reshape(want.shape), want) < 1e-2
        assert L.save(d) == payload
        L.close()
        # ---- ResConvLayer (ResConvLayer.h:12): the payload order Conv0, BN0, Conv1, BN1, shortcut survives a round trip
        L = _LayerObj(U, "ResConvLayer", [1, 32, 64, 16, 32])
        p = SY.make_resconv_params(rng, 32, 64, False)
        payload = _b(p["c0w"], p["c0b"]) + SY._bn_bytes(p["bn0"]) + _b(p["c1w"], p["c1b"]) + SY._bn_bytes(p["bn1"]) + _b(p["sw"], p["sb"])
        L.load(payload, d)
        assert L.save(d) == payload
        L.close()
    # ---- in-place activations (Swish.h:6, LeakyReLU.h:7 with slope 1/128, Dropout.h:8 at inference)
    x = (rng.standard_normal(1000) * 3).astype(f16)
    for kind, iargs, want in (("Swish", [1000], O.swish(x)), ("LeakyReLU", [1000], O.leaky_relu(x, 1.0 / 128.0)),
                              ("Dropout", [1, 10, 10, 10], x)):
        L = _LayerObj(U, kind, iargs)
        got, in_place = L.forward(x, 1000)
        assert in_place, kind + " must return its argument"
        U.assert_close16(got, want, max_ulp=1 if kind == "Swish" else 0, what=kind)
        L.close()
    assert math.isfinite(float(got.astype(np.float32).sum()))


@gpu
def test_infer_loop_body_through_the_reference_names_without_synchronisation(env):
    """Infer.cpp:103-112 as the reference writes it -- ARGBtoRGBplanar, ConvertAndNormalize, NN::Forward,
    ConvertHalfToFloat, cudaMemcpy -- on a handle made the way Infer.cpp:76-79 makes it, with no stream or
    event call in between: the legacy default stream alone must order the steps, frame after frame."""
    U = env
    import torch

    pk = U.pkg()
    lib = pk.lib()
    W, H = 64, 32
    p = PL.make_refnn_params(23, W, H)
    handle = ctypes.c_void_p()
    assert lib.aig_compat_handle_create(ctypes.byref(handle)) == 0
    assert lib.aig_ctx_stream(handle) is None                 # the legacy default stream
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "AIGamer.ckpt")
        with open(path, "wb") as f:
            f.write(PL.serialize_refnn_checkpoint(p))
        nn = ctypes.c_void_p()
        rc = lib.aig_refnn_create(handle, 0, 0, path.encode(), ctypes.byref(nn))
        assert rc == 0, lib.aig_layers_last_error().decode()
    rng = np.random.default_rng(8)
    frames = rng.integers(0, 256, (6, H, W, 4), dtype=np.uint8)
    d_frames = [U.dev(f) for f in frames]
    planar = torch.zeros(3 * H * W, dtype=torch.uint8, device="cuda")
    half = torch.zeros(3 * H * W, dtype=torch.float16, device="cuda")
    out_dev = torch.zeros(16, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    out_host = np.zeros(16, np.float32)
    for i in range(frames.shape[0]):
        rc = lib.aig_refnn_infer_frame(nn, pk.ptr(d_frames[i]), pk.ptr(planar), pk.ptr(half), pk.ptr(out_dev), pk.ptr(out_host))
        assert rc == 0, lib.aig_layers_last_error().decode()
        want = PL.refnn_forward(p, O.preprocess_frames(frames[i:i + 1]))[0].astype(np.float32)
        assert U.rel_err(out_host, want, 0.05).max() < 5e-3, "frame %d" % i
    lib.aig_refnn_destroy(nn)
    lib.aig_ctx_destroy(handle)
