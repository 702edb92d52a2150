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
