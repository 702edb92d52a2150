"""End-to-end GPU parity of the 2-D frame encoder (host runner + kernels) against the oracle
composition, on the benchmark configuration's shapes at a batch the oracle finishes in seconds."""
import numpy as np
import pytest

from oracle import oracle as O
from oracle import pipelines as PL

gpu = pytest.mark.gpu

REL_TOL = 2e-2    # relative tolerance on the key/mouse outputs (fp16 compute, fp32 accumulation)
STAGE_TOL = 1e-2  # intermediate activations: max error relative to max(|value|, rms of the tensor)


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_util as U

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return U


@gpu
@pytest.mark.parametrize("trivial", [True, False])
def test_cnn_encoder_matches_oracle(env, trivial):
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    B, H, W = 4, 144, 256
    widths = (32, 64, 128, 256, 256)
    params = PL.make_cnn_params(0 if trivial else 1, widths=widths, trivial=trivial)
    frames = PL.make_frames(0, B, H, W)
    feat, logits, want, stages = PL.cnn_forward(params, frames, return_all=True)
    enc = pk.CnnEncoder(c, B, H, W, widths=widths)
    blob = PL.serialize_cnn_checkpoint(params, W, H)
    assert len(blob) == enc.checkpoint_bytes()
    enc.load_bytes(blob)
    d_frames = U.dev(frames)
    enc.forward(d_frames)
    c.sync()
    # layer by layer first: a failure names the first stage that drifts
    for i, st in enumerate(stages):
        got = U.nchw(U.host(enc.stage_output(i)))
        err = U.scaled_err(got, st)
        assert err < STAGE_TOL, "stage %d: max scaled err %.4f" % (i, err)
    got_feat = U.host(enc.features())
    assert U.rel_err(got_feat, feat, 0.02).max() < REL_TOL
    got = U.host(enc.outputs_f32())
    assert np.array_equal(got.astype(np.float16), U.host(enc.outputs_half()))
    assert U.rel_err(got, want.astype(np.float32), 0.05).max() < REL_TOL
    # decisions (Infer.cpp:8-57): button thresholds must agree wherever the oracle is not within the
    # tolerance of the 0.5 threshold; the mouse deltas (int(p*256)) may differ by one count
    a_got, a_want = O.actions(got, 18, 16), O.actions(want.astype(np.float32), 18, 16)
    clear = np.abs(want.astype(np.float32)[:, :16] - 0.5) > 2e-3
    assert (a_got[:, :16] == a_want[:, :16])[clear].all()
    assert (a_got[:, :16] == a_want[:, :16]).mean() >= 0.999
    assert np.abs(a_got[:, 16:] - a_want[:, 16:]).max() <= 1
    # graph replay and the host-buffer frame step give the same bytes
    enc.forward(d_frames, graph=True)
    c.sync()
    assert np.array_equal(U.host(enc.outputs_f32()), got)
    pinned_in = torch.from_numpy(frames).pin_memory()
    pinned_out = torch.empty((B, 18), dtype=torch.float32).pin_memory()
    enc.infer_host(pinned_in, pinned_out)
    assert np.array_equal(pinned_out.numpy(), got)
    # pipelined submit/wait over two slots: same bytes, any order of slots
    outs = [torch.zeros((B, 18), dtype=torch.float32).pin_memory() for _ in range(2)]
    for step in range(5):
        if step >= 2:
            enc.wait(step & 1)
            assert np.array_equal(outs[step & 1].numpy(), got)
            outs[step & 1].zero_()
        enc.submit_host(step & 1, pinned_in, outs[step & 1])
    for step in (3, 4):
        enc.wait(step & 1)
        assert np.array_equal(outs[step & 1].numpy(), got)
    enc.close()


@gpu
def test_cnn_checkpoint_errors(env):
    U = env
    c = U.ctx()
    pk = U.pkg()
    widths = (32, 64)
    enc = pk.CnnEncoder(c, 1, 32, 64, widths=widths)
    params = PL.make_cnn_params(3, widths=widths)
    blob = PL.serialize_cnn_checkpoint(params, 64, 32)
    with pytest.raises(pk.AigError):
        enc.load_bytes(blob[:-2])  # truncated
    with pytest.raises(pk.AigError):
        enc.load_bytes(PL.serialize_cnn_checkpoint(params, 32, 64))  # wrong resolution in the header
    with pytest.raises(pk.AigError):
        import torch

        enc.forward(torch.zeros(1, dtype=torch.uint8, device="cuda"))  # parameters not loaded
    enc.load_bytes(blob)
    enc.close()


@gpu
def test_full_size_properties(env):
    """The benchmark's own size (256 frames of 144x256) is beyond what the CPU oracle finishes in seconds, so
    the full-size run is checked through properties that do not need it: frames are independent (a frame's
    outputs do not depend on the batch it travels in, up to the fp32 summation order of the tile shape chosen
    for that batch), the run is deterministic bit for bit, the oracle agrees
    on a sample of the frames, and the two convolution paths (fused down-sampling over space-to-depth vs the
    two separate stride-2 convolutions) agree within the fp16 tolerance."""
    U = env
    import os

    c = U.ctx()
    pk = U.pkg()
    B, H, W = 256, 144, 256
    widths = (32, 64, 128, 256, 256)
    params = PL.make_cnn_params(4, widths=widths, trivial=False)
    blob = PL.serialize_cnn_checkpoint(params, W, H)
    frames = PL.make_frames(11, B, H, W)
    enc = pk.CnnEncoder(c, B, H, W, widths=widths)
    enc.load_bytes(blob)
    d_frames = U.dev(frames)
    enc.forward(d_frames)
    c.sync()
    full = U.host(enc.outputs_f32()).copy()
    assert np.isfinite(full).all()
    enc.forward(d_frames)
    c.sync()
    assert np.array_equal(U.host(enc.outputs_f32()), full), "two runs on the same frames differ"
    enc.close()
    # the same frames in batches of 8: other tile shapes (channel-block groups are summed in another order),
    # same values up to a few fp16 ulps; within one batch size the bytes do not depend on the position in the batch
    small = pk.CnnEncoder(c, 8, H, W, widths=widths)
    small.load_bytes(blob)
    for lo in (0, 120, 248):
        small.forward(U.dev(frames[lo:lo + 8]))
        c.sync()
        assert np.abs(U.host(small.outputs_f32()) - full[lo:lo + 8]).max() < 2e-3, "outputs depend on the batch composition"
    small.forward(U.dev(np.ascontiguousarray(frames[7::-1])))
    c.sync()
    rev = U.host(small.outputs_f32()).copy()
    small.forward(U.dev(frames[0:8]))
    c.sync()
    assert np.array_equal(U.host(small.outputs_f32()), rev[::-1]), "a frame's outputs depend on its position in the batch"
    small.close()
    # the oracle on three of the 256 frames
    pick = [0, 131, 255]
    _, _, want = PL.cnn_forward(params, frames[pick])
    assert U.rel_err(full[pick], want.astype(np.float32), 0.05).max() < REL_TOL
    a_got, a_want = O.actions(full[pick], 18, 16), O.actions(want.astype(np.float32), 18, 16)
    clear = np.abs(want.astype(np.float32)[:, :16] - 0.5) > 2e-3
    assert (a_got[:, :16] == a_want[:, :16])[clear].all()
    # the unfused path (two separate stride-2 convolutions per block) on the same frames
    os.environ["AIG_CNN_NO_FUSED_DOWN"] = "1"
    try:
        plain = pk.CnnEncoder(c, B, H, W, widths=widths)
    finally:
        del os.environ["AIG_CNN_NO_FUSED_DOWN"]
    plain.load_bytes(blob)
    plain.forward(d_frames)
    c.sync()
    other = U.host(plain.outputs_f32())
    plain.close()
    assert np.abs(other - full).max() < 4e-3   # outputs live in [-1, 1]


@gpu
def test_recording_file_to_batched_inference(env, tmp_path):
    """Records of the reference's recording format -> planar RGB frames -> batched inference through the pipelined
    host entry point: same outputs as the device path on the BGRA form of the same frames, action agreement with the
    oracle on every record, the last (partial) batch included."""
    U = env
    import struct

    c = U.ctx()
    pk = U.pkg()
    B, H, W, n = 4, 144, 256, 11
    widths = (32, 64, 128, 256, 256)
    params = PL.make_cnn_params(6, widths=widths, trivial=False)
    bgra = PL.make_frames(21, n, H, W)
    planar = np.ascontiguousarray(bgra[..., [2, 1, 0]].transpose(0, 3, 1, 2))          # what the recorder stores
    rng = np.random.default_rng(2)
    keys = rng.integers(0, 1 << 14, n).astype(np.uint16)
    mouse = rng.integers(-200, 200, (n, 2)).astype(np.int32)
    path = tmp_path / "training_data.bin"
    with open(path, "wb") as f:
        f.write(struct.pack("<ii", W, H))
        for i in range(n):
            f.write(struct.pack("<Hii", int(keys[i]), int(mouse[i, 0]), int(mouse[i, 1])))
            f.write(planar[i].tobytes())
    rec = pk.Recording(path)
    assert (rec.width, rec.height, rec.n_records) == (W, H, n)
    enc = pk.CnnEncoder(c, B, H, W, widths=widths)
    enc.load_bytes(PL.serialize_cnn_checkpoint(params, W, H))
    got = rec.infer(enc, 0, n)
    # the device path on BGRA frames, batch by batch
    want_dev = []
    for lo in range(0, n, B):
        chunk = bgra[lo:lo + B]
        if chunk.shape[0] < B:
            chunk = np.concatenate([chunk, np.repeat(chunk[-1:], B - chunk.shape[0], axis=0)])
        enc.forward(U.dev(chunk))
        c.sync()
        want_dev.append(U.host(enc.outputs_f32())[: min(B, n - lo)])
    assert np.array_equal(got, np.concatenate(want_dev)), "planar RGB records and BGRA frames give different outputs"
    # a sub-range
    assert np.array_equal(rec.infer(enc, 3, 5), got[3:8])
    _, _, want = PL.cnn_forward(params, bgra)
    want = want.astype(np.float32)
    assert np.abs(got - want).max() < 2e-3
    a_got, a_want = O.actions(got, 18, 16), O.actions(want, 18, 16)
    clear = np.abs(want[:, :16] - 0.5) > 2e-3
    assert (a_got[:, :16] == a_want[:, :16])[clear].all()
    # the recorded inputs come back as the reference's training targets (Train.cpp:70-76)
    _, k, m = rec.read(0, n)
    t = pk.Recording.targets(k, m)
    assert np.array_equal(t[:, :14], ((keys[:, None] >> np.arange(14)) & 1).astype(np.float32))
    enc.close()
    rec.close()
