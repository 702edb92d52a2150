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
