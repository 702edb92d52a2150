"""GPU parity of the host-side runners for the sequence head (LSTM -> MHA -> LayerNorm -> FC) and
the streaming agent (frame encoder -> FC -> sequence-head step with carried state and ring cache)
against the oracle compositions.  Streaming must reproduce the full-sequence forward step by step."""
import numpy as np
import pytest

from oracle import oracle as O
from oracle import pipelines as PL

gpu = pytest.mark.gpu
TOL = 2e-2  # relative tolerance on the outputs (fp16 compute), see the north-star statement


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_util as U

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return U


def _seq_head(U, batch, seq_len, d, heads, window):
    from ai_gamer_b200 import runners as R

    return R.SeqHead(U.ctx(), batch, seq_len, in_c=d, hidden=d, layers=2, heads=heads, rope_base=10000.0, window=window)


@gpu
@pytest.mark.parametrize("B", [4, 6, 1])   # up to 4 sequences stream through the one-kernel step, more through the per-operator launches
def test_sequence_head_full_and_streaming(env, B):
    U = env
    U.pkg()
    T, d, heads = 16, 128, 2
    p = PL.make_seq_params(5, d=d, hid=d, layers=2, heads=heads)
    emb = PL.make_embeddings(5, T, B, d)                    # [T][B][d]
    y, a, logits, want = PL.seq_forward(p, emb, rope_base=10000.0, window=0)
    head = _seq_head(U, B, T, d, heads, 0)
    blob = PL.serialize_seq_params(p)
    assert len(blob) == head.param_bytes()
    head.load_bytes(blob)
    emb_bt = np.ascontiguousarray(emb.transpose(1, 0, 2))    # the runner is batch-major
    head.forward(U.dev(emb_bt))
    got_y = U.host(head.lstm_output())
    assert np.abs(got_y.astype(np.float32) - y.transpose(1, 0, 2).astype(np.float32)).max() < 6e-3
    got = U.host(head.outputs_f32())
    assert U.rel_err(got, want.astype(np.float32), 0.05).max() < TOL
    # streaming: the same sequence one frame at a time
    outs = []
    for t in range(T):
        head.step(U.dev(np.ascontiguousarray(emb[t])))
        outs.append(U.host(head.outputs_f32(step=True)))
    got_s = np.stack(outs, axis=1)
    assert U.rel_err(got_s, want.astype(np.float32), 0.05).max() < TOL
    assert np.abs(got_s - got).max() < 5e-3, "streaming and full-sequence forward disagree"
    # reset starts a new sequence
    head.reset()
    head.step(U.dev(np.ascontiguousarray(emb[0])))
    assert np.abs(U.host(head.outputs_f32(step=True)) - got_s[:, 0]).max() < 1e-6
    head.close()


@gpu
def test_streaming_agent_matches_oracle(env):
    U = env
    import torch

    U.pkg()
    from ai_gamer_b200 import runners as R

    B, H, W, widths, d, heads, window, steps = 2, 32, 64, (32, 64), 128, 2, 8, 12
    p = PL.make_agent_params(3, widths=widths, d=d, layers=2, heads=heads)
    frames = [PL.make_frames(100 + t, B, H, W) for t in range(steps)]
    emb = np.stack([O.fc(PL.cnn_forward(p["cnn"], f)[0], p["bw"], p["bb"]) for f in frames])   # [T][B][d]
    _, _, _, want = PL.seq_forward(p["seq"], emb, rope_base=10000.0, window=window)             # [B][T][n_out]
    agent = R.Agent(U.ctx(), B, H, W, widths=widths, d=d, layers=2, heads=heads, window=window)
    blob = PL.serialize_agent_params(p, W, H)
    assert len(blob) == agent.param_bytes()
    agent.load_bytes(blob)
    outs = []
    for t in range(steps):
        agent.step(U.dev(frames[t]))
        outs.append(U.host(agent.outputs_f32()))
    got = np.stack(outs, axis=1)
    assert U.rel_err(got, want.astype(np.float32), 0.05).max() < TOL
    # the host-buffer frame step returns the same numbers
    agent.reset()
    out_h = torch.empty((B, 18), dtype=torch.float32).pin_memory()
    for t in range(3):
        agent.step_host(torch.from_numpy(frames[t]).pin_memory(), out_h)
        assert np.array_equal(out_h.numpy(), got[:, t])
    agent.close()


@gpu
def test_clip_encoder_matches_oracle(env):
    """Conv3D temporal encoder (three Conv3D+BN+LeakyReLU layers, 2x2 adaptive pool, FC head) on short
    clips against the oracle composition, with non-trivial BatchNorm statistics and biases."""
    U = env
    U.pkg()
    from ai_gamer_b200 import runners as R

    B, D, H, W = 2, 4, 32, 64
    p = PL.make_conv3d_params(7, trivial=False)
    clips = PL.make_clips(7, B, D, H, W)
    feat, logits, want = PL.conv3d_forward(p, clips)
    enc = R.ClipEncoder(U.ctx(), B, D, H, W)
    blob = PL.serialize_conv3d_params(p)
    assert len(blob) == enc.param_bytes()
    enc.load_bytes(blob)
    enc.forward(U.dev(clips))
    got_feat = U.host(enc.features()).astype(np.float32)
    assert U.scaled_err(got_feat, feat.astype(np.float32)) < 1e-2
    got = U.host(enc.outputs_f32())
    assert U.rel_err(got, want.astype(np.float32), 0.05).max() < TOL
    # a second call on the same buffers is deterministic
    enc.forward(U.dev(clips))
    assert np.array_equal(U.host(enc.outputs_f32()), got)
    with pytest.raises(Exception, match="size"):
        enc.load_bytes(blob[:-2])                            # a short blob is refused before anything is copied
    enc.close()


@gpu
@pytest.mark.parametrize("rows", [32, 64])
def test_fc_layernorm_swish_twin(env, rows):
    """The CPU-runnable configuration's GPU twin: FC 1024->1024, row LayerNorm (eps 1e-5), Swish; 64 rows is the
    configuration's own batch."""
    U = env
    pk = U.pkg()
    import torch

    c = U.ctx()
    d = 1024
    p = PL.make_fc_ln_params(11, d, d)
    x = np.random.default_rng(11).standard_normal((rows, d)).astype(np.float16)
    want = PL.fc_ln_swish_forward(p, x)
    plan = pk.FcPlan(c, rows, d, d, two_step=True)
    dW, db, dg, dbeta, dx = (U.dev(a) for a in (p["W"], p["b"], p["gamma"], p["beta"], x))  # kept alive to the sync
    plan.set_weights(dW, db)
    y = torch.empty((rows, d), dtype=torch.float16, device="cuda")
    plan.forward(dx, y)
    z = torch.empty_like(y)
    c.call("aig_layernorm_rows_forward", U.p(z), U.p(y), U.p(dg), U.p(dbeta), rows, d, 1e-5)
    c.call("aig_swish_forward", U.p(z), rows * d)
    c.sync()
    got = U.host(z).astype(np.float32)
    assert np.abs(got - want.astype(np.float32)).max() < 6e-3
    assert U.rel_err(got, want.astype(np.float32), 0.05).max() < TOL
