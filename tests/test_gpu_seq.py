"""GPU parity of the sequence operators (LSTM, multi-head attention with RoPE and the ring KV cache)
through the C ABI against the CPU oracle.  The reference delegates both to cuDNN and pins nothing:
the oracle's definitions (gate order, blob layout, weight orientation, RoPE) are this library's."""
import numpy as np
import pytest

from oracle import oracle as O
from oracle import pipelines as PL

gpu = pytest.mark.gpu


def h(a):
    return np.asarray(a, np.float32).astype(np.float16)


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_util as U

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return U


LSTM_CASES = [
    # T, B, in, hid, layers, clip, double_bias
    (6, 3, 64, 64, 1, 5.0, True),
    (8, 20, 32, 128, 2, 5.0, True),
    (5, 130, 64, 64, 2, 0.0, False),     # two batch groups, single bias, no clip
    (16, 128, 512, 512, 2, 5.0, True),   # the sequence-head geometry at a short length
]


@gpu
@pytest.mark.parametrize("T,B,I,H,L,clip,dbl", LSTM_CASES)
def test_lstm_matches_oracle(env, T, B, I, H, L, clip, dbl):
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    rng = np.random.default_rng(T * 1000 + B)
    blob = PL.make_lstm_blob(rng, I, H, L, dbl, 1.0)
    if dbl:
        blob[-4 * H:] = h(rng.uniform(-0.2, 0.2, 4 * H))
    x = h(rng.standard_normal((T, B, I)))
    assert blob.size == pk.lib().aig_lstm_weight_count(I, H, L, 1 if dbl else 0)
    want = O.lstm(x, blob, H, L, clip, dbl)
    plan = pk.LstmPlan(c, T, L, H, B, I, clip=clip, double_bias=dbl)
    d_blob = U.dev(blob)
    plan.set_weights(d_blob)
    dy = torch.zeros(T * B * H, dtype=torch.float16, device="cuda")
    plan.forward(U.dev(x), dy)
    c.sync()
    got = U.host(dy).reshape(T, B, H)
    err = np.abs(got.astype(np.float32) - want.astype(np.float32)).max()
    assert err < 6e-3, "max |h - oracle| = %.4g" % err
    # carried state: two halves with state == one pass over the whole sequence
    if T % 2 == 0:
        half = T // 2
        plan2 = pk.LstmPlan(c, half, L, H, B, I, clip=clip, double_bias=dbl)
        plan2.set_weights(d_blob)
        hs = torch.zeros(L * B * H, dtype=torch.float16, device="cuda")
        cs = torch.zeros(L * B * H, dtype=torch.float16, device="cuda")
        y1 = torch.zeros(half * B * H, dtype=torch.float16, device="cuda")
        y2 = torch.zeros(half * B * H, dtype=torch.float16, device="cuda")
        plan2.forward(U.dev(x[:half]), y1, hs, cs, use_state=True)
        plan2.forward(U.dev(x[half:]), y2, hs, cs, use_state=True)
        c.sync()
        both = np.concatenate([U.host(y1), U.host(y2)]).reshape(T, B, H)
        assert np.array_equal(both, got), "streaming halves differ from the full-sequence pass"
        plan2.close()
    plan.close()


@gpu
def test_lstm_batch_major_and_step_by_step(env):
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    T, B, I, H, L = 4, 5, 64, 64, 2
    rng = np.random.default_rng(77)
    blob = PL.make_lstm_blob(rng, I, H, L, False, 1.0)
    x = h(rng.standard_normal((T, B, I)))
    want = O.lstm(x, blob, H, L, 0.0, False)
    d_blob = U.dev(blob)
    # cuDNN-8 style layer: batch-major in and out, single bias, no clip (LSTMLayerv8.cpp:9,12,80)
    plan = pk.LstmPlan(c, T, L, H, B, I, clip=0.0, double_bias=False, batch_major=True)
    plan.set_weights(d_blob)
    dy = torch.zeros(B * T * H, dtype=torch.float16, device="cuda")
    plan.forward(U.dev(np.ascontiguousarray(x.transpose(1, 0, 2))), dy)
    c.sync()
    got = U.host(dy).reshape(B, T, H).transpose(1, 0, 2)
    assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() < 6e-3
    # one step at a time with carried state
    step = pk.LstmPlan(c, 1, L, H, B, I, clip=0.0, double_bias=False)
    step.set_weights(d_blob)
    hs = torch.zeros(L * B * H, dtype=torch.float16, device="cuda")
    cs = torch.zeros(L * B * H, dtype=torch.float16, device="cuda")
    outs = []
    for t in range(T):
        y = torch.zeros(B * H, dtype=torch.float16, device="cuda")
        step.forward(U.dev(x[t:t + 1]), y, hs, cs, use_state=True)
        outs.append(U.host(y).reshape(B, H))
    c.sync()
    assert np.abs(np.stack(outs).astype(np.float32) - want.astype(np.float32)).max() < 6e-3
    plan.close()
    step.close()


@gpu
@pytest.mark.parametrize("B,T,E,Hh,rope,window", [(2, 9, 128, 2, 0.0, 0), (3, 64, 512, 8, 10000.0, 0), (2, 40, 128, 2, 10000.0, 16),
                                                  (2, 100, 128, 2, 10000.0, 0)])
def test_mha_full_sequence(env, B, T, E, Hh, rope, window):
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    rng = np.random.default_rng(B * 100 + T)
    x = h(rng.standard_normal((B, T, E)))
    ws = [PL.xavier_uniform(rng, (E, E), E, E) for _ in range(4)]
    want = O.mha(x, *ws, Hh, rope, 3, window)
    plan = pk.MhaPlan(c, B, T, E, Hh, rope_base=rope, window=window)
    dws = [U.dev(w) for w in ws]
    plan.set_weights(*dws)
    dy = torch.zeros(B * T * E, dtype=torch.float16, device="cuda")
    plan.forward(U.dev(x), dy, pos0=3)
    c.sync()
    got = U.host(dy).reshape(B, T, E)
    assert U.scaled_err(got, want) < 1e-2
    plan.close()


@gpu
def test_mha_streaming_ring_cache_equals_windowed_full_sequence(env):
    U = env
    import torch

    c = U.ctx()
    pk = U.pkg()
    B, E, Hh, window, steps = 2, 128, 2, 8, 21
    rng = np.random.default_rng(9)
    x = h(rng.standard_normal((B, steps, E)))
    ws = [PL.xavier_uniform(rng, (E, E), E, E) for _ in range(4)]
    want = O.mha(x, *ws, Hh, 10000.0, 0, window)  # sliding window of `window` steps
    plan = pk.MhaPlan(c, B, window, E, Hh, rope_base=10000.0, window=window)
    dws = [U.dev(w) for w in ws]
    plan.set_weights(*dws)
    outs = []
    for t in range(steps):
        y = torch.zeros(B * E, dtype=torch.float16, device="cuda")
        plan.step(U.dev(np.ascontiguousarray(x[:, t])), y, t)
        outs.append(U.host(y).reshape(B, E))
    c.sync()
    got = np.stack(outs, axis=1)
    assert U.scaled_err(got, want) < 1e-2
    # after a reset the cache is empty again
    plan.reset()
    y = torch.zeros(B * E, dtype=torch.float16, device="cuda")
    plan.step(U.dev(np.ascontiguousarray(x[:, 0])), y, 0)
    c.sync()
    assert U.scaled_err(U.host(y).reshape(B, E), want[:, 0]) < 1e-2
    plan.close()
