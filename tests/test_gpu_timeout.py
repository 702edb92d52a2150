"""The time-out path shared by every kernel of the library, exercised without faulting anything: a kernel
whose only work is a bounded wait on a barrier nobody arrives at gives up after a short limit, records an
error code and returns; the host sees AIG_ERR_TIMEOUT once and the context keeps working."""
import numpy as np
import pytest

from oracle import oracle as O

gpu = pytest.mark.gpu
AIG_ERR_INVALID, AIG_ERR_TIMEOUT = -1, -3


@pytest.fixture(scope="module")
def env():
    import torch
    from tests import gpu_util as U

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return U


@gpu
def test_expired_wait_reports_timeout_and_the_context_stays_usable(env):
    U = env
    import torch

    pk = U.pkg()
    lib = pk.lib()
    torch.cuda.set_device(0)
    c = pk.Context(0, use_torch_stream=False)   # a context of its own: the shared one never sees the error
    try:
        assert lib.aig_selftest_expiring_wait(c.handle, 0) == AIG_ERR_INVALID
        assert lib.aig_selftest_expiring_wait(c.handle, 10 ** 10) == AIG_ERR_INVALID   # limits stay short by design
        assert lib.aig_ctx_sync(c.handle) == 0
        assert lib.aig_selftest_expiring_wait(c.handle, 2_000_000) == 0                # about 1 ms of SM clocks
        rc = lib.aig_ctx_sync(c.handle)
        assert rc == AIG_ERR_TIMEOUT
        assert b"901" in lib.aig_last_error(c.handle)
        assert lib.aig_ctx_sync(c.handle) == 0, "the error word must clear once it has been reported"
        # the same context still computes
        x = (np.random.default_rng(5).standard_normal(4096) * 3).astype(np.float16)
        dx = torch.from_numpy(x).cuda()
        torch.cuda.synchronize()
        assert lib.aig_swish_forward(c.handle, pk.ptr(dx), x.size) == 0
        assert lib.aig_ctx_sync(c.handle) == 0
        U.assert_close16(U.host(dx), O.swish(x), max_ulp=1, what="swish after a timeout")
        # and a second expiry is reported again
        assert lib.aig_selftest_expiring_wait(c.handle, 1_000_000) == 0
        assert lib.aig_ctx_sync(c.handle) == AIG_ERR_TIMEOUT
        assert lib.aig_ctx_sync(c.handle) == 0
    finally:
        c.close()


@gpu
def test_streaming_step_keeps_working_after_a_reported_timeout(env):
    """The one-kernel streaming step keeps its grid-barrier state per launch, so an error reported between two
    steps (here: from the self-test kernel on the same context) does not disturb the steps that follow."""
    U = env
    from oracle import pipelines as PL

    pk = U.pkg()
    lib = pk.lib()
    from ai_gamer_b200 import runners as R

    c = U.ctx()
    B, T, d, heads = 1, 6, 128, 2
    p = PL.make_seq_params(31, d=d, hid=d, layers=2, heads=heads)
    emb = PL.make_embeddings(31, T, B, d)
    _, _, _, want = PL.seq_forward(p, emb, rope_base=10000.0, window=0)
    head = R.SeqHead(c, B, T, in_c=d, hidden=d, layers=2, heads=heads, rope_base=10000.0, window=0)
    head.load_bytes(PL.serialize_seq_params(p))
    outs = []
    for t in range(T):
        if t == 3:
            assert lib.aig_selftest_expiring_wait(c.handle, 1_000_000) == 0
            assert lib.aig_ctx_sync(c.handle) == AIG_ERR_TIMEOUT
        head.step(U.dev(np.ascontiguousarray(emb[t])))
        outs.append(U.host(head.outputs_f32(step=True)))
    head.close()
    got = np.stack(outs, axis=1)
    assert U.rel_err(got, want.astype(np.float32), 0.05).max() < 2e-2
