"""Helpers shared by the GPU parity tests: package/context loading, host<->device staging and
fp16 comparison utilities.  Everything the tests run on the GPU goes through the C ABI."""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libaig_refcuda.so")

_state = {}


def pkg():
    return entry.load_package()


def ctx():
    """One shared context on cuda:0 bound to torch's current stream."""
    if "ctx" not in _state:
        import torch

        torch.cuda.set_device(0)
        _state["ctx"] = pkg().Context(0)
    return _state["ctx"]


def dev(a):
    """Host array -> device tensor, complete on return.  The copy runs on torch's stream and the library's context
    has a stream of its own (non-blocking), so the copy is waited for here: a copy from pageable memory may return
    while its last chunk is still on the way."""
    import torch

    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    torch.cuda.synchronize()
    return t


def host(t):
    return t.detach().cpu().numpy()


def nhwc(x):
    """NCHW / NCDHW numpy -> channels-last contiguous."""
    return np.ascontiguousarray(np.moveaxis(x, 1, -1))


def nchw(x):
    return np.ascontiguousarray(np.moveaxis(x, -1, 1))


def ulp16_diff(a, b):
    """Distance in fp16 units-in-the-last-place between two float16 arrays (finite values)."""
    def key(x):
        u = np.asarray(x, np.float16).view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)

    return np.abs(key(a) - key(b))


def assert_close16(got, want, max_ulp=1, frac_exact=None, what="", atol=0.0):
    """Every element within max_ulp fp16 ulps of the oracle, or within atol in absolute terms (results
    formed by cancellation sit near zero, where an fp16 ulp is far below the accumulation error)."""
    d = ulp16_diff(got, want)
    if atol > 0:
        ok = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64)) <= atol
        d = np.where(ok, np.minimum(d, max_ulp), d)
    assert d.max() <= max_ulp, "%s: max fp16 ulp distance %d > %d (%d of %d differ)" % (
        what, d.max(), max_ulp, (d > 0).sum(), d.size)
    if frac_exact is not None:
        assert (d == 0).mean() >= frac_exact, "%s: only %.4f bit-exact" % (what, (d == 0).mean())


def assert_two_step(got, want, bias, what="", frac_exact=0.99):
    """Check of the reference's conv/FC rounding sequence y = half(half(acc) + bias): fp32 accumulation
    on the tensor cores against the oracle's double accumulation may move half(acc) by one fp16 ulp at
    the magnitude of acc = y - bias, which the bias add can carry into a smaller binade of y, and the
    second rounding can add up to one ulp of y between the two results.  So the bound is
    ulp(acc) + ulp(y) <= 2 ulp of max(|y|, |y - bias|); almost all elements must be bit-exact."""
    got = np.asarray(got, np.float64)
    want64 = np.asarray(want, np.float64)
    scale = np.maximum(np.abs(want64), np.abs(want64 - np.asarray(bias, np.float64)))
    ulp = np.maximum(2.0 ** (np.floor(np.log2(np.maximum(scale, 2.0 ** -14))) - 10), 2.0 ** -24)
    bad = np.abs(got - want64) > ulp * 2.0001
    assert not bad.any(), "%s: %d of %d beyond ulp(acc) + ulp(y)" % (what, bad.sum(), bad.size)
    exact = (got == want64).mean()
    assert exact >= frac_exact, "%s: only %.4f bit-exact" % (what, exact)


def rel_err(got, want, floor=1e-2):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return np.abs(got - want) / np.maximum(np.abs(want), floor)


def scaled_err(got, want):
    """max |got - want| relative to max(|want|, rms(want)): element-wise relative error with a floor at
    the tensor's own scale, so that near-zero activations do not dominate."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    rms = float(np.sqrt(np.mean(want * want))) + 1e-12
    return float((np.abs(got - want) / np.maximum(np.abs(want), rms)).max())


def ref_cuda():
    """The reference's own CudaStuff.cu built as a shared library (oracle/_ref), or None."""
    if "ref" not in _state:
        lib = None
        if os.path.exists(REF_LIB):
            try:
                lib = ctypes.CDLL(REF_LIB)
                lib.InitCUDA()
            except OSError:
                lib = None
        _state["ref"] = lib
    return _state["ref"]


P = ctypes.c_void_p


def p(t):
    return P(t.data_ptr())
