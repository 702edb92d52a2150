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
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


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


def assert_close16(got, want, max_ulp=1, frac_exact=None, what=""):
    d = ulp16_diff(got, want)
    assert d.max() <= max_ulp, "%s: max fp16 ulp distance %d > %d (%d of %d differ)" % (
        what, d.max(), max_ulp, (d > 0).sum(), d.size)
    if frac_exact is not None:
        assert (d == 0).mean() >= frac_exact, "%s: only %.4f bit-exact" % (what, (d == 0).mean())


def rel_err(got, want, floor=1e-2):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return np.abs(got - want) / np.maximum(np.abs(want), floor)


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
