"""CPU-side checks of the boundary: the CUDA library builds, loads, and exports every symbol the
public headers declare (no compute calls are made -- there is no GPU here), error paths that need no
device behave, and the checkpoint writer produces the byte layout the loader expects."""
import ctypes
import os
import re

import numpy as np
import pytest

import __graft_entry__ as entry

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def pkg():
    return entry.build()


def declared_symbols():
    names = []
    for hdr in ("aig_b200.h", "aig_host.h"):
        text = open(os.path.join(ROOT, "include", hdr)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(aig_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


COMPAT_NAMES = ["InitCUDA", "ConvertAndNormalize", "UnConvertAndUnNormalize", "ConvertFloatToHalf", "ConvertHalfToFloat", "HeInit",
                "LeakyReluForward", "SwishForward", "SigmoidForward", "LayerNormForward", "SpatialAttentionForward", "ARGBtoRGB",
                "ARGBtoRGBplanar", "aig_compat_context", "aig_compat_last_status", "aig_compat_set_attention_group"]


def test_library_exports_the_reference_launcher_names(pkg):
    """include/aig_compat.h: the forward-path launchers of the reference (common.h:104-139, NvDisplayCap.h:68-69)
    exist under their own names, and the header declares each of them."""
    lib = ctypes.CDLL(pkg.LIB_PATH)
    text = open(os.path.join(ROOT, "include", "aig_compat.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for n in COMPAT_NAMES:
        assert re.search(r"\b%s\s*\(" % n, text), n + " not declared"
        assert hasattr(lib, n), n + " not exported"


def test_library_exports_every_declared_symbol(pkg):
    lib = ctypes.CDLL(pkg.LIB_PATH)
    names = declared_symbols()
    assert len(names) > 60
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, "declared in include/*.h but not exported: %s" % missing


def exported_symbols(path):
    """Dynamic, defined function symbols of a shared library (`nm -D --defined-only`)."""
    import subprocess

    out = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True, check=True).stdout
    return sorted({ln.split()[2] for ln in out.splitlines() if len(ln.split()) == 3 and ln.split()[1] in "TW"})


def test_every_exported_entry_point_is_declared_in_a_header(pkg):
    """The reverse direction: nothing with the library's prefix, and none of the reference's launcher names, is
    exported without a declaration in include/*.h (no undocumented back doors, no debugging hooks)."""
    declared = set(declared_symbols())
    text = open(os.path.join(ROOT, "include", "aig_compat.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared |= set(re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\(", text))
    exported = [n for n in exported_symbols(pkg.LIB_PATH) if n.startswith("aig_") or n in COMPAT_NAMES]
    assert len(exported) > 100
    undeclared = [n for n in exported if n not in declared]
    assert not undeclared, "exported but declared in no header: %s" % undeclared


def test_python_binding_declares_every_symbol(pkg):
    missing = [n for n in declared_symbols() if n not in pkg.SIGNATURES]
    assert not missing, "no ctypes signature for: %s" % missing


def test_no_device_is_an_error_not_a_fallback(pkg):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(pkg.AigError):
        pkg.Context(0, use_torch_stream=False)


def test_host_side_actions(pkg):
    p = np.array([[0.6] * 14 + [0.5, -0.25]], np.float32)
    out = np.zeros((1, 16), np.int32)
    rc = pkg.lib().aig_actions_from_outputs(pkg.ptr(p), pkg.ptr(out), 1, 16, 14)
    assert rc == 0
    assert out[0].tolist() == [1] * 14 + [128, -64]
    assert pkg.lib().aig_actions_from_outputs(None, pkg.ptr(out), 1, 16, 14) == -1


def test_checkpoint_size_matches_writer(pkg):
    from ai_gamer_b200 import synth as SY

    widths = (32, 64, 128, 256, 256)
    w = (ctypes.c_int * 8)(*widths)
    cfg = pkg.CnnConfig(4, 144, 256, 4, w, 5, 18, 16, pkg.ACT_SWISH, 0.01)
    blob = SY.serialize_cnn_checkpoint(SY.make_cnn_params(0, widths=widths), 256, 144)
    assert pkg.lib().aig_cnn_checkpoint_bytes(ctypes.byref(cfg)) == len(blob)
    assert np.frombuffer(blob[:8], np.int32).tolist() == [256, 144]  # NN.cpp:118-119: width then height


def test_process_output_event_list(pkg):
    """Infer::ProcessOutput (Infer.cpp:8-57) as a portable event list: 11 key events, 3 mouse-button events, one
    relative move when it is non-zero, in the reference's order; the callback form delivers the same events."""
    import ctypes

    class Event(ctypes.Structure):
        _fields_ = [(n, ctypes.c_int) for n in ("type", "code", "down", "dx", "dy")]

    lib = pkg.lib()
    key_map = (ctypes.c_ubyte * 14)(*range(30, 44))
    p = np.array([0.9, 0.1, 0.5, 0.51, 0, 1, 0, 0, 0, 0.7, 0.2, 0.6, 0.4, 0.99, 0.25, -0.031], np.float32)
    ev = (Event * 16)()
    n = lib.aig_process_output(pkg.ptr(p), key_map, ev, 16)
    assert n == 15
    keys = [(e.type, e.code, e.down) for e in ev[:11]]
    assert keys == [(0, 30 + i, int(p[i] > 0.5)) for i in range(11)]          # p == 0.5 is a release (Infer.cpp:15)
    assert [(e.type, e.code, e.down) for e in ev[11:14]] == [(1, 0, 1), (1, 1, 0), (1, 2, 1)]
    assert (ev[14].type, ev[14].dx, ev[14].dy) == (2, 64, -7)                  # (int)(p*256.0f): truncation toward zero
    p[14:] = [0.003, -0.003]                                                   # both truncate to zero: no move event
    assert lib.aig_process_output(pkg.ptr(p), key_map, ev, 16) == 14
    assert lib.aig_process_output(pkg.ptr(p), key_map, ev, 3) == 14            # count returned even when capacity is short
    got = []
    SINK = ctypes.CFUNCTYPE(None, ctypes.POINTER(Event), ctypes.c_void_p)
    sink = SINK(lambda e, user: got.append((e.contents.type, e.contents.code, e.contents.down)))
    assert lib.aig_process_output_to(pkg.ptr(p), key_map, sink, None) == 14
    assert got[:11] == keys and len(got) == 14
    assert lib.aig_process_output(None, key_map, ev, 16) == -1
