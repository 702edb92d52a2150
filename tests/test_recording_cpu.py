"""Reader for the reference's recording files (input_recorder.cpp:24-27,122-133; index scan main.cpp:41-92;
targets Train.cpp:70-76) on a synthetic file written byte by byte the way the recorder writes it.  Host code only:
runs without a GPU."""
import os
import struct

import numpy as np
import pytest

import __graft_entry__ as entry


@pytest.fixture(scope="module")
def pkg():
    return entry.build()


def write_recording(path, width, height, keys, mouse, frames, tail=b""):
    """The recorder's own write order: header once, then per frame keyStates (uint16), mouseDeltaX, mouseDeltaY
    (int32 each), the planar RGB frame."""
    with open(path, "wb") as f:
        f.write(struct.pack("<ii", width, height))
        for k, (dx, dy), fr in zip(keys, mouse, frames):
            f.write(struct.pack("<Hii", int(k), int(dx), int(dy)))
            f.write(np.ascontiguousarray(fr, np.uint8).tobytes())
        f.write(tail)


def test_read_index_and_targets(pkg, tmp_path):
    rng = np.random.default_rng(3)
    w, h, n = 24, 10, 7
    keys = rng.integers(0, 1 << 14, n).astype(np.uint16)
    mouse = rng.integers(-300, 300, (n, 2)).astype(np.int32)
    frames = rng.integers(0, 256, (n, 3, h, w), dtype=np.uint8)
    path = tmp_path / "training_data.bin"
    write_recording(path, w, h, keys, mouse, frames, tail=b"\x01" * (10 + 3 * w * h - 1))   # a partial record at the end is ignored
    assert struct.calcsize("<Hii") == 10
    rec = pkg.Recording(path)
    assert (rec.width, rec.height, rec.n_records) == (w, h, n)
    f, k, m = rec.read(0, n)
    assert np.array_equal(f, frames) and np.array_equal(k, keys) and np.array_equal(m, mouse)
    f, k, m = rec.read(5, 2)
    assert np.array_equal(f, frames[5:]) and np.array_equal(k, keys[5:]) and np.array_equal(m, mouse[5:])
    with pytest.raises(pkg.AigError):
        rec.read(6, 2)                                   # past the last whole record
    t = pkg.Recording.targets(keys, mouse)
    want = np.zeros((n, 16), np.float32)
    for i in range(n):
        for j in range(14):
            want[i, j] = float((int(keys[i]) >> j) & 1)   # Train.cpp:71-73
        want[i, 14] = np.float32(mouse[i, 0]) / np.float32(256.0)
        want[i, 15] = np.float32(mouse[i, 1]) / np.float32(256.0)
    assert np.array_equal(t, want)
    rec.close()


def test_open_errors(pkg, tmp_path):
    with pytest.raises(pkg.AigError, match="cannot open"):
        pkg.Recording(tmp_path / "missing.bin")
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"\x00\x00")
    with pytest.raises(pkg.AigError, match="header"):
        pkg.Recording(bad)
    empty = tmp_path / "empty.bin"
    empty.write_bytes(struct.pack("<ii", 16, 8))
    rec = pkg.Recording(empty)
    assert rec.n_records == 0
    rec.close()


def test_byte_normalisation_by_reciprocal_is_exact():
    """The first-layer kernel computes half(float(byte) * fl(1/255)) where the reference computes
    half(float(byte) / 255.0f) (CudaStuff.cu:150-153): the two agree for every byte value."""
    v = np.arange(256, dtype=np.float32)
    by_div = (v / np.float32(255.0)).astype(np.float16)
    recip = np.float32(1.0) / np.float32(255.0)
    assert recip.view(np.uint32) == 0x3B808081
    assert np.array_equal(by_div.view(np.uint16), (v * recip).astype(np.float16).view(np.uint16))
