"""The multi-process plumbing of the frame path on CPU: two gloo ranks share nothing but the checkpoint
bytes (one broadcast) and the timing maximum; frames are sharded as independent units."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _mod(name):
    """ai-gamer_b200/<name>.py as a module (the package directory is not a Python identifier)."""
    import importlib

    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry

    entry.load_package()
    return importlib.import_module("ai_gamer_b200." + name)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    pkg = _mod("sharding")
    synth = _mod("synth")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # rank 0 builds the checkpoint; both must end up with the same bytes
        params = synth.make_cnn_params(3, widths=(32, 64))
        blob = synth.serialize_cnn_checkpoint(params, 64, 32) if rank == 0 else None
        nbytes = len(synth.serialize_cnn_checkpoint(params, 64, 32))
        got = pkg.broadcast_bytes(blob, nbytes)
        # frames: 11 units over 2 ranks
        lo, hi = pkg.shard_range(11, world, rank)
        frames = synth.make_frames(9, 11, 8, 16)[lo:hi]
        # timing rule: max over ranks
        tmax = pkg.max_over_ranks([1.0 + rank, 5.0 - rank])
        np.savez(os.path.join(out_dir, "rank%d.npz" % rank), blob=np.frombuffer(got, np.uint8), lo=lo, hi=hi, checksum=int(frames.sum()),
                 tmax=np.array(tmax))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_share_checkpoint_and_split_frames(tmp_path):
    synth = _mod("synth")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % i)) for i in range(world)]
    want = synth.serialize_cnn_checkpoint(synth.make_cnn_params(3, widths=(32, 64)), 64, 32)
    assert r[0]["blob"].tobytes() == want and r[1]["blob"].tobytes() == want
    assert (int(r[0]["lo"]), int(r[0]["hi"]), int(r[1]["lo"]), int(r[1]["hi"])) == (0, 6, 6, 11)
    all_frames = synth.make_frames(9, 11, 8, 16)
    assert int(r[0]["checksum"]) + int(r[1]["checksum"]) == int(all_frames.sum())   # every frame on exactly one rank
    assert list(r[0]["tmax"]) == [2.0, 5.0] and list(r[1]["tmax"]) == [2.0, 5.0]


def test_shard_range_partitions_units():
    sh = _mod("sharding")
    for n in (0, 1, 7, 256, 1000):
        for world in (1, 2, 3, 8):
            spans = [sh.shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sh.shard_range(4, 2, 2)
