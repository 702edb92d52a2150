"""Generates tests/golden/reference_kernels.npz: seeded inputs and the outputs of the REFERENCE's own
CUDA kernels (CudaStuff.cu, compiled by oracle/Makefile into oracle/_ref/libaig_refcuda.so) for the
operators of the forward path that the reference implements itself.  Needs a CUDA device; run it from
the repository root:

    python tests/golden/make_reference_golden.py [output.npz]

The CPU test suite checks the oracle against this file, so the oracle stays pinned to what the
reference computes even where no GPU is present."""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main(out_path):
    import torch

    ref = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libaig_refcuda.so"))
    ref.InitCUDA()
    rng = np.random.default_rng(20240607)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    host = lambda t: t.cpu().numpy()
    out = {}

    # ARGBtoRGBplanar + ConvertAndNormalize (CudaStuff.cu:63-74,150-157); every byte value appears
    n = 4099
    bgra = rng.integers(0, 256, 4 * n, dtype=np.uint8)
    bgra[:1024] = np.repeat(np.arange(256, dtype=np.uint8), 4)
    d_src = dev(bgra)
    d_planar = torch.zeros(3 * n, dtype=torch.uint8, device="cuda")
    d_half = torch.zeros(3 * n, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    ref.ARGBtoRGBplanar(P(d_src), P(d_planar), ctypes.c_int(n))
    ref.ConvertAndNormalize(P(d_half), P(d_planar), ctypes.c_size_t(3 * n))
    torch.cuda.synchronize()
    out.update(pre_bgra=bgra, pre_planar=host(d_planar), pre_half=host(d_half).view(np.uint16))

    # activations (CudaStuff.cu:400-442)
    m = 8195
    x = np.concatenate([rng.standard_normal(m - 4) * 4, [0.0, -0.0, 65504.0, -65504.0]]).astype(np.float32).astype(np.float16)
    out["act_x"] = x.view(np.uint16)
    for name, call in (("swish", lambda d: ref.SwishForward(P(d), ctypes.c_int(m))),
                       ("leaky", lambda d: ref.LeakyReluForward(P(d), ctypes.c_int(m), ctypes.c_float(0.01))),
                       ("sigmoid", lambda d: ref.SigmoidForward(P(d), ctypes.c_int(16), ctypes.c_int(14), ctypes.c_int(m)))):
        d = dev(x)
        torch.cuda.synchronize()
        call(d)
        torch.cuda.synchronize()
        out["act_" + name] = host(d).view(np.uint16)

    # SpatialAttentionForward, scalar branch (CudaStuff.cu:673-746)
    B, inC, attC, H, W = 4, 32, 9, 4, 8
    Pn = B * H * W
    sx = (rng.standard_normal(Pn * inC) * 0.5).astype(np.float16)
    ws = [(rng.standard_normal(attC * inC) / np.sqrt(inC)).astype(np.float16) for _ in range(3)]
    dx, dw = dev(sx), [dev(w) for w in ws]
    rb = [torch.zeros(Pn * attC, dtype=torch.float16, device="cuda") for _ in range(3)]
    rs = torch.zeros(Pn, dtype=torch.float16, device="cuda")
    ro = torch.zeros(Pn * attC, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    ref.SpatialAttentionForward(P(dx), *[P(w) for w in dw], *[P(b) for b in rb], P(rs), P(ro), *[ctypes.c_int(v) for v in (B, inC, attC, H, W)])
    torch.cuda.synchronize()
    out.update(sa_dims=np.array([B, inC, attC, H, W], np.int32), sa_x=sx.view(np.uint16), sa_wk=ws[0].view(np.uint16),
               sa_wq=ws[1].view(np.uint16), sa_wv=ws[2].view(np.uint16), sa_key=host(rb[0]).view(np.uint16),
               sa_query=host(rb[1]).view(np.uint16), sa_value=host(rb[2]).view(np.uint16), sa_scores=host(rs).view(np.uint16),
               sa_out=host(ro).view(np.uint16))

    # LayerNorm kernels with one block per channel (CudaStuff.cu:457-515)
    N, C, HW = 3, 70, 64
    lx = (rng.standard_normal((N, C, HW)) * 2 + 0.3).astype(np.float16)
    g = rng.uniform(0.5, 1.5, C).astype(np.float32)
    b = rng.uniform(-1, 1, C).astype(np.float32)
    dlx, dg, db = dev(lx), dev(g), dev(b)
    ry = torch.zeros_like(dlx)
    rm = torch.zeros(C, dtype=torch.float32, device="cuda")
    rv = torch.zeros(C, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    rc = ref.ref_layernorm_forward_fullgrid(P(ry), P(dlx), P(dg), P(db), P(rm), P(rv), ctypes.c_int(N), ctypes.c_int(C), ctypes.c_int(HW))
    torch.cuda.synchronize()
    assert rc == 0
    out.update(ln_dims=np.array([N, C, HW], np.int32), ln_x=lx.view(np.uint16), ln_gamma=g, ln_beta=b, ln_y=host(ry).view(np.uint16),
               ln_mean=host(rm), ln_var=host(rv))
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_kernels.npz"))
