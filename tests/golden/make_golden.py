"""Generates the golden fixtures in this folder by running the REFERENCE's own CUDA kernels
(compiled unmodified by `make -C oracle ref` into oracle/_ref/libref_kernels.so) on a GPU.

    python tests/golden/make_golden.py <output_dir>

Inputs are small seeded tensors; every fixture stores inputs and the reference kernel's
outputs, so the CPU tests can check the oracle against them without a GPU or the reference.
The reference implements R = 2 and R = 4 H-strip grids in fp32 NCHW only
(src/spatial.cc:75-134), so those are the cases recorded.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests import helpers as H  # noqa: E402


def ref_lib():
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_kernels.so"))
    return lib


def run_halo(lib, reduce, strips, p, W, h, Cc, N):
    """All ranks' kernels, one after another on one stream (the reference launches one kernel per rank)."""
    R = len(strips)
    d = [torch.from_numpy(s).cuda() for s in strips]
    u = C.c_uint32
    ptrs = [C.c_void_p(t.data_ptr()) for t in d]
    for r in range(R):
        if R == 2:
            st = lib.ref_halo_1x2(int(reduce), u(r), u(p), u(W), u(h), u(Cc), u(N), *ptrs, None)
        else:
            st = lib.ref_halo_1x4(int(reduce), u(r), u(p), u(W), u(h), u(Cc), u(N), *ptrs, None)
        assert st == 0, st
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in d]


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    lib = ref_lib()
    u = C.c_uint32
    fx = {}
    # --- halo exchange / reduce
    case = 0
    for R in (2, 4):
        for p, W, h, Cc, N in ((1, 5, 2, 3, 2), (3, 8, 6, 2, 1), (2, 17, 5, 1, 2)):
            full = H.uniform(1000 + case, (N, Cc, h * R, W))
            strips = H.split_strips(full, R, p)
            out = run_halo(lib, 0, [s.copy() for s in strips], p, W, h, Cc, N)
            g = [H.uniform(2000 + 10 * case + r, s.shape) for r, s in enumerate(strips)]
            red = run_halo(lib, 1, [x.copy() for x in g], p, W, h, Cc, N)
            fx[f"halo{case}_meta"] = np.array([R, p, W, h, Cc, N], np.int64)
            for r in range(R):
                fx[f"halo{case}_in{r}"] = strips[r]
                fx[f"halo{case}_exch{r}"] = out[r]
                fx[f"halo{case}_gin{r}"] = g[r]
                fx[f"halo{case}_red{r}"] = red[r]
            case += 1
    fx["halo_cases"] = np.array([case], np.int64)
    # --- slice copy / add
    src = H.uniform(3000, (2, 3, 7, 9))
    for add in (0, 1):
        dst = H.uniform(3001, (2, 3, 5, 11))
        d_src, d_dst = torch.from_numpy(src).cuda(), torch.from_numpy(dst).cuda()
        st = lib.ref_slice2d(add, u(4), u(3), u(9), u(7), u(11), u(5), u(3), u(2), C.c_void_p(d_src.data_ptr()), u(2), u(1),
                             C.c_void_p(d_dst.data_ptr()), u(5), u(2), None)
        assert st == 0
        torch.cuda.synchronize()
        fx[f"slice_src"] = src
        fx[f"slice_dst_in"] = dst
        fx[f"slice_out{add}"] = d_dst.cpu().numpy()
    # --- NLL loss
    B, Cc = 9, 7
    y = H.uniform(4000, (B, Cc), 0.01, 1.0)
    label = np.array([0, 6, 3, 1, 5, 2, 4, 6, 0], np.uint32)
    dloss = H.uniform(4001, (B,))
    dx0 = H.uniform(4002, (B, Cc))
    d_y, d_l, d_dl, d_dx = (torch.from_numpy(a).cuda() for a in (y, label.view(np.int32), dloss, dx0))
    d_loss = torch.empty(B, device="cuda")
    P = lambda t: C.c_void_p(t.data_ptr())
    assert lib.ref_softmax_nll_loss_fwd(u(Cc), u(B), P(d_y), P(d_l), P(d_loss), None) == 0
    assert lib.ref_softmax_nll_loss_bwd(u(Cc), u(B), P(d_y), P(d_l), P(d_dl), P(d_dx), None) == 0
    torch.cuda.synchronize()
    fx.update(nll_y=y, nll_label=label, nll_dloss=dloss, nll_dx_in=dx0, nll_loss=d_loss.cpu().numpy(),
              nll_dx_out=d_dx.cpu().numpy())
    # --- packed array arithmetic (rounding of the fused multiply-adds)
    n = 1031
    x, y0 = H.normal(5000, (n,), 3.0), H.normal(5001, (n,), 3.0)
    fx.update(arr_x=x, arr_y=y0, arr_a=np.float32(0.37), arr_b=np.float32(-1.21))
    for op, name in enumerate(["add", "add_scaled", "add_online", "scale", "scale_add"]):
        d_x, d_y2 = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
        assert lib.ref_array_op(op, u(n), C.c_float(0.37), C.c_float(-1.21), P(d_x), P(d_y2), None) == 0
        torch.cuda.synchronize()
        fx[f"arr_{name}"] = d_y2.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "reference_kernels.npz"), **fx)
    print("wrote", os.path.join(out_dir, "reference_kernels.npz"), len(fx), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
