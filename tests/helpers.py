"""Shared test plumbing: seeded inputs, torch <-> C-ABI glue, error metrics."""
import ctypes as C

import numpy as np

from arraydiff_cuda_b200 import abi


def rng(seed):
    return np.random.default_rng(seed)


def uniform(seed, shape, lo=-1.0, hi=1.0):
    return rng(seed).uniform(lo, hi, size=shape).astype(np.float32)


def normal(seed, shape, std=1.0):
    return (rng(seed).standard_normal(size=shape) * std).astype(np.float32)


def max_rel(a, b):
    """max|a-b| / max|b| : the error metric of the conv / softmax tolerances."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


def split_strips(full, R, p):
    """Zero-padded strips of an NCHW tensor: interior rows of rank r, halos zero."""
    N, Cc, H, W = full.shape
    h = H // R
    out = []
    for r in range(R):
        s = np.zeros((N, Cc, h + 2 * p, W + 2 * p), full.dtype)
        s[:, :, p:p + h, p:p + W] = full[:, :, r * h:(r + 1) * h, :]
        out.append(s)
    return out


def expected_strips_after_exchange(full, R, p):
    """Window of the zero-padded full tensor that each strip must equal after the exchange."""
    N, Cc, H, W = full.shape
    h = H // R
    padded = np.zeros((N, Cc, H + 2 * p, W + 2 * p), full.dtype)
    padded[:, :, p:p + H, p:p + W] = full
    return [np.ascontiguousarray(padded[:, :, r * h:r * h + h + 2 * p, :]) for r in range(R)]


# ---------------------------------------------------------------- GPU glue (torch is plumbing only)
def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def dev_bf16(a_f32):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a_f32)).cuda().to(torch.bfloat16)


def host(t):
    import torch
    if t.dtype == torch.bfloat16:
        return t.float().cpu().numpy()
    return t.cpu().numpy()


def bits_bf16(t):
    """bf16 torch tensor -> uint16 numpy bit patterns."""
    import torch
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def from_bits_bf16(u16):
    import torch
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).cuda().view(torch.bfloat16)


def stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def sync():
    import torch
    torch.cuda.synchronize()


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def ad_dtype(t):
    import torch
    return abi.AD_F32 if t.dtype == torch.float32 else abi.AD_BF16


def view_nchw(t, interior=None):
    """Tensor4 over a torch tensor laid out [N][C][H][W]; interior=(p, h, W) selects the
    interior of a halo-padded buffer."""
    N, Cc, H, W = t.shape
    sn, sc, sy, sx = t.stride()
    base = t.data_ptr()
    if interior:
        p, h, w = interior
        base += (p * sy + p * sx) * t.element_size()
        H, W = h, w
    return abi.Tensor4(base, ad_dtype(t), N, Cc, H, W, sn, sc, sy, sx)


def view_nhwc(t, interior=None):
    """Tensor4 over a torch tensor laid out [N][H][W][C]."""
    N, H, W, Cc = t.shape
    sn, sy, sx, sc = t.stride()
    base = t.data_ptr()
    if interior:
        p, h, w = interior
        base += (p * sy + p * sx) * t.element_size()
        H, W = h, w
    return abi.Tensor4(base, ad_dtype(t), N, Cc, H, W, sn, sc, sy, sx)


def halo_args(bufs, dtype, layout, p, W, h, Cc, N, rank_first=0, rank_count=None, push=1):
    a = abi.HaloArgs()
    a.dtype, a.layout = dtype, layout
    a.halo_pad, a.base_width, a.base_height, a.num_channels, a.batch_size = p, W, h, Cc, N
    a.num_ranks = len(bufs)
    a.rank_first = rank_first
    a.rank_count = len(bufs) if rank_count is None else rank_count
    a.push = push
    for i, b in enumerate(bufs):
        a.bufs[i] = b.data_ptr() if hasattr(b, "data_ptr") else b
    return a
