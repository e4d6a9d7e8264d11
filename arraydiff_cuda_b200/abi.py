"""ctypes view of include/arraydiff_b200.h.  Field order and types mirror the header exactly."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libarraydiff_b200.so")

AD_MAX_PEERS = 8
AD_OK, AD_ERR_BAD_ARG, AD_ERR_UNSUPPORTED, AD_ERR_CUDA, AD_ERR_TIMEOUT, AD_ERR_ALIGN, AD_ERR_SCRATCH = 0, -1, -2, -3, -4, -5, -6
AD_ERR_LIMIT = -7
AD_F32, AD_BF16 = 0, 3
AD_NCHW, AD_NHWC = 0, 1
CONV_NONE, CONV_DIRECT_F32, CONV_TC_GENERAL, CONV_TC_ROW = 0, 1, 2, 3

vp, u32, i32, u64, i64, f32, sz = C.c_void_p, C.c_uint32, C.c_int32, C.c_uint64, C.c_int64, C.c_float, C.c_size_t


class HaloArgs(C.Structure):
    _fields_ = [
        ("dtype", i32), ("layout", i32),
        ("halo_pad", u32), ("base_width", u32), ("base_height", u32), ("num_channels", u32), ("batch_size", u32),
        ("num_ranks", u32), ("rank_first", u32), ("rank_count", u32),
        ("push", i32), ("reserved", u32),
        ("bufs", vp * AD_MAX_PEERS),
        ("signal_flags", vp * AD_MAX_PEERS),
        ("epoch", u64),
        ("block_counter", vp),
        ("epoch_base", vp),
    ]


class Halo2dArgs(C.Structure):
    _fields_ = [
        ("dtype", i32), ("layout", i32),
        ("halo_pad", u32), ("base_width", u32), ("base_height", u32), ("num_channels", u32), ("batch_size", u32),
        ("grid_w", u32), ("grid_h", u32), ("rank_first", u32), ("rank_count", u32),
        ("push", i32),
        ("bufs", vp * AD_MAX_PEERS),
        ("signal_flags", vp * AD_MAX_PEERS),
        ("epoch", u64),
        ("block_counter", vp),
        ("epoch_base", vp),
    ]


class Tensor4(C.Structure):
    _fields_ = [("base", vp), ("dtype", i32), ("N", u32), ("C", u32), ("H", u32), ("W", u32),
                ("sn", i64), ("sc", i64), ("sy", i64), ("sx", i64)]


class Conv2dArgs(C.Structure):
    _fields_ = [
        ("dtype", i32), ("layout", i32),
        ("N", u32), ("C", u32), ("H", u32), ("W", u32),
        ("K", u32), ("kh", u32), ("kw", u32),
        ("stride_h", u32), ("stride_w", u32), ("dil_h", u32), ("dil_w", u32), ("pad_h", u32), ("pad_w", u32),
        ("relu", i32), ("accumulate", i32),
        ("x", vp), ("w", vp), ("bias", vp), ("y", vp),
        ("y_pitch", i64), ("y_plane", i64),
        ("dx", vp), ("dw", vp), ("db", vp),
        ("scratch", vp), ("scratch_bytes", sz),
        ("out_row_begin", u32), ("out_row_count", u32),
        ("dx_col_begin", u32), ("dx_col_count", u32),
        ("dw_kcrs", i32), ("reserved_tail", i32),
    ]


class ConvProfileEntry(C.Structure):
    _fields_ = [("pass_", i32), ("kernel", i32), ("status", i32),
                ("N", u32), ("C", u32), ("H", u32), ("W", u32), ("K", u32), ("kh", u32), ("kw", u32),
                ("stride", u32), ("dil", u32), ("pad", u32), ("out_rows", u32), ("ms", f32)]


# name -> (restype, argtypes); every symbol the header declares.
SIGNATURES = {
    "ad_status_string": (C.c_char_p, [C.c_int]),
    "ad_launch_count": (u64, []),
    "ad_halo_exchange": (C.c_int, [C.POINTER(HaloArgs), vp]),
    "ad_halo_reduce": (C.c_int, [C.POINTER(HaloArgs), vp]),
    "ad_halo2d_exchange": (C.c_int, [C.POINTER(Halo2dArgs), vp]),
    "ad_halo2d_reduce": (C.c_int, [C.POINTER(Halo2dArgs), vp]),
    "ad_flag_wait": (C.c_int, [vp, u64, u64, vp, vp]),
    "ad_flag_signal": (C.c_int, [vp, u64, vp]),
    "ad_ipc_get_handle": (C.c_int, [vp, C.c_char_p]),
    "ad_ipc_open_handle": (C.c_int, [C.c_char_p, C.POINTER(vp)]),
    "ad_flag_wait_rel": (C.c_int, [vp, vp, u64, u64, vp, vp]),
    "ad_flag_signal_rel": (C.c_int, [vp, vp, u64, vp]),
    "ad_flag_advance": (C.c_int, [vp, u64, vp]),
    "ad_peer_sum": (C.c_int, [u32, vp, vp, sz, sz, vp]),
    "ad_ipc_close_handle": (C.c_int, [vp]),
    "ad_enable_peer_access": (C.c_int, [C.c_int, C.c_int]),
    "ad_device_malloc": (C.c_int, [sz, C.POINTER(vp)]),
    "ad_device_free": (C.c_int, [vp]),
    "ad_slice2d_copy_hw_nchw_packed": (C.c_int, [i32] + [u32] * 8 + [vp, u32, u32, vp, u32, u32, vp]),
    "ad_slice2d_add_hw_nchw_packed": (C.c_int, [i32] + [u32] * 8 + [vp, u32, u32, vp, u32, u32, vp]),
    "ad_array_set_constant": (C.c_int, [sz, f32, vp, vp]),
    "ad_array_add": (C.c_int, [sz, vp, vp, vp]),
    "ad_array_add_scaled": (C.c_int, [sz, f32, f32, vp, vp, vp]),
    "ad_array_add_online": (C.c_int, [sz, f32, vp, vp, vp]),
    "ad_array_scale": (C.c_int, [sz, f32, vp, vp, vp]),
    "ad_array_scale_add": (C.c_int, [sz, f32, vp, vp, vp]),
    "ad_fill_zero": (C.c_int, [vp, sz, vp]),
    "ad_sgd_step": (C.c_int, [sz, vp, vp, vp, f32, f32, f32, f32, i32, vp, vp]),
    "ad_sgd_step_guarded": (C.c_int, [sz, vp, vp, vp, f32, f32, f32, f32, i32, vp, vp, vp]),
    "ad_softmax_nll_loss_fwd": (C.c_int, [u32, u32, vp, vp, vp, vp]),
    "ad_softmax_nll_loss_bwd": (C.c_int, [u32, u32, vp, vp, vp, vp, vp]),
    "ad_softmax_ce_pixel_fwd": (C.c_int, [i32, i32, u32, u32, u32, vp, vp, vp, vp, vp]),
    "ad_softmax_ce_pixel_bwd": (C.c_int, [i32, i32, u32, u32, u32, vp, vp, vp, vp, i32, vp]),
    "ad_bn_scratch_bytes": (sz, [u32]),
    "ad_bn_fwd_train": (C.c_int, [C.POINTER(Tensor4), C.POINTER(Tensor4), vp, vp, vp, vp, vp, f32, i32, vp, sz, vp]),
    "ad_bn_fwd_train_noalloc": (C.c_int, [C.POINTER(Tensor4), C.POINTER(Tensor4), vp, vp, vp, vp, vp, f32, i32, vp]),
    "ad_bn_fwd_inference": (C.c_int, [C.POINTER(Tensor4), C.POINTER(Tensor4), vp, vp, vp, vp, vp, f32, i32, vp]),
    "ad_bn_bwd": (C.c_int, [C.POINTER(Tensor4)] * 3 + [vp, vp, vp, vp, vp, vp, i32, i32, vp, sz, vp]),
    "ad_bn_partial_stats": (C.c_int, [C.POINTER(Tensor4), vp, vp, sz, vp]),
    "ad_bn_finalize_apply": (C.c_int, [C.POINTER(Tensor4), C.POINTER(Tensor4), vp, C.c_double, vp, vp, vp, vp, vp, f32, i32, vp]),
    "ad_maxpool2d_fwd": (C.c_int, [C.POINTER(Tensor4), C.POINTER(Tensor4), u32, u32, u32, u32, vp]),
    "ad_maxpool2d_bwd": (C.c_int, [C.POINTER(Tensor4)] * 3 + [u32, u32, u32, u32, i32, vp]),
    "ad_relu_fwd": (C.c_int, [C.POINTER(Tensor4), C.POINTER(Tensor4), vp]),
    "ad_relu_bwd": (C.c_int, [C.POINTER(Tensor4)] * 3 + [i32, vp]),
    "ad_add": (C.c_int, [C.POINTER(Tensor4)] * 3 + [vp]),
    "ad_convert": (C.c_int, [C.POINTER(Tensor4), C.POINTER(Tensor4), i32, vp]),
    "ad_avgpool2d_fwd": (C.c_int, [C.POINTER(Tensor4), C.POINTER(Tensor4), u32, u32, u32, u32, vp]),
    "ad_avgpool2d_bwd": (C.c_int, [C.POINTER(Tensor4), C.POINTER(Tensor4), u32, u32, u32, u32, i32, vp]),
    "ad_linear_fwd": (C.c_int, [i32, u32, u32, u32, vp, vp, vp, vp, vp]),
    "ad_linear_bwd": (C.c_int, [i32, u32, u32, u32, vp, vp, vp, vp, vp, vp, i32, i32, vp]),
    "ad_upsample_bilinear_fwd": (C.c_int, [C.POINTER(Tensor4), C.POINTER(Tensor4), u32, i32, u32, u32, vp]),
    "ad_upsample_bilinear_bwd": (C.c_int, [C.POINTER(Tensor4), C.POINTER(Tensor4), u32, i32, u32, u32, i32, vp]),
    "ad_im2col": (C.c_int, [C.POINTER(Tensor4)] + [u32] * 8 + [vp, u32, vp]),
    "ad_conv2d_scratch_bytes": (sz, [C.POINTER(Conv2dArgs), i32]),
    "ad_conv2d_fprop": (C.c_int, [C.POINTER(Conv2dArgs), vp]),
    "ad_conv2d_dgrad": (C.c_int, [C.POINTER(Conv2dArgs), vp]),
    "ad_conv2d_wgrad": (C.c_int, [C.POINTER(Conv2dArgs), vp]),
    "ad_conv2d_last_kernel": (i32, []),
    "ad_conv2d_profile": (C.c_int, [i32]),
    "ad_conv2d_profile_read": (sz, [C.POINTER(ConvProfileEntry), sz]),
}


class AdError(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        super().__init__(f"{what}: {status}")


_lib = None


def load(path=None):
    """Load the C-ABI library.  Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    path = path or LIB_PATH
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing -- build it with `python -m arraydiff_cuda_b200.build`; "
                          "there is no CPU or PyTorch fallback for these kernels")
    lib_ = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib_, name)  # AttributeError if a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib_
    return lib_


def lib():
    return load()


def conv_profile_read():
    """Records of the convolution calls made since ad_conv2d_profile(1), as ConvProfileEntry objects."""
    L = load()
    n = L.ad_conv2d_profile_read(None, 0)
    buf = (ConvProfileEntry * max(1, n))()
    n = L.ad_conv2d_profile_read(buf, n)
    return [buf[i] for i in range(n)]


def check(status, what="arraydiff_b200 call"):
    if status != AD_OK:
        msg = lib().ad_status_string(status).decode()
        raise AdError(status, f"{what} failed ({msg})")
