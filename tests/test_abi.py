"""The C-ABI library loads and exports every symbol that include/arraydiff_b200.h declares."""
import os
import re

from arraydiff_cuda_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "arraydiff_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ad_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_bound_and_exported():
    syms = declared_symbols()
    assert len(syms) >= 35
    lib = abi.load()
    missing_binding = [s for s in syms if s not in abi.SIGNATURES]
    assert not missing_binding, missing_binding
    for s in syms:
        assert hasattr(lib, s), s
    extra = [s for s in abi.SIGNATURES if s not in syms]
    assert not extra, extra


def test_status_strings():
    lib = abi.load()
    assert lib.ad_status_string(0) == b"ok"
    for code in range(-6, 0):
        assert lib.ad_status_string(code) not in (b"ok", b"unknown status")


def test_struct_sizes_match_header_layout():
    import ctypes as C
    # 12 x 4 bytes, 8 + 8 pointers, u64, pointer
    assert C.sizeof(abi.HaloArgs) == 48 + 64 + 64 + 8 + 8 + 8
    assert C.sizeof(abi.Tensor4) == 8 + 4 + 16 + 4 + 32
    assert C.sizeof(abi.Conv2dArgs) == 17 * 4 + 4 + 4 * 8 + 16 + 3 * 8 + 16 + 8 + 8 + 8


def test_missing_library_fails_loudly(tmp_path):
    import pytest
    with pytest.raises(ImportError):
        abi.load(str(tmp_path / "nope.so"))


def test_ctypes_layout_matches_c_compiler(tmp_path):
    """Compile the header with gcc and compare sizeof / offsetof with the ctypes mirror."""
    import ctypes as C
    import subprocess
    src = tmp_path / "layout.c"
    exe = tmp_path / "layout"
    fields = {
        "ad_halo_args": (abi.HaloArgs, ["dtype", "bufs", "signal_flags", "epoch", "block_counter", "epoch_base"]),
        "ad_tensor4": (abi.Tensor4, ["base", "dtype", "N", "sn", "sx"]),
        "ad_conv2d_args": (abi.Conv2dArgs, ["K", "relu", "x", "y_pitch", "dx", "scratch", "scratch_bytes", "out_row_begin", "out_row_count", "dx_col_begin", "dx_col_count", "dw_kcrs"]),
    }
    body = ['#include <stdio.h>', '#include <stddef.h>', '#include "arraydiff_b200.h"', "int main(void){"]
    for cname, (_, fl) in fields.items():
        body.append(f'printf("{cname} %zu\\n", sizeof({cname}));')
        for f in fl:
            body.append(f'printf("{cname}.{f} %zu\\n", offsetof({cname}, {f}));')
    body.append("return 0;}")
    src.write_text("\n".join(body))
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    out = dict(line.split() for line in subprocess.check_output([str(exe)], text=True).splitlines())
    for cname, (ct, fl) in fields.items():
        assert int(out[cname]) == C.sizeof(ct)
        for f in fl:
            assert int(out[f"{cname}.{f}"]) == getattr(ct, f).offset, (cname, f)
