"""The C++ host layer's C entry points (host/src/capi.cc) load without a GPU and every symbol that
arraydiff_cuda_b200/hostlib.py binds is exported; no compute call is made here."""
import re
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_host_library_loads_and_exports_every_bound_symbol():
    from arraydiff_cuda_b200 import hostlib
    if not os.path.exists(hostlib.LIB_PATH):
        pytest.skip("host library not built (python -m arraydiff_cuda_b200.host.build)")
    L = hostlib.load()
    src = open(os.path.join(ROOT, "arraydiff_cuda_b200", "hostlib.py")).read()
    names = sorted(set(re.findall(r"\badh_[a-z0-9_]+", src)))
    assert len(names) > 30
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_capi_defines_what_the_bindings_name():
    capi = open(os.path.join(ROOT, "arraydiff_cuda_b200", "host", "src", "capi.cc")).read()
    src = open(os.path.join(ROOT, "arraydiff_cuda_b200", "hostlib.py")).read()
    for n in sorted(set(re.findall(r"\badh_[a-z0-9_]+", src))):
        assert re.search(r"\b%s\s*\(" % n, capi), n
