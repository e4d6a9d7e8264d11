"""arraydiff_cuda_b200 -- B200 (sm_100a) kernels for arraydiff's spatially parallel convolution path.

The product is the C-ABI shared library ``libarraydiff_b200.so`` (declared in
``include/arraydiff_b200.h``) and the C++ host layer on top of it.  This Python package is
plumbing: it loads the library through ctypes so that tests and the benchmark driver can call
the C ABI with device pointers obtained from torch.  There is no CPU fallback: if the library
is missing, loading raises.
"""
from .abi import lib, load, LIB_PATH, AdError, check  # noqa: F401
