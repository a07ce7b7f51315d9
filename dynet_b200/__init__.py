"""dynet_b200: B200 (sm_100a) kernels for DyNet's fused-layer nodes behind a C ABI.

The product is ``libdyb200.so`` (built in-tree by ``dynet_b200.build``); this package is the
thin ctypes binding the tests and the benchmark use.  There is no CPU or PyTorch fallback:
importing ``dynet_b200.capi`` raises if the library is missing, and creating a context raises
if no sm_100 device is present.
"""
from .capi import Context, DyTensor, Dyb200Error, lib, lib_path  # noqa: F401
