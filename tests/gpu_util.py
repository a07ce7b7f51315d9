"""Helpers for the GPU parity tests: device buffers come from torch, every computation goes
through the C ABI of libdyb200.so."""
import ctypes as C

import numpy as np

from dynet_b200 import capi

_CTX = None
_KEEP = []   # device buffers stay alive until the test ends: kernels run asynchronously on raw pointers


def release():
    import torch
    torch.cuda.synchronize()
    _KEEP.clear()


def ctx():
    global _CTX
    if _CTX is None:
        _CTX = capi.Context(0)
    return _CTX


def dev(a, misalign=0):
    """numpy -> CUDA tensor (optionally starting `misalign` floats past a 256-byte boundary)."""
    import torch
    a = np.ascontiguousarray(a)
    if misalign:
        buf = torch.empty(a.size + misalign, dtype=torch.from_numpy(a).dtype, device="cuda")
        t = buf[misalign:misalign + a.size].view(a.shape)
        t.copy_(torch.from_numpy(a))
        _KEEP.append(buf)
        return t
    t = torch.from_numpy(a).cuda()
    _KEEP.append(t)
    return t


def zeros_like_dev(a):
    import torch
    return torch.zeros(a.shape, dtype=torch.float32, device="cuda")


def host(t):
    return t.detach().cpu().numpy()


def T(t, dims=None, bd=None):
    """DyTensor view of a torch tensor shaped (bd, ..., d1, d0) (batch first, C order)."""
    if dims is None:
        shape = list(t.shape)
        bd = shape[0]
        dims = shape[1:][::-1]
    return capi.DyTensor.of(t.data_ptr(), dims, bd)


def u32(a):
    a = np.ascontiguousarray(a, dtype=np.uint32)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint32))
