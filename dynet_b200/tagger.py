"""Python front-end of the BiLSTM tagger pass (libdyb200_host.so, host/tagger.cc): the autobatched schedule of
examples/tagger/train_tag-bilstm.cc over a mini-batch of ragged sentences.

Device memory (flat parameter / gradient buffers, the workspace) is owned by torch tensors; all compute happens in the C++
driver through the C ABI of libdyb200.so.  The flat gradient buffer is what data-parallel training all-reduces.
"""
import ctypes as C

import numpy as np

from . import capi
from .lm import host_lib

NAMES = ["emb", "Wx_f", "Wh_f", "b_f", "Wx_r", "Wh_r", "b_r", "l2th", "r2th", "thbias", "th2t", "tbias"]


class TaggerConfig(C.Structure):
    _fields_ = [("V", C.c_uint32), ("E", C.c_uint32), ("H", C.c_uint32), ("TH", C.c_uint32), ("NT", C.c_uint32),
                ("lr", C.c_float), ("clip", C.c_float)]


def _bind(L):
    if getattr(L, "_tagger_bound", False):
        return L
    u32p = C.POINTER(C.c_uint32)
    L.dyb200h_tagger_num_params.restype = C.c_size_t
    L.dyb200h_tagger_num_params.argtypes = [C.POINTER(TaggerConfig)]
    L.dyb200h_tagger_param_offsets.restype = C.c_int
    L.dyb200h_tagger_param_offsets.argtypes = [C.POINTER(TaggerConfig), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.c_int]
    L.dyb200h_tagger_workspace_bytes.restype = C.c_size_t
    L.dyb200h_tagger_workspace_bytes.argtypes = [C.POINTER(TaggerConfig), C.c_uint32, C.c_uint32]
    L.dyb200h_tagger_create.restype = C.c_int
    L.dyb200h_tagger_create.argtypes = [C.POINTER(TaggerConfig), C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32,
                                        C.c_uint32, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]
    L.dyb200h_tagger_destroy.argtypes = [C.c_void_p]
    L.dyb200h_tagger_error.restype = C.c_char_p
    L.dyb200h_tagger_error.argtypes = [C.c_void_p]
    L.dyb200h_tagger_forward_backward.restype = C.c_int
    L.dyb200h_tagger_forward_backward.argtypes = [C.c_void_p, C.c_uint32, u32p, u32p, u32p, C.c_void_p]
    L.dyb200h_tagger_grad_sumsq.restype = C.c_int
    L.dyb200h_tagger_grad_sumsq.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    L.dyb200h_tagger_update.restype = C.c_int
    L.dyb200h_tagger_update.argtypes = [C.c_void_p]
    L.dyb200h_tagger_time_movers.restype = C.c_int
    L.dyb200h_tagger_time_movers.argtypes = [C.c_void_p, C.c_int]
    L.dyb200h_tagger_mover_ms.restype = C.c_int
    L.dyb200h_tagger_mover_ms.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_double)]
    L.dyb200h_tagger_side_stats.restype = C.c_int
    L.dyb200h_tagger_side_stats.argtypes = [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)]
    L._tagger_bound = True
    return L


def param_shapes(V, E, H, TH, NT):
    """(rows, cols) of the 12 parameter tensors in buffer order (see NAMES)."""
    G = 4 * H
    return [(E, V), (G, E), (G, H), (G, 1), (G, E), (G, H), (G, 1), (TH, H), (TH, H), (TH, 1), (NT, TH), (NT, 1)]


def init_params(V, E, H, TH, NT, seed):
    """DyNet's default initialisers: Glorot-uniform matrices, U(+-sqrt(3/E)) lookup table, zero biases
    (dynet/param-init.cc:26-40, dynet/model.cc:415).  Flat float32 arrays, column-major."""
    r = np.random.Generator(np.random.PCG64(seed))
    out = []
    for k, (rows, cols) in enumerate(param_shapes(V, E, H, TH, NT)):
        if k == 0:
            a = np.sqrt(3.0 / rows)
            out.append(r.uniform(-a, a, rows * cols).astype(np.float32))
        elif cols == 1:
            out.append(np.zeros(rows, np.float32))
        else:
            a = np.sqrt(6.0 / (rows + cols))
            out.append(r.uniform(-a, a, rows * cols).astype(np.float32))
    return out


def synthetic_corpus(n_sent, V, NT, seed, lo=5, hi=100, zipf_s=1.1):
    """Sentences with lengths ~ U{lo..hi}, word ids ~ Zipf(s) over the vocabulary, tags ~ U{0..NT-1}.  Returns
    (lens uint32[n_sent], words uint32[tokens], tags uint32[tokens]) sorted by length, longest first, words / tags
    concatenated sentence by sentence."""
    r = np.random.Generator(np.random.PCG64(seed))
    lens = np.sort(r.integers(lo, hi + 1, n_sent).astype(np.uint32))[::-1].copy()
    n = int(lens.sum())
    ranks = np.arange(1, V + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** (-zipf_s))
    cdf /= cdf[-1]
    words = np.minimum(np.searchsorted(cdf, r.random(n)), V - 1).astype(np.uint32)
    tags = r.integers(0, NT, n).astype(np.uint32)
    return lens, words, tags


class Tagger:
    """BiLSTM tagger training pass on one GPU."""

    def __init__(self, V, E, H, TH, NT, max_sentences, max_tokens, max_len, device=0, seed=0, lr=0.1, clip=5.0, stream=None,
                 params=None):
        import torch
        self.torch = torch
        self.dims = (V, E, H, TH, NT)
        self.cfg = TaggerConfig(V, E, H, TH, NT, lr, clip)
        self.H = _bind(host_lib())
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        self.ctx = capi.Context(device, stream)
        self.n_params = int(self.H.dyb200h_tagger_num_params(C.byref(self.cfg)))
        host = params if params is not None else init_params(V, E, H, TH, NT, seed)
        self.sizes = [int(p.size) for p in host]
        assert sum(self.sizes) == self.n_params
        self.params = torch.from_numpy(np.concatenate([np.asarray(p, np.float32).ravel() for p in host])).to(self.device)
        self.grads = torch.zeros(self.n_params, dtype=torch.float32, device=self.device)
        ws = int(self.H.dyb200h_tagger_workspace_bytes(C.byref(self.cfg), max_sentences, max_tokens))
        self.workspace = torch.empty(ws, dtype=torch.uint8, device=self.device)
        self.loss_dev = torch.zeros(1, dtype=torch.float32, device=self.device)
        h = C.c_void_p()
        rc = self.H.dyb200h_tagger_create(C.byref(self.cfg), self.params.data_ptr(), self.grads.data_ptr(), self.workspace.data_ptr(),
                                          ws, max_sentences, max_tokens, max_len, self.ctx.h, stream, C.byref(h))
        if rc != 0:
            raise capi.Dyb200Error("dyb200h_tagger_create failed with status %d" % rc)
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.torch.cuda.synchronize()
            self.H.dyb200h_tagger_destroy(self.h)
            self.h = None

    def _check(self, rc):
        if rc != 0:
            exc = {1: capi.InvalidArgument, 2: capi.RuntimeErr, 3: capi.CudaError, 4: capi.OutOfMemory}.get(rc, capi.Dyb200Error)
            raise exc(self.H.dyb200h_tagger_error(self.h).decode())

    def launch_forward_backward(self, lens, words, tags):
        """Asynchronous; lens / words / tags are contiguous uint32 numpy arrays (host).  Gradients accumulate."""
        u32p = C.POINTER(C.c_uint32)
        for a in (lens, words, tags):
            assert a.dtype == np.uint32 and a.flags["C_CONTIGUOUS"]
        self._keep = (lens, words, tags)
        self._check(self.H.dyb200h_tagger_forward_backward(self.h, len(lens), lens.ctypes.data_as(u32p), words.ctypes.data_as(u32p),
                                                           tags.ctypes.data_as(u32p), self.loss_dev.data_ptr()))

    def forward_backward(self, lens, words, tags):
        self.launch_forward_backward(lens, words, tags)
        return float(self.loss_dev.item())

    def allreduce_grads(self):
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(self.grads, op=dist.ReduceOp.SUM)

    def update(self):
        self._check(self.H.dyb200h_tagger_grad_sumsq(self.h, None))
        self._check(self.H.dyb200h_tagger_update(self.h))

    def time_movers(self, enable):
        self._check(self.H.dyb200h_tagger_time_movers(self.h, int(enable)))

    def mover_ms(self):
        """({copy fwd-direction, copy bwd-direction, accumulate fwd-direction, accumulate bwd-direction} in ms, host ms spent on the
        schedule and pointer tables) of the last pass; waits for it."""
        ms, host = (C.c_float * 4)(), C.c_double(0)
        self._check(self.H.dyb200h_tagger_mover_ms(self.h, ms, C.byref(host)))
        return [float(v) for v in ms], float(host.value)

    def launches(self):
        """Kernel launches so far, both directions' contexts together."""
        n = C.c_uint64(0)
        self._check(self.H.dyb200h_tagger_side_stats(self.h, C.byref(n), None))
        return self.ctx.launches() + int(n.value)

    def device_errors(self):
        """Device error flags of both contexts (waits for the work issued so far)."""
        f = C.c_uint32(0)
        self._check(self.H.dyb200h_tagger_side_stats(self.h, None, C.byref(f)))
        return self.ctx.device_errors() | int(f.value)

    def grads_host(self):
        flat = self.grads.cpu().numpy()
        return dict(zip(NAMES, [a.copy() for a in np.split(flat, np.cumsum(self.sizes)[:-1])]))

    def params_host(self):
        flat = self.params.cpu().numpy()
        return dict(zip(NAMES, [a.copy() for a in np.split(flat, np.cumsum(self.sizes)[:-1])]))
