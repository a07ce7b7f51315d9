"""Python front-end of the LSTM language-model step driver (libdyb200_host.so).

Device memory (flat parameter / gradient buffers, the activation workspace) is owned by torch
tensors; all compute happens in the C++ driver through the C ABI of libdyb200.so.  The flat
gradient buffer is what data-parallel training all-reduces (see `allreduce_grads`).
"""
import ctypes as C
import os

import numpy as np

from . import capi

_HERE = os.path.dirname(os.path.abspath(__file__))
_HOST = None


class LmConfig(C.Structure):
    _fields_ = [("V", C.c_uint32), ("E", C.c_uint32), ("H", C.c_uint32), ("L", C.c_uint32), ("T", C.c_uint32),
                ("B", C.c_uint32), ("lr", C.c_float), ("clip", C.c_float), ("dropout", C.c_int32), ("fused", C.c_int32)]


def host_lib():
    global _HOST
    if _HOST is None:
        capi.lib()  # libdyb200.so first (RPATH $ORIGIN resolves it as well)
        p = os.path.join(_HERE, "libdyb200_host.so")
        if not os.path.exists(p):
            raise ImportError("libdyb200_host.so is missing: run `python -m dynet_b200.build`")
        L = C.CDLL(p)
        L.dyb200h_lm_num_params.restype = C.c_size_t
        L.dyb200h_lm_num_params.argtypes = [C.POINTER(LmConfig)]
        L.dyb200h_lm_workspace_bytes.restype = C.c_size_t
        L.dyb200h_lm_workspace_bytes.argtypes = [C.POINTER(LmConfig)]
        L.dyb200h_lm_param_offsets.restype = C.c_int
        L.dyb200h_lm_param_offsets.argtypes = [C.POINTER(LmConfig), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.c_int]
        L.dyb200h_lm_create.restype = C.c_int
        L.dyb200h_lm_create.argtypes = [C.POINTER(LmConfig), C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p,
                                        C.c_void_p, C.POINTER(C.c_void_p)]
        L.dyb200h_lm_destroy.argtypes = [C.c_void_p]
        L.dyb200h_lm_error.restype = C.c_char_p
        L.dyb200h_lm_error.argtypes = [C.c_void_p]
        L.dyb200h_lm_forward_backward.restype = C.c_int
        L.dyb200h_lm_forward_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.c_void_p]
        L.dyb200h_lm_num_phases.restype = C.c_int
        L.dyb200h_lm_num_phases.argtypes = [C.c_void_p]
        L.dyb200h_lm_phase_grad_range.restype = C.c_int
        L.dyb200h_lm_phase_grad_range.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
        L.dyb200h_lm_forward_backward_phase.restype = C.c_int
        L.dyb200h_lm_forward_backward_phase.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.c_void_p]
        L.dyb200h_lm_grad_sumsq.restype = C.c_int
        L.dyb200h_lm_grad_sumsq.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        L.dyb200h_lm_update.restype = C.c_int
        L.dyb200h_lm_update.argtypes = [C.c_void_p]
        L.dyb200h_lm_set_graph.restype = C.c_int
        L.dyb200h_lm_set_graph.argtypes = [C.c_void_p, C.c_int]
        L.dyb200h_lm_set_time_major.restype = C.c_int
        L.dyb200h_lm_set_time_major.argtypes = [C.c_void_p, C.c_int]
        L.dyb200h_lm_graph_launches.restype = C.c_uint64
        L.dyb200h_lm_graph_launches.argtypes = [C.c_void_p]
        L.dyb200h_lm_mask_buffers.restype = C.c_int
        L.dyb200h_lm_mask_buffers.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int]
        L.dyb200h_lm_hidden_states.restype = C.c_void_p
        L.dyb200h_lm_hidden_states.argtypes = [C.c_void_p]
        _HOST = L
    return _HOST


def param_shapes(V, E, H, L):
    """(rows, cols) of the 3L+3 parameter tensors: C, (Wx, Wh, b) per layer, R, bias."""
    shapes = [(E, V)]
    for l in range(L):
        shapes += [(4 * H, E if l == 0 else H), (4 * H, H), (4 * H, 1)]
    shapes += [(V, H), (V, 1)]
    return shapes


def init_params(V, E, H, L, seed):
    """DyNet's default initialisers (dynet/param-init.cc:26-40, dynet/model.cc:415): Glorot-uniform
    U(+-sqrt(6/(r+c))) for matrices, U(+-sqrt(3/E)) for the lookup table (vocab dim excluded),
    zero biases.  Returns flat float32 arrays (column-major)."""
    r = np.random.Generator(np.random.PCG64(seed))
    out = []
    for k, (rows, cols) in enumerate(param_shapes(V, E, H, L)):
        if k == 0:
            a = np.sqrt(3.0 / rows)
            out.append(r.uniform(-a, a, rows * cols).astype(np.float32))
        elif cols == 1:
            out.append(np.zeros(rows, np.float32))
        else:
            a = np.sqrt(6.0 / (rows + cols))
            out.append(r.uniform(-a, a, rows * cols).astype(np.float32))
    return out


def synthetic_batch(dims, seed, dropout=0.2, zipf_s=1.1):
    """Token ids ~ Zipf(s) over the vocabulary, (T+1) x B, and per-layer dropout masks
    Bernoulli(1-p)/(1-p) fixed over the sequence (dynet/lstm.cc:964-982).  Returns
    (tokens uint32 [T+1, B], (mask_x list, mask_h list) of float32 [B, I_l] / [B, H]) or masks None."""
    V, E, H, L, T, B = (dims[k] for k in "VEHLTB")
    r = np.random.Generator(np.random.PCG64(seed))
    ranks = np.arange(1, V + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** (-zipf_s))
    cdf /= cdf[-1]
    tokens = np.minimum(np.searchsorted(cdf, r.random((T + 1) * B)), V - 1).astype(np.uint32).reshape(T + 1, B)
    if not dropout:
        return tokens, None
    keep = 1.0 - dropout
    mx = [((r.random((B, E if l == 0 else H)) < keep) / keep).astype(np.float32) for l in range(L)]
    mh = [((r.random((B, H)) < keep) / keep).astype(np.float32) for l in range(L)]
    return tokens, (mx, mh)


class LstmLm:
    """2-layer (L-layer) LSTM language model training step on one GPU."""

    def __init__(self, V, E, H, L, T, B, device=0, seed=0, lr=0.1, clip=5.0, dropout=True, stream=None, fused=True):
        import torch
        self.torch = torch
        self.dims = (V, E, H, L, T, B)
        # fused=False drives every node and every backward argument separately (the drop-in contract);
        # fused=True uses the per-layer fused entry points (same values, fewer launches)
        self.cfg = LmConfig(V, E, H, L, T, B, lr, clip, 1 if dropout else 0, 1 if fused else 0)
        self.H = host_lib()
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        self.ctx = capi.Context(device, stream)
        n = self.H.dyb200h_lm_num_params(C.byref(self.cfg))
        self.n_params = n
        host = init_params(V, E, H, L, seed)
        self.sizes = [p.size for p in host]
        self.params = torch.from_numpy(np.concatenate(host)).to(self.device)
        self.grads = torch.zeros(n, dtype=torch.float32, device=self.device)
        ws = self.H.dyb200h_lm_workspace_bytes(C.byref(self.cfg))
        self.workspace = torch.empty(ws, dtype=torch.uint8, device=self.device)
        self.loss_dev = torch.zeros(1, dtype=torch.float32, device=self.device)
        h = C.c_void_p()
        rc = self.H.dyb200h_lm_create(C.byref(self.cfg), self.params.data_ptr(), self.grads.data_ptr(),
                                      self.workspace.data_ptr(), ws, self.ctx.h, stream, C.byref(h))
        if rc != 0:
            raise capi.Dyb200Error("dyb200h_lm_create failed with status %d" % rc)
        self.h = h
        self._mask_keep = None

    def close(self):
        if getattr(self, "h", None):
            self.torch.cuda.synchronize()
            self.H.dyb200h_lm_destroy(self.h)
            self.h = None

    def _check(self, rc):
        if rc != 0:
            exc = {1: capi.InvalidArgument, 2: capi.RuntimeErr, 3: capi.CudaError, 4: capi.OutOfMemory}.get(rc, capi.Dyb200Error)
            raise exc(self.H.dyb200h_lm_error(self.h).decode())

    def masks_to_device(self, masks):
        """(mask_x list, mask_h list) of numpy arrays -> list of 2L CUDA tensors in driver order."""
        mx, mh = masks
        out = []
        for l in range(self.dims[3]):
            out += [self.torch.from_numpy(np.ascontiguousarray(mx[l])).to(self.device),
                    self.torch.from_numpy(np.ascontiguousarray(mh[l])).to(self.device)]
        return out

    def launch_forward_backward(self, tokens, masks_dev):
        """Asynchronous: tokens is a numpy uint32 / pinned int32 host tensor [(T+1), B] or a CUDA int32 tensor;
        masks_dev is the list from masks_to_device (or None).  The loss lands in self.loss_dev."""
        torch = self.torch
        if isinstance(tokens, np.ndarray):
            assert tokens.dtype == np.uint32 and tokens.flags["C_CONTIGUOUS"]
            ptr, on_dev = tokens.ctypes.data, 0
        else:
            ptr, on_dev = tokens.data_ptr(), 1 if tokens.is_cuda else 0
        mp = None
        if masks_dev is not None:
            mp = (C.c_void_p * len(masks_dev))(*[m.data_ptr() for m in masks_dev])
        self._check(self.H.dyb200h_lm_forward_backward(self.h, ptr, on_dev, mp, self.loss_dev.data_ptr()))

    def _token_ptr(self, tokens):
        if isinstance(tokens, np.ndarray):
            assert tokens.dtype == np.uint32 and tokens.flags["C_CONTIGUOUS"]
            return tokens.ctypes.data, 0
        return tokens.data_ptr(), 1 if tokens.is_cuda else 0

    def num_phases(self):
        return int(self.H.dyb200h_lm_num_phases(self.h))

    def phase_grad_range(self, phase):
        """(offset, count) in floats of the gradients that are final after `phase`."""
        off, n = C.c_size_t(0), C.c_size_t(0)
        self._check(self.H.dyb200h_lm_phase_grad_range(self.h, phase, C.byref(off), C.byref(n)))
        return int(off.value), int(n.value)

    def launch_phase(self, phase, tokens, masks_dev):
        ptr, on_dev = self._token_ptr(tokens)
        mp = None
        if masks_dev is not None:
            mp = (C.c_void_p * len(masks_dev))(*[m.data_ptr() for m in masks_dev])
        self._check(self.H.dyb200h_lm_forward_backward_phase(self.h, phase, ptr, on_dev, mp, self.loss_dev.data_ptr()))

    def launch_forward_backward_overlapped(self, tokens, masks_dev):
        """Data-parallel step: forward + backward in phases; the gradients that a phase makes final (output layer first,
        then the LSTM layers top down, the embedding table last) are summed over the ranks on a side stream while the next
        phase runs.  The current stream waits for the sums at the end.  Same results as launch_forward_backward followed
        by allreduce_grads (a sum per bucket instead of one over the whole buffer: the same additions per element)."""
        import torch.distributed as dist
        torch = self.torch
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
        n = self.num_phases()
        if not multi or n == 1:
            self.launch_forward_backward(tokens, masks_dev)
            self.allreduce_grads()
            return
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=self.device)
        main = torch.cuda.current_stream()
        works = []
        for p in range(n):
            self.launch_phase(p, tokens, masks_dev)
            ev = torch.cuda.Event()
            ev.record(main)
            off, cnt = self.phase_grad_range(p)
            with torch.cuda.stream(self._side):
                self._side.wait_event(ev)
                works.append(dist.all_reduce(self.grads[off:off + cnt], op=dist.ReduceOp.SUM, async_op=True))
        self._after_last_phase = torch.cuda.Event(enable_timing=True)
        self._after_last_phase.record(main)
        for w in works:
            w.wait()          # the current stream waits for the collective

    def forward_backward(self, tokens, masks=None):
        """Synchronous convenience wrapper used by the tests: returns the loss as a float."""
        md = self.masks_to_device(masks) if masks is not None else None
        self._keep = md
        self.launch_forward_backward(tokens, md)
        return float(self.loss_dev.item())

    def set_graph(self, enable):
        """Replay forward + backward as one CUDA graph (needs a non-default stream and one eager step before)."""
        self._check(self.H.dyb200h_lm_set_graph(self.h, int(enable)))

    def set_time_major(self, enable):
        """Fused driver: run the (time step, layer) calls time step by time step (the reference's order) instead of layer by layer."""
        self._check(self.H.dyb200h_lm_set_time_major(self.h, int(enable)))

    def graph_launches(self):
        return int(self.H.dyb200h_lm_graph_launches(self.h))

    def mask_buffers(self):
        """The driver's own 2L mask buffers as torch views into the workspace (mask_x_l is [B, I_l], mask_h_l [B, H])."""
        V, E, H, L, T, B = self.dims
        ptrs = (C.c_void_p * (2 * L))()
        n = self.H.dyb200h_lm_mask_buffers(self.h, ptrs, 2 * L)
        out, base = [], self.workspace.data_ptr()
        for k in range(n):
            cols = (E if k == 0 else H) if k % 2 == 0 else H
            off = ptrs[k] - base
            out.append(self.workspace[off:off + 4 * B * cols].view(self.torch.float32).view(B, cols))
        return out

    def draw_masks(self, keep, seed, step):
        """Fresh dropout masks in the driver's buffers: RandomBernoulli(keep, 1/keep) per layer input and hidden state
        (dynet/lstm.cc:964-982), one launch per mask; `step` selects a disjoint stretch of the random stream."""
        from . import capi
        bufs = self.mask_buffers()
        off = 0
        for k, mk in enumerate(bufs):
            n = mk.numel()
            at = capi.BernoulliAttrs(float(keep), 1.0 / float(keep), int(seed), int(step) * self._mask_quads + off)
            self.ctx.fwd("random_bernoulli", [], capi.DyTensor.of(mk.data_ptr(), [mk.shape[1]], mk.shape[0]), at)
            off += (n + 3) // 4
        return bufs

    @property
    def _mask_quads(self):
        V, E, H, L, T, B = self.dims
        return sum(((B * ((E if l == 0 else H)) + 3) // 4) + ((B * H + 3) // 4) for l in range(L))

    def allreduce_grads(self):
        """Sum the flat gradient buffer over the data-parallel ranks (NCCL over NVLink)."""
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(self.grads, op=dist.ReduceOp.SUM)

    def update(self):
        """Gradient-norm clipping + SimpleSGD + zeroing of the gradients (all on the device)."""
        self._check(self.H.dyb200h_lm_grad_sumsq(self.h, None))
        self._check(self.H.dyb200h_lm_update(self.h))

    def params_host(self):
        flat = self.params.cpu().numpy()
        return [a.copy() for a in np.split(flat, np.cumsum(self.sizes)[:-1])]

    def grads_host(self):
        flat = self.grads.cpu().numpy()
        return [a.copy() for a in np.split(flat, np.cumsum(self.sizes)[:-1])]

    def set_params_host(self, arrays):
        self.params.copy_(self.torch.from_numpy(np.concatenate([a.ravel() for a in arrays])))
        self.ctx.params_changed()   # the packed copies in the GEMM's parameter cache are stale

    def hidden_states_host(self):
        V, E, H, L, T, B = self.dims
        n = T * L * H * B
        ptr = self.H.dyb200h_lm_hidden_states(self.h)
        out = self.torch.empty(n, dtype=self.torch.float32, device=self.device)
        base = self.workspace.data_ptr()
        off = ptr - base
        out.copy_(self.workspace[off:off + 4 * n].view(self.torch.float32))
        return out.cpu().numpy().reshape(L, T, B, H).transpose(1, 0, 2, 3)   # stored layer-major
