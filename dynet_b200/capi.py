"""ctypes binding of include/dyb200.h.

Device memory is handled by the caller (the tests and the benchmark use torch CUDA tensors
and pass ``tensor.data_ptr()``); nothing here computes on the host.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

OK, EINVAL, ERUNTIME, ECUDA, ENOMEM = 0, 1, 2, 3, 4


class Dyb200Error(Exception):
    """Base of the errors raised for a non-zero status."""


class InvalidArgument(Dyb200Error, ValueError):
    """DYB200_EINVAL: the reference throws std::invalid_argument here."""


class RuntimeErr(Dyb200Error, RuntimeError):
    """DYB200_ERUNTIME: the reference throws std::runtime_error here."""


class CudaError(Dyb200Error):
    """DYB200_ECUDA: the reference throws dynet::cuda_exception here."""


class OutOfMemory(Dyb200Error, MemoryError):
    """DYB200_ENOMEM: the reference throws dynet::out_of_memory here."""


_EXC = {EINVAL: InvalidArgument, ERUNTIME: RuntimeErr, ECUDA: CudaError, ENOMEM: OutOfMemory}


class DyTensor(C.Structure):
    """struct dyb200_tensor"""
    _fields_ = [("v", C.c_void_p), ("d", C.c_uint32 * 7), ("nd", C.c_uint32), ("bd", C.c_uint32)]

    @staticmethod
    def of(ptr, dims, bd=1):
        t = DyTensor()
        t.v = ptr
        dims = list(dims)
        assert len(dims) <= 7
        for k, d in enumerate(dims):
            t.d[k] = d
        t.nd = len(dims)
        t.bd = bd
        return t


class EluAttrs(C.Structure):
    _fields_ = [("alpha", C.c_float), ("lam", C.c_float)]


class DimAttrs(C.Structure):
    _fields_ = [("dimension", C.c_uint32)]


class PickAttrs(C.Structure):
    _fields_ = [("ids_host", C.POINTER(C.c_uint32)), ("n", C.c_uint32)]


class LookupAttrs(C.Structure):
    _fields_ = [("all_values", C.c_void_p), ("vocab", C.c_uint32), ("ids_host", C.POINTER(C.c_uint32)),
                ("n", C.c_uint32), ("weight_decay_scale", C.c_float)]


class LstmGatesAttrs(C.Structure):
    _fields_ = [("dropout", C.c_int32), ("weightnoise_std", C.c_float), ("forget_gate_bias", C.c_float)]


class PickRangeAttrs(C.Structure):
    _fields_ = [("start", C.c_uint), ("end", C.c_uint), ("dim", C.c_uint)]


class SumDimAttrs(C.Structure):
    _fields_ = [("dims", C.c_uint * 2), ("ndims", C.c_uint), ("include_batch_dim", C.c_int)]


class ConstAttrs(C.Structure):
    _fields_ = [("c", C.c_float)]


class BernoulliAttrs(C.Structure):
    _fields_ = [("p", C.c_float), ("scale", C.c_float), ("seed", C.c_uint64), ("offset", C.c_uint64)]


class TrainerHyper(C.Structure):
    _fields_ = [("learning_rate", C.c_float), ("clip_threshold", C.c_float), ("weight_decay", C.c_float),
                ("momentum", C.c_float), ("epsilon", C.c_float), ("rho", C.c_float), ("beta_1", C.c_float),
                ("beta_2", C.c_float), ("updates", C.c_uint64)]


RULES = {"sgd": 0, "momentum": 1, "adagrad": 2, "adadelta": 3, "rmsprop": 4, "adam": 5, "amsgrad": 6}


class AffineAttrs(C.Structure):
    _fields_ = [("flags", C.c_uint)]


class MomentAttrs(C.Structure):
    _fields_ = [("dims", C.c_uint32 * 2), ("ndims", C.c_uint32), ("order", C.c_uint32),
                ("include_batch_dim", C.c_int32), ("overwrite_n", C.c_uint32)]


NODES = ["tanh", "logistic", "rectify", "elu", "cmult", "csum", "cdiv", "softmax", "log_softmax",
         "logsumexp_dim", "logsumexp", "pickneglogsoftmax", "weight_norm", "moment_dim", "std_dim",
         "layer_norm", "vanilla_lstm_gates", "vanilla_lstm_c", "vanilla_lstm_h", "matmul", "affine_transform",
         "pick_range", "concatenate", "sum", "sum_dim", "squared_norm", "negate", "constant_plus_x", "constant_minus_x"]
FWD_ONLY = ["lookup", "random_bernoulli"]
OTHER = ["dyb200_ctx_create", "dyb200_ctx_destroy", "dyb200_last_error", "dyb200_ctx_check_device_errors",
         "dyb200_ctx_launch_count", "dyb200_version", "dyb200_lookup_accumulate_grads",
         "dyb200_lookup_accumulate_grads_noalloc",
         "dyb200_parallel_memcpy", "dyb200_parallel_accumulate", "dyb200_gemm", "dyb200_fill", "dyb200_sum_all",
         "dyb200_squared_norm", "dyb200_sgd_update", "dyb200_trainer_update", "dyb200_ctx_profile_begin", "dyb200_ctx_profile_end",
         "dyb200_ctx_profile_count", "dyb200_ctx_profile_launch",
         "dyb200_ctx_param_cache", "dyb200_ctx_params_changed", "dyb200_ctx_dependent_launch", "dyb200_ctx_cluster_splitk", "dyb200_vanilla_lstm_fwd_fused",
         "dyb200_vanilla_lstm_bwd_fused", "dyb200_vanilla_lstm_fwd_fused_at", "dyb200_vanilla_lstm_bwd_fused_at",
         "dyb200_vanilla_lstm_seq_fwd", "dyb200_vanilla_lstm_seq_bwd", "dyb200_ctx_sequence_kernels", "dyb200_wgrad_create", "dyb200_wgrad_destroy", "dyb200_wgrad_push",
         "dyb200_wgrad_flush", "dyb200_wgrad_pack_inputs", "dyb200_softmax_output_bwd_fused"]


def exported_symbols():
    """Every symbol include/dyb200.h declares."""
    syms = list(OTHER)
    for n in NODES:
        syms += ["dyb200_%s_fwd" % n, "dyb200_%s_bwd" % n]
    syms += ["dyb200_%s_fwd" % n for n in FWD_ONLY]
    return syms


def lib_path():
    """The in-tree library; DYB200_LIB names another build of it (kernel experiments)."""
    return os.environ.get("DYB200_LIB") or os.path.join(_HERE, "libdyb200.so")


def lib():
    """Loads libdyb200.so; raises (no fallback) if it has not been built."""
    global _LIB
    if _LIB is None:
        p = lib_path()
        if not os.path.exists(p):
            raise ImportError("libdyb200.so is missing: run `python -m dynet_b200.build` (nvcc, sm_100a); "
                              "there is no CPU fallback")
        L = C.CDLL(p)
        tp = C.POINTER(DyTensor)
        for n in NODES + FWD_ONLY:
            f = getattr(L, "dyb200_%s_fwd" % n)
            f.restype = C.c_int
            f.argtypes = [tp, C.c_int, tp, C.c_void_p, C.c_void_p, C.c_void_p]
        for n in NODES:
            f = getattr(L, "dyb200_%s_bwd" % n)
            f.restype = C.c_int
            f.argtypes = [tp, C.c_int, tp, tp, C.c_uint, tp, C.c_void_p, C.c_void_p, C.c_void_p]
        L.dyb200_ctx_create.restype = C.c_int
        L.dyb200_ctx_create.argtypes = [C.c_int, C.c_void_p, C.POINTER(C.c_void_p)]
        L.dyb200_ctx_destroy.argtypes = [C.c_void_p]
        L.dyb200_last_error.restype = C.c_char_p
        L.dyb200_last_error.argtypes = [C.c_void_p]
        L.dyb200_ctx_check_device_errors.restype = C.c_int
        L.dyb200_ctx_check_device_errors.argtypes = [C.c_void_p, C.POINTER(C.c_uint32)]
        L.dyb200_ctx_launch_count.restype = C.c_uint64
        L.dyb200_ctx_launch_count.argtypes = [C.c_void_p]
        L.dyb200_version.restype = C.c_char_p
        L.dyb200_vanilla_lstm_fwd_fused.restype = C.c_int
        L.dyb200_vanilla_lstm_fwd_fused.argtypes = [tp] * 8 + [C.POINTER(LstmGatesAttrs)] + [tp] * 3 + [C.c_void_p]
        L.dyb200_vanilla_lstm_bwd_fused.restype = C.c_int
        L.dyb200_vanilla_lstm_bwd_fused.argtypes = [tp] * 17 + [C.POINTER(LstmGatesAttrs), C.c_void_p, C.c_void_p]
        L.dyb200_vanilla_lstm_fwd_fused_at.restype = C.c_int
        L.dyb200_vanilla_lstm_fwd_fused_at.argtypes = [tp] * 8 + [C.POINTER(LstmGatesAttrs)] + [tp] * 3 + [C.c_void_p, C.c_uint32, C.c_void_p]
        L.dyb200_vanilla_lstm_bwd_fused_at.restype = C.c_int
        L.dyb200_vanilla_lstm_bwd_fused_at.argtypes = [tp] * 17 + [C.POINTER(LstmGatesAttrs), C.c_void_p, C.c_uint32, C.c_void_p]
        L.dyb200_vanilla_lstm_seq_fwd.restype = C.c_int
        L.dyb200_vanilla_lstm_seq_fwd.argtypes = [tp] * 8 + [C.POINTER(LstmGatesAttrs)] + [tp] * 3 + [C.c_void_p, C.c_uint32, C.c_void_p]
        L.dyb200_vanilla_lstm_seq_bwd.restype = C.c_int
        L.dyb200_vanilla_lstm_seq_bwd.argtypes = [tp] * 7 + [C.POINTER(LstmGatesAttrs)] + [tp] * 9 + [C.c_void_p, C.c_uint32, C.c_void_p]
        L.dyb200_ctx_sequence_kernels.restype = C.c_int
        L.dyb200_ctx_sequence_kernels.argtypes = [C.c_void_p, C.c_int]
        L.dyb200_wgrad_create.restype = C.c_int
        L.dyb200_wgrad_create.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_void_p)]
        L.dyb200_wgrad_destroy.restype = C.c_int
        L.dyb200_wgrad_destroy.argtypes = [C.c_void_p]
        L.dyb200_wgrad_push.restype = C.c_int
        L.dyb200_wgrad_push.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_int,
                                        C.c_void_p, C.c_uint32, C.c_void_p, C.c_int, C.c_void_p]
        L.dyb200_wgrad_flush.restype = C.c_int
        L.dyb200_wgrad_flush.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p]
        L.dyb200_ctx_param_cache.restype = C.c_int
        L.dyb200_ctx_param_cache.argtypes = [C.c_void_p, C.c_int]
        L.dyb200_ctx_dependent_launch.restype = C.c_int
        L.dyb200_ctx_dependent_launch.argtypes = [C.c_void_p, C.c_int]
        L.dyb200_ctx_cluster_splitk.restype = C.c_int
        L.dyb200_ctx_cluster_splitk.argtypes = [C.c_void_p, C.c_int]
        L.dyb200_ctx_params_changed.restype = C.c_int
        L.dyb200_ctx_params_changed.argtypes = [C.c_void_p]
        L.dyb200_ctx_profile_begin.restype = C.c_int
        L.dyb200_ctx_profile_begin.argtypes = [C.c_void_p, C.c_int]
        L.dyb200_ctx_profile_end.restype = C.c_int
        L.dyb200_ctx_profile_end.argtypes = [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_uint64), C.POINTER(C.c_double)]
        L.dyb200_ctx_profile_count.restype = C.c_int
        L.dyb200_ctx_profile_count.argtypes = [C.c_void_p]
        L.dyb200_ctx_profile_launch.restype = C.c_int
        L.dyb200_ctx_profile_launch.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_int), C.POINTER(C.c_float),
                                                C.POINTER(C.c_double)]
        L.dyb200_lookup_accumulate_grads.restype = C.c_int
        L.dyb200_lookup_accumulate_grads.argtypes = [C.c_uint, C.POINTER(C.c_uint32), C.c_void_p, C.c_void_p,
                                                     C.c_void_p, C.c_uint, C.c_uint, C.c_void_p]
        L.dyb200_lookup_accumulate_grads_noalloc.restype = C.c_int
        L.dyb200_lookup_accumulate_grads_noalloc.argtypes = L.dyb200_lookup_accumulate_grads.argtypes
        for n in ("dyb200_parallel_memcpy", "dyb200_parallel_accumulate"):
            f = getattr(L, n)
            f.restype = C.c_int
            f.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        # every pointer-taking entry point gets explicit argtypes: without them ctypes passes Python ints as 32-bit C ints
        L.dyb200_fill.restype = C.c_int
        L.dyb200_fill.argtypes = [C.c_void_p, C.c_size_t, C.c_float, C.c_void_p]
        for name in ("dyb200_sum_all", "dyb200_squared_norm"):
            f = getattr(L, name)
            f.restype = C.c_int
            f.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_int, C.c_void_p]
        L.dyb200_sgd_update.restype = C.c_int
        L.dyb200_sgd_update.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_float, C.c_void_p, C.c_void_p]
        L.dyb200_trainer_update.restype = C.c_int
        L.dyb200_trainer_update.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                            C.POINTER(TrainerHyper), C.c_void_p, C.c_int, C.c_void_p]
        L.dyb200_wgrad_pack_inputs.restype = C.c_int
        L.dyb200_wgrad_pack_inputs.argtypes = [C.c_void_p, tp, tp, C.c_uint32, C.c_void_p]
        L.dyb200_softmax_output_bwd_fused.restype = C.c_int
        L.dyb200_softmax_output_bwd_fused.argtypes = [tp, tp, tp, tp, C.c_void_p, tp, tp, tp, tp, C.c_uint32, C.c_void_p]
        L.dyb200_gemm.restype = C.c_int
        L.dyb200_gemm.argtypes = [C.c_int, C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32,
                                  C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_int, C.c_uint, C.c_void_p]
        _LIB = L
    return _LIB


class Context:
    """Owns one dyb200_ctx (device, stream, scratch arena)."""

    def __init__(self, device=0, stream=None):
        self.L = lib()
        h = C.c_void_p()
        rc = self.L.dyb200_ctx_create(device, stream, C.byref(h))
        if rc != OK:
            raise _EXC.get(rc, Dyb200Error)("dyb200_ctx_create(device=%d) failed with status %d: a B200 "
                                            "(sm_100) device is required, there is no CPU fallback" % (device, rc))
        self.h = h

    def close(self):
        if self.h:
            self.L.dyb200_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, rc):
        if rc != OK:
            raise _EXC.get(rc, Dyb200Error)(self.L.dyb200_last_error(self.h).decode())

    def launches(self):
        return int(self.L.dyb200_ctx_launch_count(self.h))

    def profile_begin(self, capacity=1 << 16):
        self.check(self.L.dyb200_ctx_profile_begin(self.h, capacity))

    def profile_end(self):
        """Returns {"simt": (ms, launches, flops), "tensor": (...)} summed over the recorded GEMM launches."""
        ms, n, fl = (C.c_double * 2)(), (C.c_uint64 * 2)(), (C.c_double * 2)()
        self.check(self.L.dyb200_ctx_profile_end(self.h, ms, n, fl))
        return {"simt": (ms[0], int(n[0]), fl[0]), "tensor": (ms[1], int(n[1]), fl[1])}

    def profile_launches(self):
        """Per recorded GEMM launch (call between profile_begin and profile_end): (M, N, K, epilogue mode, path, ms, flops)."""
        out = []
        for k in range(int(self.L.dyb200_ctx_profile_count(self.h))):
            shape, path, ms, fl = (C.c_uint32 * 4)(), C.c_int(0), C.c_float(0), C.c_double(0)
            self.check(self.L.dyb200_ctx_profile_launch(self.h, k, shape, C.byref(path), C.byref(ms), C.byref(fl)))
            out.append((shape[0], shape[1], shape[2], shape[3], path.value, ms.value, fl.value))
        return out

    def device_errors(self):
        f = C.c_uint32(0)
        self.check(self.L.dyb200_ctx_check_device_errors(self.h, C.byref(f)))
        return f.value

    @staticmethod
    def _arr(ts):
        if not ts:
            return None, 0
        a = (DyTensor * len(ts))(*ts)
        return a, len(ts)

    def fwd(self, node, xs, fx, attrs=None, aux=None):
        a, n = self._arr(xs)
        f = getattr(self.L, "dyb200_%s_fwd" % node)
        self.check(f(a, n, C.byref(fx), C.cast(C.byref(attrs), C.c_void_p) if attrs is not None else None, aux, self.h))

    def bwd(self, node, xs, fx, dEdf, i, dEdxi, attrs=None, aux=None):
        a, n = self._arr(xs)
        f = getattr(self.L, "dyb200_%s_bwd" % node)
        self.check(f(a, n, C.byref(fx), C.byref(dEdf), i, C.byref(dEdxi),
                     C.cast(C.byref(attrs), C.c_void_p) if attrs is not None else None, aux, self.h))

    def lookup_accumulate_grads(self, ids_host, ids_dev_ptr, g_ptr, all_grads_ptr, dim_size, vocab, n=None):
        """ids_host may be empty with n given: the ids are then only read on the device."""
        arr = None
        if n is None:
            n = len(ids_host)
            arr = (C.c_uint32 * n)(*[int(i) for i in ids_host]) if n else None
        self.check(self.L.dyb200_lookup_accumulate_grads(n, arr, ids_dev_ptr, g_ptr, all_grads_ptr, dim_size, vocab, self.h))

    def lookup_accumulate_grads_noalloc(self, ids_host, ids_dev_ptr, g_ptr, all_grads_ptr, dim_size, vocab):
        """Same as lookup_accumulate_grads, through the entry point that never allocates device memory."""
        n = len(ids_host)
        arr = (C.c_uint32 * n)(*[int(i) for i in ids_host]) if n else None
        self.check(self.L.dyb200_lookup_accumulate_grads_noalloc(n, arr, ids_dev_ptr, g_ptr, all_grads_ptr, dim_size, vocab, self.h))

    def parallel_memcpy(self, num_seqs, max_len, src_tbl, trg_tbl, len_tbl):
        self.check(self.L.dyb200_parallel_memcpy(num_seqs, max_len, src_tbl, trg_tbl, len_tbl, self.h))

    def parallel_accumulate(self, num_seqs, max_len, src_tbl, trg_tbl, len_tbl):
        self.check(self.L.dyb200_parallel_accumulate(num_seqs, max_len, src_tbl, trg_tbl, len_tbl, self.h))

    def gemm(self, transA, transB, M, N, K, A, lda, B, ldb, Cp, ldc, accumulate, flags=0):
        self.check(self.L.dyb200_gemm(int(transA), int(transB), M, N, K, A, lda, B, ldb, Cp, ldc, int(accumulate), flags, self.h))

    @staticmethod
    def _opt(t):
        return C.byref(t) if t is not None else None

    def lstm_fwd_fused(self, x, h_tm1, c_tm1, Wx, Wh, b, mask_x, mask_h, attrs, gates, c_t, h_t):
        o = self._opt
        self.check(self.L.dyb200_vanilla_lstm_fwd_fused(o(x), o(h_tm1), o(c_tm1), o(Wx), o(Wh), o(b), o(mask_x), o(mask_h),
                                                        C.byref(attrs), o(gates), o(c_t), o(h_t), self.h))

    def lstm_bwd_fused(self, x, h_tm1, c_tm1, Wx, Wh, mask_x, mask_h, gates, c_t, dEdh, dEdc, dx, dh_tm1, dc_tm1, dWx, dWh, db, attrs,
                       deferred=None):
        o = self._opt
        self.check(self.L.dyb200_vanilla_lstm_bwd_fused(o(x), o(h_tm1), o(c_tm1), o(Wx), o(Wh), o(mask_x), o(mask_h), o(gates), o(c_t),
                                                        o(dEdh), o(dEdc), o(dx), o(dh_tm1), o(dc_tm1), o(dWx), o(dWh), o(db),
                                                        C.byref(attrs), deferred, self.h))

    WGRAD_APPEND = 0xffffffff

    def lstm_fwd_fused_at(self, x, h_tm1, c_tm1, Wx, Wh, b, mask_x, mask_h, attrs, gates, c_t, h_t, deferred, col):
        o = self._opt
        self.check(self.L.dyb200_vanilla_lstm_fwd_fused_at(o(x), o(h_tm1), o(c_tm1), o(Wx), o(Wh), o(b), o(mask_x), o(mask_h),
                                                           C.byref(attrs), o(gates), o(c_t), o(h_t), deferred, col, self.h))

    def lstm_seq_fwd(self, x_all, h0, c0, Wx, Wh, b, mask_x, mask_h, attrs, gates_all, c_all, h_all, deferred, steps):
        o = self._opt
        self.check(self.L.dyb200_vanilla_lstm_seq_fwd(o(x_all), o(h0), o(c0), o(Wx), o(Wh), o(b), o(mask_x), o(mask_h), C.byref(attrs),
                                                      o(gates_all), o(c_all), o(h_all), deferred, steps, self.h))

    def lstm_seq_bwd(self, x_all, h0, c0, Wx, Wh, mask_x, mask_h, attrs, gates_all, c_all, h_all, dh_all, dc_all, dx_all, dWx, dWh, db,
                     deferred, steps):
        o = self._opt
        self.check(self.L.dyb200_vanilla_lstm_seq_bwd(o(x_all), o(h0), o(c0), o(Wx), o(Wh), o(mask_x), o(mask_h), C.byref(attrs),
                                                      o(gates_all), o(c_all), o(h_all), o(dh_all), o(dc_all), o(dx_all), o(dWx), o(dWh),
                                                      o(db), deferred, steps, self.h))

    def sequence_kernels(self, enable):
        self.check(self.L.dyb200_ctx_sequence_kernels(self.h, int(enable)))

    def lstm_bwd_fused_at(self, x, h_tm1, c_tm1, Wx, Wh, mask_x, mask_h, gates, c_t, dEdh, dEdc, dx, dh_tm1, dc_tm1, dWx, dWh, db, attrs,
                          deferred, col):
        o = self._opt
        self.check(self.L.dyb200_vanilla_lstm_bwd_fused_at(o(x), o(h_tm1), o(c_tm1), o(Wx), o(Wh), o(mask_x), o(mask_h), o(gates), o(c_t),
                                                           o(dEdh), o(dEdc), o(dx), o(dh_tm1), o(dc_tm1), o(dWx), o(dWh), o(db),
                                                           C.byref(attrs), deferred, col, self.h))

    def softmax_output_bwd_fused(self, x, h, R, dEdf, aux_ptr, dR, db, dh, dx_scratch=None, flags=0):
        """Backward of PickNegLogSoftmax(affine_transform({b, R, h})) in one call (DyTensor arguments, aux_ptr: device pointer)."""
        o = self._opt
        self.check(self.L.dyb200_softmax_output_bwd_fused(o(x), o(h), o(R), o(dEdf), aux_ptr, o(dR), o(db), o(dh), o(dx_scratch),
                                                          flags, self.h))

    def wgrad_pack_inputs(self, w, x_all, mask_x, step):
        self.check(self.L.dyb200_wgrad_pack_inputs(w, self._opt(x_all), self._opt(mask_x), step, self.h))

    def wgrad_create(self, M, N0, N1, Kcap):
        h = C.c_void_p()
        self.check(self.L.dyb200_wgrad_create(self.h, M, N0, N1, Kcap, C.byref(h)))
        return h

    def wgrad_destroy(self, w):
        self.L.dyb200_wgrad_destroy(w)

    def wgrad_push(self, w, k, a, lda, b0, ldb0, mask0=None, mask0_full=0, b1=None, ldb1=0, mask1=None, mask1_full=0):
        self.check(self.L.dyb200_wgrad_push(w, k, a, lda, b0, ldb0, mask0, mask0_full, b1, ldb1, mask1, mask1_full, self.h))

    def wgrad_flush(self, w, C0, ldc0, C1=None, ldc1=0):
        self.check(self.L.dyb200_wgrad_flush(w, C0, ldc0, C1, ldc1, self.h))

    def squared_norm(self, x_ptr, n, out_ptr, accumulate=False):
        self.check(self.L.dyb200_squared_norm(x_ptr, n, out_ptr, int(accumulate), self.h))

    def sum_all(self, x_ptr, n, out_ptr, accumulate=False):
        self.check(self.L.dyb200_sum_all(x_ptr, n, out_ptr, int(accumulate), self.h))

    def trainer_update(self, rule, params, grads, states, n, hyper, grad_sumsq=None, zero_grads=True):
        """rule: key of RULES; params / grads / states / grad_sumsq: device pointers (ints)."""
        st = list(states) + [None] * (3 - len(states))
        self.check(self.L.dyb200_trainer_update(RULES[rule], params, grads, st[0], st[1], st[2], n, C.byref(hyper), grad_sumsq,
                                                int(zero_grads), self.h))

    def cluster_splitk(self, enable):
        self.check(self.L.dyb200_ctx_cluster_splitk(self.h, int(bool(enable))))

    def dependent_launch(self, enable):
        self.check(self.L.dyb200_ctx_dependent_launch(self.h, int(enable)))

    def param_cache(self, enable):
        self.check(self.L.dyb200_ctx_param_cache(self.h, int(enable)))

    def params_changed(self):
        self.check(self.L.dyb200_ctx_params_changed(self.h))
