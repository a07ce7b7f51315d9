"""ctypes/numpy front-end of the CPU oracle (test infrastructure only).

The oracle is a plain-C restatement of the CPU branches of DyNet's fused-layer
nodes (see dynet_oracle.c for the per-function reference citations).  Only the
test-suite, the smoke check and the benchmark's CPU-baseline leg import this
package; the shipped CUDA library never does.

All arrays are float32, column-major with the batch as the slowest axis; a
numpy array of shape (bd, ..., d1, d0) in C order has exactly that memory
layout, so callers build arrays "reversed" (batch first).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

f32p = C.POINTER(C.c_float)
u32p = C.POINTER(C.c_uint32)


def build(force=False):
    """Compile liboracle.so next to the sources (gcc via the Makefile)."""
    so = os.path.join(_HERE, "liboracle.so")
    srcs = [os.path.join(_HERE, f) for f in ("dynet_oracle.c", "lstm_lm_oracle.c", "Makefile")]
    if force or not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "liboracle.so"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(so):
            build()
        _LIB = C.CDLL(so)
        _LIB.orc_sigmoid_packet.restype = C.c_float
        _LIB.orc_sigmoid_packet.argtypes = [C.c_float]
        _LIB.orc_sigmoid_scalar.restype = C.c_float
        _LIB.orc_sigmoid_scalar.argtypes = [C.c_float]
        _LIB.orc_sgd_update.restype = C.c_float
    return _LIB


def _f(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"], (a.dtype, a.flags)
    return a.ctypes.data_as(f32p)


def _u(a):
    assert a.dtype == np.uint32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(u32p)


def _shape5(a_shape):
    """numpy shape (bd, d3, d2, d1, d0)-style (batch first) -> uint32[5] = d0..d3, bd."""
    s = list(a_shape)
    bd, dims = s[0], s[1:][::-1]
    dims = dims + [1] * (4 - len(dims))
    return (C.c_uint32 * 5)(*dims, bd)


# ---------------- unary activations ----------------
def unary_fwd(name, x, alpha=1.0, lam=1.0, packet=8):
    y = np.empty_like(x)
    n = C.c_size_t(x.size)
    L = lib()
    if name == "tanh":
        L.orc_tanh_fwd(_f(x), _f(y), n)
    elif name == "logistic":
        L.orc_logistic_fwd(_f(x), _f(y), n, C.c_int(packet))
    elif name == "rectify":
        L.orc_rectify_fwd(_f(x), _f(y), n)
    elif name == "elu":
        L.orc_elu_fwd(_f(x), _f(y), n, C.c_float(alpha), C.c_float(lam))
    else:
        raise KeyError(name)
    return y


def unary_bwd(name, x, y, dy, dx, alpha=1.0, lam=1.0):
    """Accumulates into dx (in place) and returns it."""
    n = C.c_size_t(x.size)
    L = lib()
    if name == "tanh":
        L.orc_tanh_bwd(_f(y), _f(dy), _f(dx), n)
    elif name == "logistic":
        L.orc_logistic_bwd(_f(y), _f(dy), _f(dx), n)
    elif name == "rectify":
        L.orc_rectify_bwd(_f(y), _f(dy), _f(dx), n)
    elif name == "elu":
        L.orc_elu_bwd(_f(x), _f(dy), _f(dx), n, C.c_float(alpha), C.c_float(lam))
    else:
        raise KeyError(name)
    return dx


# ---------------- cwise binary ----------------
_OPS = {"cmult": 0, "csum": 1, "cdiv": 2}


def cwise_fwd(op, a, b):
    """a, b: numpy arrays shaped (bd, [d3, d2, d1,] d0) with equal rank."""
    assert a.ndim == b.ndim
    out_shape = tuple(max(x, y) for x, y in zip(a.shape, b.shape))
    y = np.empty(out_shape, np.float32)
    lib().orc_cwise_fwd(C.c_int(_OPS[op]), _f(a), _shape5(a.shape), _f(b), _shape5(b.shape), _f(y))
    return y


def cwise_bwd(op, a, b, dy, i, dxi):
    lib().orc_cwise_bwd(C.c_int(_OPS[op]), _f(a), _shape5(a.shape), _f(b), _shape5(b.shape),
                        _f(dy), C.c_uint(i), _f(dxi))
    return dxi


# ---------------- softmax family ----------------
def _rcb(x):
    """(bd, cols, rows) view parameters of a 2-D-per-batch tensor."""
    assert x.ndim == 3
    bd, cols, rows = x.shape
    return C.c_uint32(rows), C.c_uint32(cols), C.c_uint32(bd)


def softmax_fwd(x, dimension=0):
    y = np.empty_like(x)
    lib().orc_softmax_fwd(_f(x), _f(y), *_rcb(x), C.c_uint(dimension))
    return y


def softmax_bwd(y, dy, dx, dimension=0):
    lib().orc_softmax_bwd(_f(y), _f(dy), _f(dx), *_rcb(y), C.c_uint(dimension))
    return dx


def logsumexp_dim_fwd(x, axis=0):
    bd, cols, rows = x.shape
    outer = cols if axis == 0 else rows
    z = np.empty((bd, outer), np.float32)
    m = np.empty((bd, outer), np.float32)
    lib().orc_logsumexp_axis(_f(x), *_rcb(x), C.c_uint(axis), _f(m), _f(z))
    return z, m


def logsumexp_dim_bwd(x, z, dz, dx, axis=0):
    lib().orc_logsumexp_dim_bwd(_f(x), _f(z), _f(dz), _f(dx), *_rcb(x), C.c_uint(axis))
    return dx


def log_softmax_fwd(x):
    bd, cols, rows = x.shape
    y = np.empty_like(x)
    z = np.empty((bd, cols), np.float32)
    m = np.empty((bd, cols), np.float32)
    lib().orc_log_softmax_fwd(_f(x), _f(y), *_rcb(x), _f(z), _f(m))
    return y


def log_softmax_bwd(y, dy, dx):
    lib().orc_log_softmax_bwd(_f(y), _f(dy), _f(dx), *_rcb(y))
    return dx


def logsumexp_nary_fwd(xs):
    """xs: list of (bd_k, n) arrays with bd_k in {1, bd}."""
    bd = max(x.shape[0] for x in xs)
    n = xs[0].shape[1]
    y = np.empty((bd, n), np.float32)
    ptrs = (f32p * len(xs))(*[_f(x) for x in xs])
    bds = (C.c_uint32 * len(xs))(*[x.shape[0] for x in xs])
    lib().orc_logsumexp_nary_fwd(ptrs, bds, C.c_uint(len(xs)), C.c_size_t(n), C.c_uint32(bd), _f(y))
    return y


def logsumexp_nary_bwd(xs, i, y, dy, dxi):
    bd, n = y.shape
    lib().orc_logsumexp_nary_bwd(_f(xs[i]), C.c_uint32(xs[i].shape[0]), C.c_uint(len(xs)), _f(y),
                                 _f(dy), C.c_size_t(n), C.c_uint32(bd), _f(dxi))
    return dxi


def pnls_fwd(x, ids):
    """x: (bd, rows). Returns (loss[bd], z[bd]); raises ValueError on a bad id."""
    bd, rows = x.shape
    loss = np.empty(bd, np.float32)
    z = np.empty(bd, np.float32)
    m = np.empty(bd, np.float32)
    rc = lib().orc_pnls_fwd(_f(x), C.c_uint32(rows), C.c_uint32(bd), _u(ids), _f(loss), _f(z), _f(m))
    if rc != 0:
        raise ValueError("Index error in PickNegLogSoftmax")
    return loss, z


def pnls_bwd(x, ids, z, dE, dx):
    bd, rows = x.shape
    lib().orc_pnls_bwd(_f(x), C.c_uint32(rows), C.c_uint32(bd), _u(ids), _f(z), _f(dE), _f(dx))
    return dx


# ---------------- norms ----------------
def weight_norm_fwd(w, g):
    y = np.empty_like(w)
    lib().orc_weight_norm_fwd(_f(w), C.c_float(g), _f(y), C.c_size_t(w.size))
    return y


def weight_norm_bwd(w, g, y, dy, i, dxi):
    lib().orc_weight_norm_bwd(_f(w), C.c_float(g), _f(y), _f(dy), C.c_uint(i), _f(dxi), C.c_size_t(w.size))
    return dxi


def moment_elems_fwd(x, order=1):
    bd, n = x.shape
    out = np.empty(bd, np.float32)
    lib().orc_moment_elems_fwd(_f(x), C.c_size_t(n), C.c_uint32(bd), C.c_uint(order), _f(out))
    return out


def moment_elems_bwd(x, order, dE, dx):
    bd, n = x.shape
    lib().orc_moment_elems_bwd(_f(x), C.c_size_t(n), C.c_uint32(bd), C.c_uint(order), _f(dE), _f(dx))
    return dx


def std_elems_fwd(x):
    bd, n = x.shape
    out = np.empty(bd, np.float32)
    lib().orc_std_elems_fwd(_f(x), C.c_size_t(n), C.c_uint32(bd), _f(out))
    return out


def std_elems_bwd(x, fx, dE, dx):
    bd, n = x.shape
    lib().orc_std_elems_bwd(_f(x), C.c_size_t(n), C.c_uint32(bd), _f(fx), _f(dE), _f(dx))
    return dx


def std_dim0_batch_fwd(x):
    bd, d1, d0 = x.shape
    out = np.empty(d1, np.float32)
    lib().orc_std_dim0_batch_fwd(_f(x), C.c_uint32(d0), C.c_uint32(d1), C.c_uint32(bd), _f(out))
    return out


def layer_norm_fwd(x, g, b):
    bd, n = x.shape
    y = np.empty_like(x)
    lib().orc_layer_norm_fwd(_f(x), _f(g), _f(b), _f(y), C.c_size_t(n), C.c_uint32(bd))
    return y


def layer_norm_bwd(x, g, dy, dx, dg, db):
    bd, n = x.shape
    lib().orc_layer_norm_bwd(_f(x), _f(g), _f(dy), _f(dx), _f(dg), _f(db), C.c_size_t(n), C.c_uint32(bd))
    return dx, dg, db


# ---------------- lookup ----------------
def lookup_fwd(table, ids, scale=1.0):
    """table: (V, E). Returns (n, E); raises ValueError on an out-of-range id."""
    V, E = table.shape
    out = np.empty((ids.size, E), np.float32)
    rc = lib().orc_lookup_fwd(_f(table), C.c_uint32(E), C.c_uint32(V), _u(ids), C.c_uint32(ids.size),
                              C.c_float(scale), _f(out))
    if rc != 0:
        raise ValueError("Out-of-bounds attempt to access index for LookupParameter")
    return out


def lookup_accumulate_grads(all_grads, ids, g):
    V, E = all_grads.shape
    lib().orc_lookup_accumulate_grads(_f(all_grads), C.c_uint32(E), _u(ids), C.c_uint32(ids.size), _f(g))
    return all_grads


# ---------------- LSTM nodes ----------------
def _xs_args(xs):
    ptrs = (f32p * len(xs))(*[_f(x) for x in xs])
    dims = (C.c_uint32 * len(xs))(*[x.shape[1] for x in xs])
    return ptrs, dims


def _mask(m):
    if m is None:
        return None, C.c_uint32(1)
    return _f(m), C.c_uint32(m.shape[0])


def lstm_gates_fwd(xs, h_tm1, Wx, Wh, b, mask_x=None, mask_h=None, forget_bias=1.0,
                   skip_matmul=False, packet=8):
    """xs: list of (B, I_k); h_tm1: (B, H); Wx: (I, 4H); Wh: (H, 4H); b: (4H,)."""
    B, H = h_tm1.shape
    I = Wx.shape[0]
    fx = np.empty((B, 4 * H), np.float32)
    ptrs, dims = _xs_args(xs)
    mx, mxbd = _mask(mask_x)
    mh, mhbd = _mask(mask_h)
    lib().orc_lstm_gates_fwd(ptrs, dims, C.c_uint(len(xs)), _f(h_tm1), _f(Wx), _f(Wh), _f(b), mx, mxbd,
                             mh, mhbd, C.c_uint32(H), C.c_uint32(I), C.c_uint32(B),
                             C.c_float(forget_bias), C.c_int(int(skip_matmul)), C.c_int(packet), _f(fx))
    return fx


def lstm_gates_bwd(xs, h_tm1, Wx, Wh, fx, dEdf, i, dxi, mask_x=None, mask_h=None):
    B, H = h_tm1.shape
    I = Wx.shape[0]
    ptrs, dims = _xs_args(xs)
    mx, mxbd = _mask(mask_x)
    mh, mhbd = _mask(mask_h)
    lib().orc_lstm_gates_bwd(ptrs, dims, C.c_uint(len(xs)), _f(h_tm1), _f(Wx), _f(Wh), mx, mxbd, mh,
                             mhbd, C.c_uint32(H), C.c_uint32(I), C.c_uint32(B), _f(fx), _f(dEdf),
                             C.c_uint(i), _f(dxi))
    return dxi


def lstm_c_fwd(c_tm1, gates):
    B, H = c_tm1.shape
    c = np.empty_like(c_tm1)
    lib().orc_lstm_c_fwd(_f(c_tm1), _f(gates), C.c_uint32(H), C.c_uint32(B), _f(c))
    return c


def lstm_c_bwd(c_tm1, gates, dc, i, dxi):
    B, H = c_tm1.shape
    lib().orc_lstm_c_bwd(_f(c_tm1), _f(gates), C.c_uint32(H), C.c_uint32(B), _f(dc), C.c_uint(i), _f(dxi))
    return dxi


def lstm_h_fwd(c_t, gates):
    B, H = c_t.shape
    h = np.empty_like(c_t)
    lib().orc_lstm_h_fwd(_f(c_t), _f(gates), C.c_uint32(H), C.c_uint32(B), _f(h))
    return h


def lstm_h_bwd(c_t, gates, dh, i, dxi):
    B, H = c_t.shape
    lib().orc_lstm_h_bwd(_f(c_t), _f(gates), C.c_uint32(H), C.c_uint32(B), _f(dh), C.c_uint(i), _f(dxi))
    return dxi


# ---------------- MatrixMultiply / AffineTransform ----------------
class OrcMat(C.Structure):
    _fields_ = [("v", f32p), ("rows", C.c_uint32), ("cols", C.c_uint32), ("bd", C.c_uint32)]


def _mats(xs):
    """xs: arrays shaped (bd, cols, rows) (column-major matrices, batch slowest); None = absent bias."""
    arr = (OrcMat * len(xs))()
    for k, x in enumerate(xs):
        if x is None:
            arr[k] = OrcMat(None, 0, 0, 1)
        else:
            assert x.ndim == 3 and x.dtype == np.float32 and x.flags.c_contiguous
            arr[k] = OrcMat(_f(x), x.shape[2], x.shape[1], x.shape[0])
    return arr


def affine_fwd(xs):
    """fx = xs[0] (tiled) + sum_k xs[2k+1] * xs[2k+2]."""
    rows = xs[1].shape[2]
    cols = xs[2].shape[1]
    bd = max(x.shape[0] for x in xs if x is not None)
    fx = np.empty((bd, cols, rows), np.float32)
    rc = lib().orc_affine_fwd(_mats(xs), C.c_uint(len(xs)), _f(fx), C.c_uint32(rows), C.c_uint32(cols), C.c_uint32(bd))
    if rc:
        raise ValueError("AffineTransform: bias broadcasting with a mini-batched bias is not implemented")
    return fx


def affine_bwd(xs, dEdf, i, dxi):
    bd, cols, rows = dEdf.shape
    rc = lib().orc_affine_bwd(_mats(xs), C.c_uint(len(xs)), _f(dEdf), C.c_uint32(rows), C.c_uint32(cols),
                              C.c_uint32(bd), C.c_uint(i), _f(dxi))
    if rc:
        raise ValueError("AffineTransform: bias broadcasting with a mini-batched bias is not implemented")
    return dxi


def matmul_fwd(a, b):
    return affine_fwd([None, a, b])


def matmul_bwd(a, b, dEdf, i, dxi):
    return affine_bwd([None, a, b], dEdf, i + 1, dxi)


def vanilla_lstm_builder_step(x, h_tm1, c_tm1, Wx, Wh, b, forget_bias=1.0):
    """One time step of one layer of VanillaLSTMBuilder::add_input_impl (dynet/lstm.cc:477-546; no dropout, no layer norm):
    the NON-fused graph  tmp = affine_transform({b, Wx, x, Wh, h_tm1});  four pick_range slices;  logistic / tanh;
    c = cmult(f, c_tm1) + cmult(i, g);  h = cmult(o, tanh(c)),  every node evaluated by its own oracle.
    x: (B, I), h_tm1 / c_tm1: (B, H) or None (no previous state), Wx: (I, 4H), Wh: (H, 4H), b: (4H,) -- C-order arrays of the
    column-major tensors.  Returns (h, c, nodes) with `nodes` the intermediate values by name."""
    B, I = x.shape
    H = Wx.shape[1] // 4
    xs = [b.reshape(1, 1, 4 * H), Wx.reshape(1, I, 4 * H), np.ascontiguousarray(x.reshape(B, 1, I))]
    if h_tm1 is not None:
        xs += [Wh.reshape(1, H, 4 * H), np.ascontiguousarray(h_tm1.reshape(B, 1, H))]
    tmp = affine_fwd(xs).reshape(B, 4 * H)
    a_i, a_f, a_o, a_g = (pick_range_fwd(tmp, k * H, (k + 1) * H, 0) for k in range(4))
    i_t = unary_fwd("logistic", a_i)
    f_t = unary_fwd("logistic", (a_f + np.float32(forget_bias)).astype(np.float32) if forget_bias != 0.0 else a_f)
    o_t = unary_fwd("logistic", a_o)
    g_t = unary_fwd("tanh", a_g)
    ig = cwise_fwd("cmult", i_t, g_t)
    c_t = sum_fwd([cwise_fwd("cmult", f_t, c_tm1), ig]) if h_tm1 is not None else ig
    tc = unary_fwd("tanh", c_t)
    h_t = cwise_fwd("cmult", o_t, tc)
    return h_t, c_t, dict(tmp=tmp, i=i_t, f=f_t, o=o_t, g=g_t, tanh_c=tc)


# ---------------- BiLSTM tagger, sentence by sentence ----------------
def _mat(a):
    """(rows, cols) parameter stored column-major -> the oracle's (bd=1, cols, rows) view of the same memory."""
    return a.reshape(1, a.shape[0], a.shape[1])


def tagger_fwdbwd(P, sents, tags):
    """The BiLSTM tagger of examples/tagger/train_tag-bilstm.cc:60-117 (without the input noise) the way the reference's CPU
    build runs it: one sentence at a time, node oracle by node oracle, batch size 1.  P: dict of parameters (numpy arrays,
    column-major tensors as (cols, rows)); sents / tags: lists of id lists.  Returns (summed loss, dict of gradients)."""
    H = P["b_f"].size // 4
    G = {k: np.zeros_like(v) for k, v in P.items()}
    loss = 0.0
    for sent, tg in zip(sents, tags):
        n = len(sent)
        states = {}
        for d in ("f", "r"):
            order = range(n) if d == "f" else range(n - 1, -1, -1)
            h = c = np.zeros((1, H), np.float32)
            for t in order:
                x = lookup_fwd(P["emb"], np.array([sent[t]], np.uint32))
                gates = lstm_gates_fwd([x], h, P["Wx_" + d], P["Wh_" + d], P["b_" + d])
                c_new = lstm_c_fwd(c, gates)
                h_new = lstm_h_fwd(c_new, gates)
                states[(d, t)] = (x, h, c, gates, c_new, h_new)
                h, c = h_new, c_new
        dh_tok = {}
        for t in range(n):
            hf, hr = states[("f", t)][5], states[("r", t)][5]
            xs1 = [P["thbias"].reshape(1, 1, -1), _mat(P["l2th"]), hf.reshape(1, 1, H), _mat(P["r2th"]), hr.reshape(1, 1, H)]
            pre = affine_fwd(xs1)
            th = unary_fwd("tanh", pre)
            xs2 = [P["tbias"].reshape(1, 1, -1), _mat(P["th2t"]), th]
            logits = affine_fwd(xs2)
            ids = np.array([tg[t]], np.uint32)
            l, z = pnls_fwd(logits.reshape(1, -1), ids)
            loss += float(l[0])
            dlog = pnls_bwd(logits.reshape(1, -1), ids, z, np.ones(1, np.float32), np.zeros((1, logits.size), np.float32))
            dlog = dlog.reshape(logits.shape)
            affine_bwd(xs2, dlog, 0, G["tbias"].reshape(1, 1, -1))
            affine_bwd(xs2, dlog, 1, _mat(G["th2t"]))
            dth = affine_bwd(xs2, dlog, 2, np.zeros_like(th))
            dpre = unary_bwd("tanh", pre, th, dth, np.zeros_like(pre))
            affine_bwd(xs1, dpre, 0, G["thbias"].reshape(1, 1, -1))
            affine_bwd(xs1, dpre, 1, _mat(G["l2th"]))
            affine_bwd(xs1, dpre, 3, _mat(G["r2th"]))
            dh_tok[("f", t)] = affine_bwd(xs1, dpre, 2, np.zeros((1, 1, H), np.float32)).reshape(1, H)
            dh_tok[("r", t)] = affine_bwd(xs1, dpre, 4, np.zeros((1, 1, H), np.float32)).reshape(1, H)
        for d in ("f", "r"):
            order = list(range(n)) if d == "f" else list(range(n - 1, -1, -1))
            dh_c = np.zeros((1, H), np.float32)
            dc_c = np.zeros((1, H), np.float32)
            for t in reversed(order):
                x, h_prev, c_prev, gates, c_new, h_new = states[(d, t)]
                dh = dh_tok[(d, t)] + dh_c
                dc = dc_c.copy()
                lstm_h_bwd(c_new, gates, dh, 0, dc)
                dg = np.zeros_like(gates)
                lstm_h_bwd(c_new, gates, dh, 1, dg)
                dc_c = lstm_c_bwd(c_prev, gates, dc, 0, np.zeros((1, H), np.float32))
                lstm_c_bwd(c_prev, gates, dc, 1, dg)
                dx = lstm_gates_bwd([x], h_prev, P["Wx_" + d], P["Wh_" + d], gates, dg, 0, np.zeros_like(x))
                dh_c = lstm_gates_bwd([x], h_prev, P["Wx_" + d], P["Wh_" + d], gates, dg, 1, np.zeros((1, H), np.float32))
                lstm_gates_bwd([x], h_prev, P["Wx_" + d], P["Wh_" + d], gates, dg, 2, G["Wx_" + d])
                lstm_gates_bwd([x], h_prev, P["Wx_" + d], P["Wh_" + d], gates, dg, 3, G["Wh_" + d])
                lstm_gates_bwd([x], h_prev, P["Wx_" + d], P["Wh_" + d], gates, dg, 4, G["b_" + d])
                lookup_accumulate_grads(G["emb"], np.array([sent[t]], np.uint32), dx)
    return loss, G


# ---------------- LSTM language model step ----------------
class LmDims(C.Structure):
    _fields_ = [(k, C.c_uint32) for k in ("V", "E", "H", "L", "T", "B")]


def lm_param_shapes(V, E, H, L):
    """(rows, cols) of every parameter tensor, in the order the oracle expects."""
    shapes = [(E, V)]
    for l in range(L):
        shapes += [(4 * H, E if l == 0 else H), (4 * H, H), (4 * H, 1)]
    shapes += [(V, H), (V, 1)]
    return shapes


def lstm_lm_fwdbwd(dims, params, grads, tokens, mask_x=None, mask_h=None, want_h=False):
    """params/grads: lists of flat float32 arrays (grads accumulated in place, or None).

    tokens: uint32 (T+1, B).  Returns (loss, h_states or None)."""
    V, E, H, L, T, B = dims
    d = LmDims(V, E, H, L, T, B)
    pp = (f32p * len(params))(*[_f(p) for p in params])
    gp = (f32p * len(params))(*[_f(g) for g in grads]) if grads is not None else None
    mxp = (f32p * L)(*[_f(m) for m in mask_x]) if mask_x is not None else None
    mhp = (f32p * L)(*[_f(m) for m in mask_h]) if mask_h is not None else None
    loss = C.c_float(0)
    h = np.empty((T, L, B, H), np.float32) if want_h else None
    rc = lib().orc_lstm_lm_fwdbwd(C.byref(d), pp, gp, _u(tokens), mxp, mhp, C.byref(loss),
                                  _f(h) if want_h else None)
    if rc != 0:
        raise ValueError("token id out of range")
    return loss.value, h


def sgd_update(params, grads, lr, clip=5.0):
    n = len(params)
    pp = (f32p * n)(*[_f(p) for p in params])
    gp = (f32p * n)(*[_f(g) for g in grads])
    sizes = (C.c_size_t * n)(*[p.size for p in params])
    return lib().orc_sgd_update(pp, gp, sizes, C.c_uint(n), C.c_float(lr), C.c_float(clip))


RULES = {"sgd": 0, "momentum": 1, "adagrad": 2, "adadelta": 3, "rmsprop": 4, "adam": 5, "amsgrad": 6}


def clip_scale(grads, clip_threshold):
    """Trainer::clip_gradients (dynet/training.cc:168-183): clip / ||g|| when the global norm exceeds clip."""
    gg = float(np.sqrt(sum(float((g.astype(np.float64) ** 2).sum()) for g in grads)))
    return np.float32(clip_threshold / gg) if clip_threshold > 0 and gg > clip_threshold else np.float32(1.0)


def trainer_update(rule, p, g, states, lr=0.1, gscale=1.0, wd=1.0, momentum=0.9, eps=1e-8, rho=0.95, beta_1=0.9,
                   beta_2=0.999, updates=0):
    """In-place update of p (and g, states) by the reference's rule; all arrays float32 of one size."""
    st = [_f(s) for s in states] + [None] * (3 - len(states))
    lib().orc_trainer_update(C.c_int(RULES[rule]), _f(p), _f(g), st[0], st[1], st[2], C.c_size_t(p.size), C.c_float(lr),
                             C.c_float(gscale), C.c_float(wd), C.c_float(momentum), C.c_float(eps), C.c_float(rho),
                             C.c_float(beta_1), C.c_float(beta_2), C.c_ulonglong(updates))
    return p


# ---------------- glue nodes (plain numpy; arrays are (bd, ..., d1, d0): batch first, C order == column-major) ----------------
def _axis(x, dim):
    """numpy axis of DyNet dimension `dim` of an array shaped (bd, d_{nd-1}, ..., d0)."""
    return x.ndim - 1 - dim


def pick_range_fwd(x, start, end, dim=0):
    """PickRange::forward_dev_impl (dynet/nodes-select.cc:229-240): slice [start, end) of dimension dim."""
    idx = [slice(None)] * x.ndim
    idx[_axis(x, dim)] = slice(start, end)
    return np.ascontiguousarray(x[tuple(idx)])


def pick_range_bwd(x_shape, start, end, dim, dEdf, dxi):
    """dynet/nodes-select.cc:243-259: dEdxi[slice] += dEdf."""
    idx = [slice(None)] * len(x_shape)
    idx[len(x_shape) - 1 - dim] = slice(start, end)
    dxi[tuple(idx)] += dEdf
    return dxi


def concatenate_fwd(xs, dimension=0):
    """Concatenate::forward_dev_impl (dynet/nodes-concat.cc:51-68); batch-1 inputs are broadcast."""
    bd = max(x.shape[0] for x in xs)
    parts = [np.broadcast_to(x, (bd,) + x.shape[1:]) for x in xs]
    return np.ascontiguousarray(np.concatenate(parts, axis=_axis(xs[0], dimension)))


def concatenate_bwd(xs, dimension, dEdf, i, dxi):
    """dynet/nodes-concat.cc:70-90: the slice of dEdf that came from argument i, summed over the batch if it was broadcast."""
    ax = _axis(xs[0], dimension)
    off = sum(x.shape[ax] for x in xs[:i])
    idx = [slice(None)] * dEdf.ndim
    idx[ax] = slice(off, off + xs[i].shape[ax])
    part = dEdf[tuple(idx)]
    if xs[i].shape[0] == dEdf.shape[0]:
        dxi += part
    else:
        dxi += part.astype(np.float64).sum(axis=0, keepdims=True).astype(np.float32)
    return dxi


def sum_fwd(xs):
    """Sum::forward_dev_impl (dynet/nodes-arith-sum.cc:66-114), float32 in the reference's grouping."""
    bd = max(x.shape[0] for x in xs)
    if all(x.shape[0] == xs[0].shape[0] for x in xs):
        def grp(g):
            s = g[0].copy()
            for a in g[1:]:
                s = s + a
            return s
        fx = grp(xs[:4])
        if len(xs) > 4:
            rem = (len(xs) - 4) % 4
            if rem:
                fx = fx + grp(xs[4:4 + rem])
            for q in range(4 + rem, len(xs), 4):
                fx = fx + grp(xs[q:q + 4])
        return fx
    fx = np.zeros((bd,) + xs[0].shape[1:], np.float32)
    for x in xs:
        fx = fx + x          # numpy broadcasts the batch-1 arguments
    return fx


def sum_bwd(dEdf, dxi):
    """dynet/nodes-arith-sum.cc:116-137."""
    if dxi.shape[0] == dEdf.shape[0]:
        dxi += dEdf
    else:
        dxi += dEdf.astype(np.float64).sum(axis=0, keepdims=True).astype(np.float32)
    return dxi


def sum_dim_fwd(x, dims, include_batch_dim=False):
    """SumDimension::forward_dev_impl (dynet/nodes-arith-sum.cc:198-217); long sums in double, rounded once."""
    axes = tuple(_axis(x, d) for d in dims) + ((0,) if include_batch_dim else ())
    y = x.astype(np.float64).sum(axis=axes, keepdims=True).astype(np.float32)
    # removed dimensions vanish from the Dim; the batch axis stays as 1
    keep = [0] + [a for a in range(1, x.ndim) if a not in axes]
    return np.ascontiguousarray(y.reshape([y.shape[a] for a in keep]))


def sum_dim_bwd(x_shape, dims, include_batch_dim, dEdf, dxi):
    """dynet/nodes-arith-sum.cc:219-248: dEdxi += broadcast(dEdf)."""
    nd = len(x_shape)
    shape = list(x_shape)
    for d in dims:
        shape[nd - 1 - d] = 1
    if include_batch_dim:
        shape[0] = 1
    dxi += dEdf.reshape(shape)
    return dxi


def squared_norm_fwd(x):
    """SquaredNorm::forward_dev_impl (dynet/nodes-norms.cc:30-34): one value per batch element."""
    return (x.reshape(x.shape[0], -1).astype(np.float64) ** 2).sum(axis=1).astype(np.float32).reshape(-1, 1)


def squared_norm_bwd(x, dEdf, dxi):
    """dynet/nodes-norms.cc:36-46: dEdxi += x * dEdf[b] * 2."""
    dxi += x * dEdf.reshape((-1,) + (1,) * (x.ndim - 1)) * np.float32(2.0)
    return dxi
