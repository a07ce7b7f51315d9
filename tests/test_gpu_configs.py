"""GPU tests at the shapes of the BASELINE configurations.

config 1 (the reference's CPU-runnable case): single-layer LSTM, I=128, H=256, B=32, T=50, loss = sum of squares of
all h_t -- every h_t, c_t, the loss and every gradient against the CPU oracle, driven node by node through the C ABI
exactly as DyNet's executor would (forward in order, backward once per argument into zeroed gradients).
configs 2 and 3 at FULL size: properties that need no CPU pass over 800 MB (row sums, picked-logit identity, mass
conservation of the scatter-add, round trips), plus a sampled comparison against the oracle on a slice."""
import ctypes as C

import numpy as np
import pytest

from util import TOL_REDUCE, assert_close, glorot, randn, rng, row_floor, zipf_ids

GEMM_FLOOR = 0.1   # states are O(1) sums of hundreds of products: see tests/test_gpu_parity.py

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def g():
    import gpu_util
    gpu_util.ctx()
    return gpu_util


@pytest.fixture(autouse=True)
def _release(g):
    yield
    g.release()


@pytest.fixture(scope="module")
def capi():
    from dynet_b200 import capi as c
    return c


def test_config1_builder_graph_pins_the_fused_chain(oracle, g, capi):
    """Config 1 the way the reference's CPU build runs it: VanillaLSTMBuilder's non-fused graph (dynet/lstm.cc:477-546:
    affine_transform -> 4 x pick_range -> logistic / tanh -> cmult / +) evaluated by the CPU oracle is the target.  On the
    device both forms run through the C ABI: the same node sequence (AffineTransform, PickRange, ConstantPlusX,
    LogisticSigmoid, Tanh, CwiseMultiply, Sum) and the fused chain (VanillaLSTMGates -> C -> H).  Both must give the
    builder graph's h_t and c_t; the bar between the two builders is the reference's own (tests/test-rnn.cc:155-184)."""
    r = rng(4321)
    I, H, B, T = 128, 256, 32, 8
    Wx, Wh, b = glorot(r, 4 * H, I), glorot(r, 4 * H, H), np.zeros(4 * H, np.float32)
    xs = [randn(r, B, I) for _ in range(T)]
    ctx = g.ctx()
    Wx_, Wh_, b_ = g.dev(Wx), g.dev(Wh), g.dev(b)
    tW = [g.T(Wx_, [4 * H, I], 1), g.T(Wh_, [4 * H, H], 1), g.T(b_, [4 * H], 1)]
    at = capi.LstmGatesAttrs(0, 0.0, 1.0)
    zeros = lambda n: g.dev(np.zeros((B, n), np.float32))
    h_ref, c_ref = np.zeros((B, H), np.float32), np.zeros((B, H), np.float32)
    hu, cu = zeros(H), zeros(H)          # device, non-fused node sequence
    hf, cf = zeros(H), zeros(H)          # device, fused chain
    for t in range(T):
        h_ref, c_ref, _ = oracle.vanilla_lstm_builder_step(xs[t], h_ref, c_ref, Wx, Wh, b)
        x_ = g.dev(xs[t])
        # non-fused graph on the device
        tmp = zeros(4 * H)
        ctx.fwd("affine_transform", [tW[2], tW[0], g.T(x_), tW[1], g.T(hu)], g.T(tmp))
        parts = []
        for k in range(4):
            pk = zeros(H)
            ctx.fwd("pick_range", [g.T(tmp)], g.T(pk), capi.PickRangeAttrs(k * H, (k + 1) * H, 0))
            parts.append(pk)
        af = zeros(H)
        ctx.fwd("constant_plus_x", [g.T(parts[1])], g.T(af), capi.ConstAttrs(1.0))
        it, ft, ot, gt = zeros(H), zeros(H), zeros(H), zeros(H)
        ctx.fwd("logistic", [g.T(parts[0])], g.T(it))
        ctx.fwd("logistic", [g.T(af)], g.T(ft))
        ctx.fwd("logistic", [g.T(parts[2])], g.T(ot))
        ctx.fwd("tanh", [g.T(parts[3])], g.T(gt))
        fc, ig, cn, tc, hn = zeros(H), zeros(H), zeros(H), zeros(H), zeros(H)
        ctx.fwd("cmult", [g.T(ft), g.T(cu)], g.T(fc))
        ctx.fwd("cmult", [g.T(it), g.T(gt)], g.T(ig))
        ctx.fwd("sum", [g.T(fc), g.T(ig)], g.T(cn))
        ctx.fwd("tanh", [g.T(cn)], g.T(tc))
        ctx.fwd("cmult", [g.T(ot), g.T(tc)], g.T(hn))
        hu, cu = hn, cn
        # fused chain on the device
        gates, cn2, hn2 = zeros(4 * H), zeros(H), zeros(H)
        ctx.fwd("vanilla_lstm_gates", [g.T(x_), g.T(hf)] + tW, g.T(gates), at)
        ctx.fwd("vanilla_lstm_c", [g.T(cf), g.T(gates)], g.T(cn2))
        ctx.fwd("vanilla_lstm_h", [g.T(cn2), g.T(gates)], g.T(hn2))
        hf, cf = hn2, cn2
        # The states are O(1) and every step adds its own rounding to the cell state it inherits: after a few steps the
        # node kernels (expf / tanhf of the device against the oracle's libm and rational sigmoid) sit at ~1e-6 absolute,
        # and the fused chain, whose gate activations come from ex2.approx / rcp.approx in the GEMM epilogue (sigmoid good to
        # 1.5e-6 relative), at 1 - 2e-6: both are held to 1e-5 of 0.25.
        for name, got, floor in (("non-fused graph", (hu, cu), 0.25), ("fused chain", (hf, cf), 0.25)):
            assert_close(g.host(got[0]), h_ref, 1e-5, floor=floor, what="h_%d, %s vs builder-graph oracle" % (t, name))
            assert_close(g.host(got[1]), c_ref, 1e-5, floor=floor, what="c_%d, %s vs builder-graph oracle" % (t, name))
    assert ctx.device_errors() == 0


def test_config1_single_layer_lstm_fwd_bwd(oracle, g, capi):
    r = rng(1234)
    I, H, B, T = 128, 256, 32, 50
    Wx, Wh, b = glorot(r, 4 * H, I), glorot(r, 4 * H, H), np.zeros(4 * H, np.float32)
    xs = [randn(r, B, I) for _ in range(T)]
    # ---- oracle: forward, loss, backward through time
    h = [np.zeros((B, H), np.float32)]
    c = [np.zeros((B, H), np.float32)]
    gates = []
    for t in range(T):
        gt = oracle.lstm_gates_fwd([xs[t]], h[-1], Wx, Wh, b)
        ct = oracle.lstm_c_fwd(c[-1], gt)
        gates.append(gt); c.append(ct); h.append(oracle.lstm_h_fwd(ct, gt))
    loss_ref = float(sum((ht.astype(np.float64) ** 2).sum() for ht in h[1:]))
    dWx, dWh, db = np.zeros_like(Wx), np.zeros_like(Wh), np.zeros_like(b)
    dxs = [np.zeros_like(x) for x in xs]
    dh = [2.0 * ht for ht in h]          # d(sum h^2)/dh_t, later steps add the recurrent part
    dc = [np.zeros((B, H), np.float32) for _ in range(T + 1)]
    for t in range(T, 0, -1):
        dg = np.zeros((B, 4 * H), np.float32)
        oracle.lstm_h_bwd(c[t], gates[t - 1], dh[t], 0, dc[t])
        oracle.lstm_h_bwd(c[t], gates[t - 1], dh[t], 1, dg)
        oracle.lstm_c_bwd(c[t - 1], gates[t - 1], dc[t], 0, dc[t - 1])
        oracle.lstm_c_bwd(c[t - 1], gates[t - 1], dc[t], 1, dg)
        for i, tgt in enumerate((dxs[t - 1], dh[t - 1], dWx, dWh, db)):
            oracle.lstm_gates_bwd([xs[t - 1]], h[t - 1], Wx, Wh, gates[t - 1], dg, i, tgt)
    # ---- device: the same node sequence through the C ABI
    ctx = g.ctx()
    at = capi.LstmGatesAttrs(0, 0.0, 1.0)
    dWx_, dWh_, db_ = g.dev(Wx), g.dev(Wh), g.dev(b)
    tW = [g.T(dWx_, [4 * H, I], 1), g.T(dWh_, [4 * H, H], 1), g.T(db_, [4 * H], 1)]
    x_ = [g.dev(x) for x in xs]
    h_ = [g.dev(np.zeros((B, H), np.float32))]
    c_ = [g.dev(np.zeros((B, H), np.float32))]
    g_ = []
    for t in range(T):
        gt, ct, ht = g.dev(np.zeros((B, 4 * H), np.float32)), g.dev(np.zeros((B, H), np.float32)), g.dev(np.zeros((B, H), np.float32))
        ctx.fwd("vanilla_lstm_gates", [g.T(x_[t]), g.T(h_[-1])] + tW, g.T(gt), at)
        ctx.fwd("vanilla_lstm_c", [g.T(c_[-1]), g.T(gt)], g.T(ct))
        ctx.fwd("vanilla_lstm_h", [g.T(ct), g.T(gt)], g.T(ht))
        g_.append(gt); c_.append(ct); h_.append(ht)
    for t in range(1, T + 1):
        assert_close(g.host(h_[t]), h[t], TOL_REDUCE, floor=0.1, what="h_%d" % t)
        assert_close(g.host(c_[t]), c[t], TOL_REDUCE, floor=0.1, what="c_%d" % t)
    loss = float(sum((g.host(ht).astype(np.float64) ** 2).sum() for ht in h_[1:]))
    assert abs(loss - loss_ref) <= 1e-4 * loss_ref
    gW = [g.dev(np.zeros_like(Wx)), g.dev(np.zeros_like(Wh)), g.dev(np.zeros_like(b))]
    tgW = [g.T(gW[0], [4 * H, I], 1), g.T(gW[1], [4 * H, H], 1), g.T(gW[2], [4 * H], 1)]
    dx_ = [g.dev(np.zeros_like(x)) for x in xs]
    dh_ = [g.dev(2.0 * g.host(ht)) for ht in h_]
    dc_ = [g.dev(np.zeros((B, H), np.float32)) for _ in range(T + 1)]
    for t in range(T, 0, -1):
        dg = g.dev(np.zeros((B, 4 * H), np.float32))
        xs_t = [g.T(x_[t - 1]), g.T(h_[t - 1])] + tW
        ctx.bwd("vanilla_lstm_h", [g.T(c_[t]), g.T(g_[t - 1])], g.T(h_[t]), g.T(dh_[t]), 0, g.T(dc_[t]))
        ctx.bwd("vanilla_lstm_h", [g.T(c_[t]), g.T(g_[t - 1])], g.T(h_[t]), g.T(dh_[t]), 1, g.T(dg))
        ctx.bwd("vanilla_lstm_c", [g.T(c_[t - 1]), g.T(g_[t - 1])], g.T(c_[t]), g.T(dc_[t]), 0, g.T(dc_[t - 1]))
        ctx.bwd("vanilla_lstm_c", [g.T(c_[t - 1]), g.T(g_[t - 1])], g.T(c_[t]), g.T(dc_[t]), 1, g.T(dg))
        for i, tgt in enumerate((g.T(dx_[t - 1]), g.T(dh_[t - 1]), tgW[0], tgW[1], tgW[2])):
            ctx.bwd("vanilla_lstm_gates", xs_t, g.T(g_[t - 1]), g.T(dg), i, tgt, at)
    for name, got, want in (("dWx", gW[0], dWx), ("dWh", gW[1], dWh), ("db", gW[2], db)):
        # per gate row: every row of dWx / dWh is held to its own magnitude (the bias gradient to 1 % of its largest entry)
        floor = row_floor(want, 0, rel=1e-3) if want.ndim == 2 else float(np.abs(want).max()) * 0.01
        assert_close(g.host(got), want, TOL_REDUCE, floor=floor, what=name + " (per-row scale)")
    for t in (0, 1, 25, 49):
        assert_close(g.host(dx_[t]), dxs[t], TOL_REDUCE, floor=row_floor(dxs[t], 1, rel=1e-3), what="dx_%d (per-column scale)" % t)
    assert ctx.device_errors() == 0


def test_config2_full_size_embedding_and_softmax_loss(oracle, g, capi):
    """V = 50,000, E = 512, N = 4,096 Zipf(1.1) ids: gather bit-exact, PickNegLogSoftmax over 50,000 x 4,096 logits."""
    import torch
    r = rng(2345)
    V, E, N = 50000, 512, 4096
    ctx = g.ctx()
    table = randn(r, V, E, scale=0.05)
    ids, tgt = zipf_ids(r, N, V), zipf_ids(r, N, V)
    tab_ = g.dev(table)
    x_ = torch.zeros(N, E, device="cuda")
    aux = torch.zeros(N, dtype=torch.int32, device="cuda")
    _, p = g.u32(ids)
    ctx.fwd("lookup", [], g.T(x_, [E], N), capi.LookupAttrs(tab_.data_ptr(), V, p, N, 1.0), aux.data_ptr())
    assert np.array_equal(g.host(x_), table[ids])                     # bit-exact gather at full size
    # logits = W x : 50,000 x 4,096 (819 MB) through the tensor-pipe GEMM
    W = torch.from_numpy(glorot(r, V, E)).cuda()                      # stored as Dim({V, E}) column-major
    logits = torch.empty(N, V, device="cuda")
    ctx.gemm(0, 0, V, N, E, W.data_ptr(), V, x_.data_ptr(), E, logits.data_ptr(), V, 0)
    ref_cols = (x_[:8].double() @ W.double()).float()                 # first 8 columns on the device in float64
    assert torch.allclose(logits[:8], ref_cols, rtol=1e-4, atol=1e-5)
    loss = torch.empty(N, device="cuda")
    paux = torch.zeros(3 * N, device="cuda")
    _, tp = g.u32(tgt)
    at = capi.PickAttrs(tp, N)
    ctx.fwd("pickneglogsoftmax", [g.T(logits, [V], N)], g.T(loss, [1], N), at, paux.data_ptr())
    z = paux[:N]
    ref_z = torch.logsumexp(logits.double(), dim=1)
    assert torch.allclose(z.double(), ref_z, rtol=1e-5, atol=1e-5)
    picked = logits[torch.arange(N, device="cuda"), torch.from_numpy(tgt.astype(np.int64)).cuda()]
    assert torch.allclose(loss, z - picked, rtol=0, atol=1e-6)        # loss = logsumexp - picked logit, index exact
    assert bool((loss > 0).all())
    # oracle on a slice (64 columns)
    l_ref, z_ref = oracle.pnls_fwd(g.host(logits[:64]).copy(), tgt[:64].copy())
    assert_close(g.host(loss[:64]), l_ref, TOL_REDUCE, what="pnls slice")
    # backward: columns of dx are softmax - onehot -> each column sums to 0 (to rounding of 50,000 terms)
    dE = torch.ones(N, device="cuda")
    dx = torch.zeros(N, V, device="cuda")
    ctx.bwd("pickneglogsoftmax", [g.T(logits, [V], N)], g.T(loss, [1], N), g.T(dE, [1], N), 0, g.T(dx, [V], N), at, paux.data_ptr())
    assert float(dx.sum(dim=1).abs().max()) < 1e-3
    assert float(dx.max()) <= 1.0 and float(dx.min()) >= -1.0
    # scatter-add into the embedding gradient: mass is conserved and rows of absent ids stay zero
    grad_x = torch.from_numpy(randn(r, N, E)).cuda()
    table_g = torch.zeros(V, E, device="cuda")
    ids_dev = torch.from_numpy(ids.view(np.int32)).cuda()
    ctx.lookup_accumulate_grads(ids, ids_dev.data_ptr(), grad_x.data_ptr(), table_g.data_ptr(), E, V)
    assert torch.allclose(table_g.sum(dim=0), grad_x.sum(dim=0), rtol=1e-4, atol=1e-3)
    absent = np.setdiff1d(np.arange(V), ids)
    assert float(table_g[torch.from_numpy(absent).cuda()].abs().max()) == 0.0
    want = oracle.lookup_accumulate_grads(np.zeros((V, E), np.float32), ids, g.host(grad_x))
    assert_close(g.host(table_g), want, TOL_REDUCE, floor=5.0, what="scatter-add full size")
    assert ctx.device_errors() == 0


@pytest.mark.parametrize("op", ["layer_norm", "weight_norm", "tanh", "logistic", "rectify", "elu", "softmax", "cmult"])
def test_config3_full_size_sweep(oracle, g, capi, op):
    """[1024, 4096] tensors: forward and backward of every op of the sweep against the oracle at full size."""
    r = rng(3456)
    R, Cn = 1024, 4096
    ctx = g.ctx()
    x = randn(r, R, Cn)
    up = randn(r, R, Cn)                      # fixed upstream gradient r: loss = sum(y * r)
    if op in ("tanh", "logistic", "rectify", "elu"):
        attrs = capi.EluAttrs(1.0, 1.0) if op == "elu" else None
        y_ref = oracle.unary_fwd(op, x)
        d_ref = oracle.unary_bwd(op, x, y_ref, up, np.zeros_like(x))
        x_, y_, d_ = g.dev(x), g.dev(np.zeros_like(x)), g.dev(np.zeros_like(x))
        ctx.fwd(op, [g.T(x_)], g.T(y_), attrs)
        ctx.bwd(op, [g.T(x_)], g.T(y_), g.T(g.dev(up)), 0, g.T(d_), attrs)
        assert_close(g.host(y_), y_ref, 1e-5, floor=2e-2, what=op)
        # (1 - y^2) amplifies a one-ulp difference of y near |y| = 1; compared against the O(1) scale of dy
        assert_close(g.host(d_), d_ref, 1e-5, floor=0.1, what=op + " bwd")
    elif op == "cmult":
        b = randn(r, R, Cn)
        y_ref = oracle.cwise_fwd("cmult", x, b)
        d_ref = oracle.cwise_bwd("cmult", x, b, up, 0, np.zeros_like(x))
        x_, b_, y_, d_ = g.dev(x), g.dev(b), g.dev(np.zeros_like(x)), g.dev(np.zeros_like(x))
        ctx.fwd("cmult", [g.T(x_), g.T(b_)], g.T(y_))
        ctx.bwd("cmult", [g.T(x_), g.T(b_)], g.T(y_), g.T(g.dev(up)), 0, g.T(d_))
        assert_close(g.host(y_), y_ref, 1e-5, what="cmult")
        assert_close(g.host(d_), d_ref, 1e-5, what="cmult bwd")
    elif op == "softmax":
        x3 = x.reshape(R, 1, Cn)
        y_ref = oracle.softmax_fwd(x3, 0)
        d_ref = oracle.softmax_bwd(y_ref, up.reshape(R, 1, Cn), np.zeros_like(x3), 0)
        x_, y_, d_ = g.dev(x), g.dev(np.zeros_like(x)), g.dev(np.zeros_like(x))
        at = capi.DimAttrs(0)
        ctx.fwd("softmax", [g.T(x_)], g.T(y_), at)
        ctx.bwd("softmax", [g.T(x_)], g.T(y_), g.T(g.dev(up)), 0, g.T(d_), at)
        yh = g.host(y_)
        assert np.abs(yh.sum(axis=1) - 1.0).max() < 1e-5
        assert_close(yh, y_ref.reshape(R, Cn), TOL_REDUCE, floor=1e-4, what="softmax")
        assert_close(g.host(d_), d_ref.reshape(R, Cn), TOL_REDUCE, floor=1e-3, what="softmax bwd")
    elif op == "layer_norm":
        gain, bias = r.uniform(0.5, 1.5, Cn).astype(np.float32), randn(r, Cn, scale=0.1)
        y_ref = oracle.layer_norm_fwd(x, gain, bias)
        dx, dg, db = oracle.layer_norm_bwd(x, gain, up, np.zeros_like(x), np.zeros_like(gain), np.zeros_like(bias))
        xs = [g.T(g.dev(x)), g.T(g.dev(gain), [Cn], 1), g.T(g.dev(bias), [Cn], 1)]
        y_ = g.dev(np.zeros_like(x))
        ctx.fwd("layer_norm", xs, g.T(y_))
        assert_close(g.host(y_), y_ref, TOL_REDUCE, floor=1e-2, what="layer_norm")
        up_ = g.dev(up)
        for i, want, dims in ((0, dx, None), (1, dg, [Cn]), (2, db, [Cn])):
            d_ = g.dev(np.zeros_like(want))
            ctx.bwd("layer_norm", xs, g.T(y_), g.T(up_), i, g.T(d_) if dims is None else g.T(d_, dims, 1))
            assert_close(g.host(d_), want, TOL_REDUCE, floor=float(np.abs(want).max()) * 0.02, what="layer_norm bwd %d" % i)
    else:  # weight_norm over the whole [1024, 4096] tensor
        w = x.reshape(-1)
        gv = np.array([r.uniform(0.5, 1.5)], np.float32)
        y_ref = oracle.weight_norm_fwd(w, float(gv[0]))
        dw = oracle.weight_norm_bwd(w, float(gv[0]), y_ref, up.reshape(-1), 0, np.zeros_like(w))
        dgr = oracle.weight_norm_bwd(w, float(gv[0]), y_ref, up.reshape(-1), 1, np.zeros(1, np.float32))
        xs = [g.T(g.dev(w), [R, Cn], 1), g.T(g.dev(gv), [1], 1)]
        y_ = g.dev(np.zeros_like(w))
        ctx.fwd("weight_norm", xs, g.T(y_, [R, Cn], 1))
        assert_close(g.host(y_), y_ref, TOL_REDUCE, floor=1e-5, what="weight_norm")
        d_ = g.dev(np.zeros_like(w))
        ctx.bwd("weight_norm", xs, g.T(y_, [R, Cn], 1), g.T(g.dev(up.reshape(-1)), [R, Cn], 1), 0, g.T(d_, [R, Cn], 1))
        assert_close(g.host(d_), dw, TOL_REDUCE, floor=1e-5, what="weight_norm bwd w")
        dg_ = g.dev(np.zeros(1, np.float32))
        ctx.bwd("weight_norm", xs, g.T(y_, [R, Cn], 1), g.T(g.dev(up.reshape(-1)), [R, Cn], 1), 1, g.T(dg_, [1], 1))
        assert_close(g.host(dg_), dgr, TOL_REDUCE, floor=float(abs(dgr[0])) + 1.0, what="weight_norm bwd g")
    assert ctx.device_errors() == 0
