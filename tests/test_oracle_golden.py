"""Pins the CPU oracle to the known answers in the reference's own test-suite
(tests/test-rnn.cc, tests/test-nodes.cc, tests/python/test.py), and checks its
backward functions by the reference's finite-difference rule
(dynet/grad-check.cc:15-97: central difference, alpha 5e-3, 1% tolerance)."""
import json
import os

import numpy as np
import pytest

from util import assert_close, rng, randn

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_known_answers.json")))


def f32(v):
    return np.asarray(v, np.float32)


def check_known(got, case):
    want = np.asarray(case["expect"], np.float64)
    got = np.asarray(got, np.float64).ravel()
    for g, w in zip(got, want):
        if w == 0.0:
            assert abs(g) <= case.get("tol_abs_zero", 1e-6)
        else:
            assert abs(g - w) <= case["tol_rel"] * abs(w) * 1.0000001 + 0, (g, w)


def test_lstm_node_h_fwd(oracle):
    c = GOLD["lstm_node_h_fwd"]
    H, B = c["H"], c["B"]
    h = oracle.lstm_h_fwd(f32(c["c_t"]).reshape(B, H), f32(c["gates_t"]).reshape(B, 4 * H))
    check_known(h, c)


def test_lstm_node_c_fwd(oracle):
    c = GOLD["lstm_node_c_fwd"]
    H, B = c["H"], c["B"]
    out = oracle.lstm_c_fwd(f32(c["c_tm1"]).reshape(B, H), f32(c["gates_t"]).reshape(B, 4 * H))
    check_known(out, c)


@pytest.mark.parametrize("packet", [0, 8])
@pytest.mark.parametrize("name", ["lstm_node_gates_fwd", "lstm_node_gates_dropout_fwd"])
def test_lstm_node_gates_fwd(oracle, name, packet):
    c = GOLD[name]
    I, H, B = c["I"], c["H"], c["B"]
    mx = f32(c["mask_x"]).reshape(B, I) if "mask_x" in c else None
    mh = f32(c["mask_h"]).reshape(B, H) if "mask_h" in c else None
    g = oracle.lstm_gates_fwd([f32(c["x_t"]).reshape(B, I)], f32(c["h_tm1"]).reshape(B, H),
                              f32(c["Wx"]).reshape(I, 4 * H), f32(c["Wh"]).reshape(H, 4 * H),
                              f32(c["b"]), mx, mh, packet=packet)
    check_known(g, c)


def test_std_dim_value(oracle):
    c = GOLD["std_dim_value"]
    x = f32(c["x"]).reshape(c["bd"], c["dims"][1], c["dims"][0])
    y = oracle.std_dim0_batch_fwd(x)
    z = float(np.float32(y.sum(dtype=np.float32) / np.float32(3.0)))
    assert abs(z - c["expect_mean_of_std_dim0_batch"]) <= c["tol_rel"] * c["expect_mean_of_std_dim0_batch"]


def test_layer_norm_forward(oracle):
    c = GOLD["layer_norm_forward"]
    y = oracle.layer_norm_fwd(f32(c["x"]).reshape(1, 3), f32(c["g"]), f32(c["b"]))
    assert abs(float(y.sum() / 3.0)) < c["expect_abs_mean_lt"]
    std = float(np.sqrt((y.astype(np.float64) ** 2).sum() / 3.0))
    assert abs(std - c["expect_std"]) <= c["tol_rel"]


def test_python_layer_norm_closed_form(oracle):
    v = np.arange(10).astype(np.float32)
    y = oracle.layer_norm_fwd(v.reshape(1, 10), v.copy(), v.copy())
    want = v / v.std() * (v - v.mean()) + v
    assert np.allclose(y.ravel(), want)


def test_weight_norm_forward(oracle):
    c = GOLD["weight_norm_forward"]
    y = oracle.weight_norm_fwd(f32(c["w"]), c["g"])
    norm = float(np.sqrt((y.astype(np.float64) ** 2).sum()))
    assert abs(norm - c["expect_norm"]) <= c["tol_rel"] * c["expect_norm"]


def test_sigmoid_packet_vs_scalar(oracle):
    L = oracle.lib()
    for x in np.linspace(-20, 20, 801):
        p, s = L.orc_sigmoid_packet(float(x)), L.orc_sigmoid_scalar(float(x))
        assert abs(p - s) <= 3e-7, (x, p, s)


# ---------------------------------------------------------------- gradient checks
def fd_check(f, xs, backward, alpha=5e-3, tol=0.01):
    """f(xs) -> scalar (float64 of float32 math); backward(i) -> analytic grad of arg i."""
    for i, x in enumerate(xs):
        g = backward(i)
        if g is None:
            continue
        flat = x.reshape(-1)
        gf = g.reshape(-1)
        for k in range(flat.size):
            old = flat[k]
            flat[k] = old - alpha
            lo = f(xs)
            flat[k] = old + alpha
            hi = f(xs)
            flat[k] = old
            num = (hi - lo) / (2 * alpha)
            fdiff = abs(num - gf[k])
            m = max(abs(num), abs(gf[k]))
            if fdiff > tol and m > 0 and fdiff / m > tol:
                raise AssertionError("arg %d elem %d: numeric %g analytic %g" % (i, k, num, gf[k]))


def sq(y):
    return float((y.astype(np.float64) ** 2).sum())


def test_lstm_gates_gradient(oracle):
    # shapes of tests/test-rnn.cc:341-357 (I=5, H=3, B=2) plus dropout masks and two inputs
    r = rng(7)
    I1, I2, H, B = 3, 2, 3, 2
    xs = [randn(r, B, I1, scale=0.5), randn(r, B, I2, scale=0.5)]
    h = randn(r, B, H, scale=0.5)
    Wx = randn(r, I1 + I2, 4 * H, scale=0.4)
    Wh = randn(r, H, 4 * H, scale=0.4)
    b = randn(r, 4 * H, scale=0.3)
    for masks in (False, True):
        mx = (r.random((B, I1 + I2)) > 0.3).astype(np.float32) * 1.25 if masks else None
        mh = (r.random((1, H)) > 0.3).astype(np.float32) * 1.25 if masks else None
        args = xs + [h, Wx, Wh, b]

        def f(a):
            return sq(oracle.lstm_gates_fwd(a[:2], a[2], a[3], a[4], a[5], mx, mh))

        fx = oracle.lstm_gates_fwd(xs, h, Wx, Wh, b, mx, mh)
        dE = 2 * fx

        def bw(i):
            d = np.zeros_like(args[i])
            return oracle.lstm_gates_bwd(xs, h, Wx, Wh, fx, dE, i, d, mx, mh)

        fd_check(f, args, bw)


def test_lstm_c_h_gradient(oracle):
    r = rng(8)
    H, B = 3, 2
    c = randn(r, B, H, scale=0.5)
    gates = randn(r, B, 4 * H, scale=0.5)
    args = [c, gates]
    fd_check(lambda a: sq(oracle.lstm_c_fwd(a[0], a[1])), args,
             lambda i: oracle.lstm_c_bwd(c, gates, 2 * oracle.lstm_c_fwd(c, gates), i, np.zeros_like(args[i])))
    fd_check(lambda a: sq(oracle.lstm_h_fwd(a[0], a[1])), args,
             lambda i: oracle.lstm_h_bwd(c, gates, 2 * oracle.lstm_h_fwd(c, gates), i, np.zeros_like(args[i])))


@pytest.mark.parametrize("name", ["tanh", "logistic", "rectify", "elu"])
def test_unary_gradient(oracle, name):
    r = rng(9)
    x = randn(r, 13) + 0.05
    y = oracle.unary_fwd(name, x)
    fd_check(lambda a: sq(oracle.unary_fwd(name, a[0])), [x],
             lambda i: oracle.unary_bwd(name, x, y, 2 * y, np.zeros_like(x)))


@pytest.mark.parametrize("op", ["cmult", "csum", "cdiv"])
def test_cwise_broadcast_gradient(oracle, op):
    r = rng(10)
    a = randn(r, 3, 2, 4) + 2.0       # bd=3, d1=2, d0=4
    b = randn(r, 1, 1, 4) + 2.0       # broadcast over d1 and batch
    y = oracle.cwise_fwd(op, a, b)
    args = [a, b]
    fd_check(lambda v: sq(oracle.cwise_fwd(op, v[0], v[1])), args,
             lambda i: oracle.cwise_bwd(op, a, b, 2 * y, i, np.zeros_like(args[i])))


@pytest.mark.parametrize("dimension", [0, 1])
def test_softmax_gradient(oracle, dimension):
    r = rng(11)
    x = randn(r, 2, 3, 4)
    w = randn(r, 2, 3, 4)
    y = oracle.softmax_fwd(x, dimension)
    fd_check(lambda a: float((oracle.softmax_fwd(a[0], dimension).astype(np.float64) * w).sum()), [x],
             lambda i: oracle.softmax_bwd(y, w, np.zeros_like(x), dimension))


def test_logsoftmax_logsumexp_pnls_gradient(oracle):
    r = rng(12)
    x = randn(r, 2, 3, 5)
    w = randn(r, 2, 3, 5)
    y = oracle.log_softmax_fwd(x)
    fd_check(lambda a: float((oracle.log_softmax_fwd(a[0]).astype(np.float64) * w).sum()), [x],
             lambda i: oracle.log_softmax_bwd(y, w, np.zeros_like(x)))
    for axis in (0, 1):
        z, _ = oracle.logsumexp_dim_fwd(x, axis)
        wz = randn(r, *z.shape)
        fd_check(lambda a: float((oracle.logsumexp_dim_fwd(a[0], axis)[0].astype(np.float64) * wz).sum()), [x],
                 lambda i: oracle.logsumexp_dim_bwd(x, z, wz, np.zeros_like(x), axis))
    xv = randn(r, 4, 6)
    ids = np.array([0, 5, 2, 2], np.uint32)
    loss, z = oracle.pnls_fwd(xv, ids)
    dE = randn(r, 4)
    fd_check(lambda a: float((oracle.pnls_fwd(a[0], ids)[0].astype(np.float64) * dE).sum()), [xv],
             lambda i: oracle.pnls_bwd(xv, ids, z, dE, np.zeros_like(xv)))
    with pytest.raises(ValueError):
        oracle.pnls_fwd(xv, np.array([0, 6, 2, 2], np.uint32))


def test_logsumexp_nary_gradient(oracle):
    r = rng(13)
    xs = [randn(r, 3, 4), randn(r, 1, 4), randn(r, 3, 4)]
    y = oracle.logsumexp_nary_fwd(xs)
    w = randn(r, 3, 4)
    fd_check(lambda a: float((oracle.logsumexp_nary_fwd(a).astype(np.float64) * w).sum()), xs,
             lambda i: oracle.logsumexp_nary_bwd(xs, i, y, w, np.zeros_like(xs[i])))


def test_norm_gradients(oracle):
    r = rng(14)
    x = randn(r, 3, 7)
    g = (r.uniform(0.5, 1.5, 7)).astype(np.float32)
    b = randn(r, 7, scale=0.1)
    w = randn(r, 3, 7)
    args = [x, g, b]

    def bw(i):
        dx, dg, db = np.zeros_like(x), np.zeros_like(g), np.zeros_like(b)
        oracle.layer_norm_bwd(x, g, w, dx, dg, db)
        return [dx, dg, db][i]

    fd_check(lambda a: float((oracle.layer_norm_fwd(a[0], a[1], a[2]).astype(np.float64) * w).sum()), args, bw)

    wt = randn(r, 12) + 0.3
    gs = np.array([1.3], np.float32)
    wy = randn(r, 12)
    y = oracle.weight_norm_fwd(wt, float(gs[0]))
    a2 = [wt, gs]
    fd_check(lambda a: float((oracle.weight_norm_fwd(a[0], float(a[1][0])).astype(np.float64) * wy).sum()), a2,
             lambda i: oracle.weight_norm_bwd(wt, float(gs[0]), y, wy, i, np.zeros_like(a2[i])))

    for order in (1, 2, 3):
        dE = randn(r, 3)
        fd_check(lambda a: float((oracle.moment_elems_fwd(a[0], order).astype(np.float64) * dE).sum()), [x],
                 lambda i: oracle.moment_elems_bwd(x, order, dE, np.zeros_like(x)))
    dE = randn(r, 3)
    s = oracle.std_elems_fwd(x)
    fd_check(lambda a: float((oracle.std_elems_fwd(a[0]).astype(np.float64) * dE).sum()), [x],
             lambda i: oracle.std_elems_bwd(x, s, dE, np.zeros_like(x)))


def test_lookup(oracle):
    r = rng(15)
    table = randn(r, 9, 4)
    ids = np.array([3, 3, 0, 8, 3], np.uint32)
    out = oracle.lookup_fwd(table, ids)
    assert np.array_equal(out, table[ids])
    with pytest.raises(ValueError):
        oracle.lookup_fwd(table, np.array([9], np.uint32))
    g = randn(r, 5, 4)
    acc = np.zeros_like(table)
    oracle.lookup_accumulate_grads(acc, ids, g)
    want = np.zeros_like(table)
    for b, i in enumerate(ids):
        want[i] += g[b]
    assert np.array_equal(acc, want)


def test_fused_chain_equals_unfused_builder_math(oracle):
    """tests/test-rnn.cc:155-184 pins the fused node chain to VanillaLSTMBuilder's
    affine_transform/pick_range/logistic/tanh/cmult graph (dynet/lstm.cc:477-546)
    within 1e-5 relative over three steps; redo that with independent numpy math."""
    r = rng(16)
    I, H, B, T = 4, 3, 2, 3
    Wx, Wh, b = randn(r, I, 4 * H, scale=0.5), randn(r, H, 4 * H, scale=0.5), randn(r, 4 * H, scale=0.2)
    h = np.zeros((B, H), np.float32)
    c = np.zeros((B, H), np.float32)
    h2, c2 = h.astype(np.float64), c.astype(np.float64)
    sig = lambda v: 1 / (1 + np.exp(-v))
    for t in range(T):
        x = randn(r, B, I)
        g = oracle.lstm_gates_fwd([x], h, Wx, Wh, b)
        c = oracle.lstm_c_fwd(c, g)
        h = oracle.lstm_h_fwd(c, g)
        a = b.astype(np.float64) + x.astype(np.float64) @ Wx.astype(np.float64) + h2 @ Wh.astype(np.float64)
        i_, f_, o_, g_ = sig(a[:, :H]), sig(a[:, H:2 * H] + 1.0), sig(a[:, 2 * H:3 * H]), np.tanh(a[:, 3 * H:])
        c2 = f_ * c2 + i_ * g_
        h2 = o_ * np.tanh(c2)
        assert_close(h, h2, 1e-5, floor=1e-2, what="h_%d" % t)
        assert_close(c, c2, 1e-5, floor=1e-2, what="c_%d" % t)


def test_builder_graph_oracle_equals_fused_chain_oracle(oracle):
    """The restatement of VanillaLSTMBuilder's non-fused graph (dynet/lstm.cc:477-546), node oracle by node oracle,
    against the fused-node chain, at the reference test's bar (tests/test-rnn.cc:155-184: 1e-5 relative) and at the
    sizes of the single-layer benchmark configuration."""
    for (I, H, B, T) in [(3, 5, 1, 3), (128, 256, 32, 6)]:
        r = rng(17 + I)
        a = np.sqrt(6.0 / (4 * H + I))
        Wx = r.uniform(-a, a, (I, 4 * H)).astype(np.float32)
        a = np.sqrt(6.0 / (4 * H + H))
        Wh = r.uniform(-a, a, (H, 4 * H)).astype(np.float32)
        b = np.zeros(4 * H, np.float32)
        h = np.zeros((B, H), np.float32); c = np.zeros((B, H), np.float32)
        hb, cb = h.copy(), c.copy()
        for t in range(T):
            x = randn(r, B, I)
            g = oracle.lstm_gates_fwd([x], h, Wx, Wh, b)
            c = oracle.lstm_c_fwd(c, g)
            h = oracle.lstm_h_fwd(c, g)
            hb, cb, _ = oracle.vanilla_lstm_builder_step(x, hb, cb, Wx, Wh, b)
            # (states are O(1) sums of O(1) products: one float32 ulp of those, ~1e-7, is the floor of any agreement)
            assert_close(h, hb, 1e-5, floor=0.1, what="h_%d builder graph vs fused chain" % t)
            assert_close(c, cb, 1e-5, floor=0.1, what="c_%d builder graph vs fused chain" % t)


# ---------------------------------------------------------------- MatrixMultiply / AffineTransform
def _np_affine(xs):
    """float64 numpy statement of bias + sum A_k B_k with DyNet's batch rules (arrays are (bd, cols, rows))."""
    bd = max(x.shape[0] for x in xs if x is not None)
    rows, cols = xs[1].shape[2], xs[2].shape[1]
    y = np.zeros((bd, cols, rows))
    if xs[0] is not None:
        y += np.resize(xs[0].astype(np.float64).ravel(), y.size).reshape(y.shape)
    for k in range(1, len(xs), 2):
        for b in range(bd):
            A = xs[k][b % xs[k].shape[0]].astype(np.float64).T          # rows x K
            Bm = xs[k + 1][b % xs[k + 1].shape[0]].astype(np.float64).T  # K x cols
            y[b] += (A @ Bm).T
    return y


# shapes of tests/test-nodes.cc:431-505 (multiply, multiply_batch, affine, affine_batch, affine_batch_col,
# affine_batch2, affine_batch3) as (bd, cols, rows) triples for {bias, A, B}; None = MatrixMultiply
AFFINE_CASES = {
    "multiply": [None, (1, 1, 3), (1, 3, 1)],
    "multiply_batch": [None, (1, 1, 3), (2, 3, 1)],
    "affine": [(1, 1, 3), (1, 1, 3), (1, 1, 1)],
    "affine_batch": [(1, 1, 3), (2, 1, 3), (1, 1, 1)],
    "affine_batch_col": [(1, 3, 1), (1, 1, 1), (2, 3, 1)],
    "affine_batch2": [(2, 3, 1), (1, 1, 1), (1, 3, 1)],
    "affine_batch3": [(1, 1, 3), (1, 3, 3), (2, 1, 3)],
    "two_products": [(1, 1, 4), (1, 3, 4), (3, 2, 3), (1, 5, 4), (3, 2, 5)],
    "both_batched": [(1, 1, 4), (3, 2, 4), (3, 5, 2)],
}


@pytest.mark.parametrize("case", sorted(AFFINE_CASES))
def test_affine_matmul_value_and_gradient(oracle, case):
    r = rng(sum(map(ord, case)))
    xs = [None if s is None else randn(r, *s) + 0.3 for s in AFFINE_CASES[case]]
    y = oracle.affine_fwd(xs)
    assert_close(y, _np_affine(xs), 1e-5, floor=1.0, what=case)
    live = [k for k, x in enumerate(xs) if x is not None]

    def f(vals):
        full = list(xs)
        for k, v in zip(live, vals):
            full[k] = v
        return sq(oracle.affine_fwd(full))

    fd_check(f, [xs[k] for k in live],
             lambda j: oracle.affine_bwd(xs, 2 * y, live[j], np.zeros_like(xs[live[j]])))


def test_affine_rejects_batched_bias_broadcast(oracle):
    r = rng(5)
    xs = [randn(r, 2, 1, 3), randn(r, 1, 4, 3), randn(r, 2, 5, 4)]   # bias {3} x2 under a {3,5} x2 result
    with pytest.raises(ValueError):
        oracle.affine_fwd(xs)


# ---------------------------------------------------------------- trainer update rules
# defaults of the reference's constructors (dynet/training.h:318, :405, :448, :489, :531, :573, :619)
TRAINER_DEFAULTS = {
    "sgd": dict(lr=0.1), "momentum": dict(lr=0.01, momentum=0.9), "adagrad": dict(lr=0.1, eps=1e-20),
    "adadelta": dict(lr=1.0, eps=1e-6, rho=0.95), "rmsprop": dict(lr=0.1, eps=1e-20, rho=0.95),
    "adam": dict(lr=0.001, beta_1=0.9, beta_2=0.999, eps=1e-8), "amsgrad": dict(lr=0.001, beta_1=0.9, beta_2=0.999, eps=1e-8),
}
N_STATES = {"sgd": 0, "momentum": 1, "adagrad": 1, "adadelta": 2, "rmsprop": 1, "adam": 2, "amsgrad": 3}


@pytest.mark.parametrize("rule", sorted(TRAINER_DEFAULTS))
def test_trainer_direction(oracle, rule):
    """tests/test-trainers.cc:53-85: one update on z = ones . x (gradient = ones) must lower z."""
    p = f32([1.1, -2.2, 3.3])
    g = np.ones(3, np.float32)
    states = [np.zeros(3, np.float32) for _ in range(N_STATES[rule])]
    before = float(p.sum())
    oracle.trainer_update(rule, p, g, states, gscale=oracle.clip_scale([g], 5.0), **TRAINER_DEFAULTS[rule])
    assert float(p.sum()) < before


def test_momentum_velocity_known_answer(oracle):
    """tests/test-trainers.cc:141-155: MomentumSGDTrainer(pc, 1.0), gradient of ones -> velocity exactly -1."""
    p, g, v = np.zeros(3, np.float32), np.ones(3, np.float32), np.zeros(3, np.float32)
    oracle.trainer_update("momentum", p, g, [v], lr=1.0, momentum=0.9)
    assert np.array_equal(v, -np.ones(3, np.float32))
    assert np.array_equal(p, -np.ones(3, np.float32))


def test_trainer_rules_against_float64(oracle):
    r = rng(321)
    n = 257
    for rule, hp in TRAINER_DEFAULTS.items():
        p, g = randn(r, n), randn(r, n)
        st = [np.abs(randn(r, n)) * 0.1 for _ in range(N_STATES[rule])]
        p0, g0, s0 = p.astype(np.float64), g.astype(np.float64) * 0.5, [s.astype(np.float64) for s in st]
        oracle.trainer_update(rule, p, g, st, gscale=0.5, wd=1.0, updates=3, **hp)
        lr = hp["lr"]
        if rule == "sgd":
            want = p0 - g0 * lr
        elif rule == "momentum":
            want = p0 + (s0[0] * hp["momentum"] - g0 * lr)
        elif rule == "adagrad":
            want = p0 - lr * g0 / np.sqrt(s0[0] + g0 * g0 + hp["eps"])
        elif rule == "rmsprop":
            want = p0 - lr * g0 / np.sqrt(s0[0] * hp["rho"] + g0 * g0 * (1 - hp["rho"]) + hp["eps"])
        elif rule == "adadelta":
            hg = s0[0] * hp["rho"] + g0 * g0 * (1 - hp["rho"])
            want = p0 - g0 * np.sqrt(s0[1] + hp["eps"]) / np.sqrt(hg + hp["eps"])
        else:
            m = s0[0] * hp["beta_1"] + g0 * (1 - hp["beta_1"])
            v = s0[1] * hp["beta_2"] + g0 * g0 * (1 - hp["beta_2"])
            if rule == "amsgrad":
                v = np.maximum(s0[2], v)
            lr_t = lr * np.sqrt(1 - hp["beta_2"] ** 4) / (1 - hp["beta_1"] ** 4)
            want = p0 - m / (np.sqrt(v) + hp["eps"]) * lr_t
        assert_close(p, want, 1e-5, floor=1.0, what=rule)


# ---------------------------------------------------------------- glue nodes
def test_glue_nodes_gradients(oracle):
    """Finite-difference rule of dynet/grad-check.cc on the numpy restatements of PickRange, Concatenate, Sum,
    SumDimension and SquaredNorm (the reference checks them the same way, tests/test-nodes.cc)."""
    r = rng(42)
    x = randn(r, 2, 3, 5)
    y = oracle.pick_range_fwd(x, 1, 4, 0)
    assert y.shape == (2, 3, 3)
    fd_check(lambda v: sq(oracle.pick_range_fwd(v[0], 1, 4, 0)), [x],
             lambda i: oracle.pick_range_bwd(x.shape, 1, 4, 0, 2 * y, np.zeros_like(x)))
    a, b = randn(r, 3, 2, 4), randn(r, 1, 5, 4)
    c = oracle.concatenate_fwd([a, b], 1)
    assert c.shape == (3, 7, 4)
    args = [a, b]
    fd_check(lambda v: sq(oracle.concatenate_fwd(v, 1)), args,
             lambda i: oracle.concatenate_bwd(args, 1, 2 * c, i, np.zeros_like(args[i])))
    xs = [randn(r, 2, 6) for _ in range(6)] + [randn(r, 1, 6)]
    s = oracle.sum_fwd(xs)
    fd_check(lambda v: sq(oracle.sum_fwd(v)), xs, lambda i: oracle.sum_bwd(2 * s, np.zeros_like(xs[i])))
    t = randn(r, 3, 4, 5)
    for dims, ib in [((0,), False), ((1,), True), ((0, 1), False), ((), True)]:
        z = oracle.sum_dim_fwd(t, dims, ib)
        fd_check(lambda v: sq(oracle.sum_dim_fwd(v[0], dims, ib)), [t],
                 lambda i: oracle.sum_dim_bwd(t.shape, dims, ib, 2 * z, np.zeros_like(t)))
    n = oracle.squared_norm_fwd(t)
    fd_check(lambda v: sq(oracle.squared_norm_fwd(v[0])), [t],
             lambda i: oracle.squared_norm_bwd(t, 2 * n, np.zeros_like(t)))
