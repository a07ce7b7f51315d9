"""GPU parity: every in-scope node, called through the C ABI of libdyb200.so, against the CPU
oracle on the same seeded inputs.  Bars: bit-exact for gather / indices, 1e-5 relative for
elementwise ops, 1e-4 for reductions, LSTM states and gradients (absolute floor for values near 0)."""
import ctypes as C
import json
import os

import numpy as np
import pytest

from util import TOL_CWISE, TOL_REDUCE, assert_close, glorot, randn, rng, zipf_ids

pytestmark = pytest.mark.gpu

# Backward results are dEdxi_before + gradient with dEdxi_before ~ N(0,1): rounding of the O(1) terms
# (one ulp ~ 1e-7) sets the achievable absolute error, so sums that cancel are compared against that scale.
ACC_FLOOR = 0.25
# Gate pre-activations are O(1) sums of hundreds of products.  The tensor pipe adds into its fp32
# accumulator with truncation, so the 3xTF32 GEMM is good to ~1e-5 of that scale (measured: 7e-6
# worst case over 32k outputs at K = 640), and the CPU sigmoid itself is a rational fit good to ~2e-7
# absolute; gate / state values near zero are therefore compared against 0.1, not against themselves.
GEMM_FLOOR = 0.1

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_known_answers.json")))


@pytest.fixture(scope="module")
def g():
    import gpu_util
    gpu_util.ctx()
    return gpu_util


@pytest.fixture(autouse=True)
def _release_device_buffers(g):
    yield
    g.release()


@pytest.fixture(scope="module")
def capi():
    from dynet_b200 import capi as c
    return c


SIZES = [1, 3, 31, 32, 33, 127, 128, 129, 1000, 4097, (1 << 16) + 3]


# ------------------------------------------------------------------ unary
@pytest.mark.parametrize("name", ["tanh", "logistic", "rectify", "elu"])
@pytest.mark.parametrize("misalign", [0, 1])
def test_unary(oracle, g, capi, name, misalign):
    r = rng(100)
    attrs = capi.EluAttrs(1.0, 1.0) if name == "elu" else None
    for n in SIZES:
        x = randn(r, 1, n, scale=3.0)
        if name == "rectify":
            x[0, ::7] = 0.0
        dy = randn(r, 1, n)
        dx0 = randn(r, 1, n)
        y_ref = oracle.unary_fwd(name, x)
        dx_ref = oracle.unary_bwd(name, x, y_ref, dy, dx0.copy())
        dx_, y_, dy_, dxo = g.dev(x, misalign), g.dev(np.zeros_like(x), misalign), g.dev(dy, misalign), g.dev(dx0, misalign)
        g.ctx().fwd(name, [g.T(dx_)], g.T(y_), attrs)
        assert_close(g.host(y_), y_ref, TOL_CWISE, floor=2e-2 if name == "logistic" else 1e-3, what="%s fwd n=%d" % (name, n))
        if name == "rectify":
            assert np.array_equal(g.host(y_), y_ref)
        g.ctx().bwd(name, [g.T(dx_)], g.T(y_), g.T(dy_), 0, g.T(dxo), attrs)
        assert_close(g.host(dxo), dx_ref, TOL_CWISE, floor=ACC_FLOOR, what="%s bwd n=%d" % (name, n))


def test_selu_constants(oracle, g, capi):
    lam, alpha = 1.0507009873554804934193349852946, 1.6732632423543772848170429916717
    r = rng(101)
    x = randn(r, 2, 1001, scale=2.0)
    y_ref = oracle.unary_fwd("elu", x, alpha, lam)
    y = g.dev(np.zeros_like(x))
    g.ctx().fwd("elu", [g.T(g.dev(x))], g.T(y), capi.EluAttrs(alpha, lam))
    assert_close(g.host(y), y_ref, TOL_CWISE, what="selu")


# ------------------------------------------------------------------ cwise binary
CW_SHAPES = [
    ((4, 128), (4, 128)),          # same shape, vector path
    ((4, 130), (4, 130)),          # same shape, n % 4 != 0
    ((5, 256), (1, 256)),          # right operand batch-broadcast (dropout mask bd=1)
    ((1, 256), (5, 256)),          # left operand batch-broadcast
    ((3, 2, 7), (1, 1, 7)),        # broadcast over dim 1 and batch
    ((3, 2, 7), (3, 2, 1)),        # broadcast over dim 0
    ((2, 3, 1), (1, 1, 5)),        # both sides broadcast
]


@pytest.mark.parametrize("op", ["cmult", "csum", "cdiv"])
@pytest.mark.parametrize("sa,sb", CW_SHAPES)
def test_cwise(oracle, g, op, sa, sb):
    if op == "cdiv" and any(y > x for x, y in zip(sa, sb)):
        pytest.skip("CwiseQuotient only broadcasts its right operand")
    r = rng(110)
    a = randn(r, *sa) + 2.5
    b = randn(r, *sb) * 0.3 + 2.0
    y_ref = oracle.cwise_fwd(op, a, b)
    a_, b_ = g.dev(a), g.dev(b)
    y_ = g.dev(np.zeros_like(y_ref))
    g.ctx().fwd(op, [g.T(a_), g.T(b_)], g.T(y_))
    assert_close(g.host(y_), y_ref, TOL_CWISE, what=op + " fwd")
    dy = randn(r, *y_ref.shape)
    for i, arg in enumerate((a, b)):
        d0 = randn(r, *arg.shape)
        want = oracle.cwise_bwd(op, a, b, dy, i, d0.copy())
        d_ = g.dev(d0)
        g.ctx().bwd(op, [g.T(a_), g.T(b_)], g.T(y_), g.T(g.dev(dy)), i, g.T(d_))
        assert_close(g.host(d_), want, TOL_REDUCE, floor=ACC_FLOOR, what="%s bwd i=%d" % (op, i))


def test_cwise_bad_shape(g, capi):
    a, b = g.dev(np.zeros((1, 4), np.float32)), g.dev(np.zeros((1, 3), np.float32))
    with pytest.raises(capi.InvalidArgument):
        g.ctx().fwd("cmult", [g.T(a), g.T(b)], g.T(g.dev(np.zeros((1, 4), np.float32))))


# ------------------------------------------------------------------ softmax family
@pytest.mark.parametrize("rows,cols,bd", [(1, 1, 1), (3, 2, 2), (45, 7, 3), (256, 3, 2), (257, 2, 2), (1024, 5, 2),
                                          (4096, 3, 2), (5001, 2, 1), (10000, 1, 3)])
def test_softmax_dim0(oracle, g, capi, rows, cols, bd):
    r = rng(120)
    x = randn(r, bd, cols, rows, scale=2.0)
    y_ref = oracle.softmax_fwd(x, 0)
    x_, y_ = g.dev(x), g.dev(np.zeros_like(x))
    at = capi.DimAttrs(0)
    g.ctx().fwd("softmax", [g.T(x_)], g.T(y_), at)
    assert_close(g.host(y_), y_ref, TOL_REDUCE, floor=1e-6, what="softmax d0")
    dy, d0 = randn(r, bd, cols, rows), randn(r, bd, cols, rows)
    want = oracle.softmax_bwd(y_ref, dy, d0.copy(), 0)
    d_ = g.dev(d0)
    g.ctx().bwd("softmax", [g.T(x_)], g.T(g.dev(y_ref)), g.T(g.dev(dy)), 0, g.T(d_), at)
    assert_close(g.host(d_), want, TOL_REDUCE, floor=ACC_FLOOR, what="softmax d0 bwd")


@pytest.mark.parametrize("rows,cols,bd", [(1, 5, 1), (7, 3, 2), (33, 200, 2), (64, 4096, 1), (9, 4500, 1)])
def test_softmax_dim1(oracle, g, capi, rows, cols, bd):
    r = rng(121)
    x = randn(r, bd, cols, rows, scale=2.0)
    y_ref = oracle.softmax_fwd(x, 1)
    x_, y_ = g.dev(x), g.dev(np.zeros_like(x))
    at = capi.DimAttrs(1)
    g.ctx().fwd("softmax", [g.T(x_)], g.T(y_), at)
    assert_close(g.host(y_), y_ref, TOL_REDUCE, floor=1e-6, what="softmax d1")
    dy, d0 = randn(r, bd, cols, rows), randn(r, bd, cols, rows)
    want = oracle.softmax_bwd(y_ref, dy, d0.copy(), 1)
    d_ = g.dev(d0)
    g.ctx().bwd("softmax", [g.T(x_)], g.T(g.dev(y_ref)), g.T(g.dev(dy)), 0, g.T(d_), at)
    assert_close(g.host(d_), want, TOL_REDUCE, floor=ACC_FLOOR, what="softmax d1 bwd")


@pytest.mark.parametrize("rows,cols,bd", [(5, 1, 1), (45, 3, 4), (300, 2, 2), (4100, 2, 1)])
def test_log_softmax(oracle, g, rows, cols, bd):
    r = rng(122)
    x = randn(r, bd, cols, rows, scale=2.0)
    y_ref = oracle.log_softmax_fwd(x)
    x_, y_ = g.dev(x), g.dev(np.zeros_like(x))
    aux = g.dev(np.zeros(2 * cols * bd, np.float32))
    g.ctx().fwd("log_softmax", [g.T(x_)], g.T(y_), None, aux.data_ptr())
    assert_close(g.host(y_), y_ref, TOL_REDUCE, what="log_softmax")
    dy, d0 = randn(r, bd, cols, rows), randn(r, bd, cols, rows)
    want = oracle.log_softmax_bwd(y_ref, dy, d0.copy())
    d_ = g.dev(d0)
    g.ctx().bwd("log_softmax", [g.T(x_)], g.T(g.dev(y_ref)), g.T(g.dev(dy)), 0, g.T(d_), None, aux.data_ptr())
    assert_close(g.host(d_), want, TOL_REDUCE, floor=ACC_FLOOR, what="log_softmax bwd")


@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("rows,cols,bd", [(6, 4, 2), (130, 70, 2), (5000, 3, 1), (3, 5000, 1)])
def test_logsumexp_dim(oracle, g, capi, axis, rows, cols, bd):
    r = rng(123)
    x = randn(r, bd, cols, rows, scale=2.0)
    z_ref, _ = oracle.logsumexp_dim_fwd(x, axis)
    x_ = g.dev(x)
    z_ = g.dev(np.zeros_like(z_ref))
    at = capi.DimAttrs(axis)
    outer = cols if axis == 0 else rows
    g.ctx().fwd("logsumexp_dim", [g.T(x_)], g.T(z_, [outer], bd), at)
    assert_close(g.host(z_), z_ref, TOL_REDUCE, what="logsumexp_dim")
    dz, d0 = randn(r, *z_ref.shape), randn(r, bd, cols, rows)
    want = oracle.logsumexp_dim_bwd(x, z_ref, dz, d0.copy(), axis)
    d_ = g.dev(d0)
    g.ctx().bwd("logsumexp_dim", [g.T(x_)], g.T(g.dev(z_ref), [outer], bd), g.T(g.dev(dz), [outer], bd), 0, g.T(d_), at)
    assert_close(g.host(d_), want, TOL_REDUCE, floor=ACC_FLOOR, what="logsumexp_dim bwd")


def test_logsumexp_nary(oracle, g):
    r = rng(124)
    for n, bd in [(5, 3), (1000, 4)]:
        xs = [randn(r, bd, n), randn(r, 1, n), randn(r, bd, n), randn(r, 1, n)]
        y_ref = oracle.logsumexp_nary_fwd(xs)
        xd = [g.dev(x) for x in xs]
        y_ = g.dev(np.zeros_like(y_ref))
        g.ctx().fwd("logsumexp", [g.T(t) for t in xd], g.T(y_))
        assert_close(g.host(y_), y_ref, TOL_REDUCE, what="logsumexp nary")
        dy = randn(r, bd, n)
        for i in range(len(xs)):
            d0 = randn(r, *xs[i].shape)
            want = oracle.logsumexp_nary_bwd(xs, i, y_ref, dy, d0.copy())
            d_ = g.dev(d0)
            g.ctx().bwd("logsumexp", [g.T(t) for t in xd], g.T(g.dev(y_ref)), g.T(g.dev(dy)), i, g.T(d_))
            assert_close(g.host(d_), want, TOL_REDUCE, floor=ACC_FLOOR, what="logsumexp nary bwd %d" % i)
    x1 = randn(r, 2, 9)
    y_ = g.dev(np.zeros_like(x1))
    g.ctx().fwd("logsumexp", [g.T(g.dev(x1))], g.T(y_))
    assert np.array_equal(g.host(y_), x1)  # single argument: copy (nodes-logsumexp.cc:39-40)


@pytest.mark.parametrize("rows,bd", [(1, 1), (45, 200), (1000, 7), (4096, 3), (10000, 64), (50000, 5)])
def test_pickneglogsoftmax(oracle, g, capi, rows, bd):
    r = rng(125)
    x = randn(r, bd, rows, scale=2.0)
    ids = zipf_ids(r, bd, rows)
    loss_ref, z_ref = oracle.pnls_fwd(x, ids)
    x_ = g.dev(x)
    loss_ = g.dev(np.zeros(bd, np.float32))
    aux = g.dev(np.zeros(3 * bd, np.float32))
    ids_np, ids_p = g.u32(ids)
    at = capi.PickAttrs(ids_p, bd)
    g.ctx().fwd("pickneglogsoftmax", [g.T(x_, [rows], bd)], g.T(loss_, [1], bd), at, aux.data_ptr())
    assert_close(g.host(loss_), loss_ref, TOL_REDUCE, what="pnls fwd")
    assert_close(g.host(aux)[:bd], z_ref, TOL_REDUCE, what="pnls z")
    dE, d0 = randn(r, bd), randn(r, bd, rows)
    want = oracle.pnls_bwd(x, ids, z_ref, dE, d0.copy())
    d_ = g.dev(d0)
    g.ctx().bwd("pickneglogsoftmax", [g.T(x_, [rows], bd)], g.T(loss_, [1], bd), g.T(g.dev(dE), [1], bd), 0,
                g.T(d_, [rows], bd), at, aux.data_ptr())
    assert_close(g.host(d_), want, TOL_REDUCE, floor=ACC_FLOOR, what="pnls bwd")
    assert g.ctx().device_errors() == 0


@pytest.mark.parametrize("rows", [45, 301, 4096, 4099, 10000])
def test_softmax_family_with_minus_infinity_entries(oracle, g, capi, rows):
    """Logits of -inf (RestrictedLogSoftmax writes them, dynet/nodes-softmaxes.cc:261) carry no probability mass: the
    reference subtracts the column maximum first, so exp(-inf - max) = 0.  Covers the warp, register and streaming
    kernels (rows > 4096, rows % 4 != 0), including a thread whose whole share of a column is -inf."""
    r = rng(126 + rows)
    bd = 3
    x = randn(r, bd, rows, scale=2.0)
    x[0, r.random(rows) < 0.3] = -np.inf
    x[1, : rows - 2] = -np.inf                     # only two finite entries, at the end of the column
    x[2, 5:] = -np.inf                             # only five finite entries, at the start
    ids = np.array([int(np.flatnonzero(np.isfinite(x[b]))[0]) for b in range(bd)], np.uint32)
    x_ = g.dev(x)
    fin = np.isfinite(x)
    # softmax
    y_ref = oracle.softmax_fwd(x.reshape(bd, 1, rows), 0).reshape(bd, rows)
    y_ = g.dev(np.zeros_like(x))
    g.ctx().fwd("softmax", [g.T(x_, [rows], bd)], g.T(y_, [rows], bd), capi.DimAttrs(0))
    got = g.host(y_)
    assert np.all(got[~fin] == 0.0)
    assert_close(got, y_ref, TOL_REDUCE, floor=1e-6, what="softmax with -inf")
    # log_softmax
    ly_ref = oracle.log_softmax_fwd(x.reshape(bd, 1, rows)).reshape(bd, rows)
    ly_ = g.dev(np.zeros_like(x))
    aux = g.dev(np.zeros(2 * bd, np.float32))
    g.ctx().fwd("log_softmax", [g.T(x_, [rows], bd)], g.T(ly_, [rows], bd), None, aux.data_ptr())
    got = g.host(ly_)
    assert np.all(got[~fin] == -np.inf) and np.all(ly_ref[~fin] == -np.inf)
    assert_close(got[fin], ly_ref[fin], TOL_REDUCE, what="log_softmax with -inf")
    # logsumexp along dim 0
    z_ref, _ = oracle.logsumexp_dim_fwd(x.reshape(bd, 1, rows), 0)
    z_ = g.dev(np.zeros_like(z_ref))
    g.ctx().fwd("logsumexp_dim", [g.T(x_, [rows, 1], bd)], g.T(z_, [1], bd), capi.DimAttrs(0))
    assert_close(g.host(z_).ravel(), z_ref.ravel(), TOL_REDUCE, what="logsumexp with -inf")
    # PickNegLogSoftmax forward and backward (picked entries are finite)
    loss_ref, zr = oracle.pnls_fwd(x, ids)
    loss_ = g.dev(np.zeros(bd, np.float32))
    aux = g.dev(np.zeros(3 * bd, np.float32))
    ids_np, ids_p = g.u32(ids)
    at = capi.PickAttrs(ids_p, bd)
    g.ctx().fwd("pickneglogsoftmax", [g.T(x_, [rows], bd)], g.T(loss_, [1], bd), at, aux.data_ptr())
    assert_close(g.host(loss_), loss_ref, TOL_REDUCE, what="pnls fwd with -inf")
    dE, d0 = randn(r, bd), randn(r, bd, rows)
    want = oracle.pnls_bwd(x, ids, zr, dE, d0.copy())
    d_ = g.dev(d0)
    g.ctx().bwd("pickneglogsoftmax", [g.T(x_, [rows], bd)], g.T(loss_, [1], bd), g.T(g.dev(dE), [1], bd), 0,
                g.T(d_, [rows], bd), at, aux.data_ptr())
    assert np.array_equal(g.host(d_)[~fin], d0[~fin])        # no gradient reaches a -inf logit
    assert_close(g.host(d_), want, TOL_REDUCE, floor=ACC_FLOOR, what="pnls bwd with -inf")
    assert g.ctx().device_errors() == 0


@pytest.mark.parametrize("V,H,n", [(1000, 256, 192), (1001, 250, 67), (2100, 128, 1300), (40, 16, 8)])
def test_softmax_output_bwd_fused(oracle, g, capi, V, H, n):
    """dyb200_softmax_output_bwd_fused == PickNegLogSoftmax backward into a zeroed d(x), then AffineTransform backward
    for the bias, R and h.  Vector and scalar paths (V, n multiples of 4 or not), a tile grid with a ragged edge, and a
    shape small enough for the node-by-node path through the scratch tensor.  The two products see bitwise the same
    operands, so dR and dh are equal bit for bit; the bias gradient is summed in another order."""
    r = rng(V + n)
    b, R, h = randn(r, 1, 1, V, scale=0.1), randn(r, 1, H, V, scale=0.1), randn(r, n, 1, H, scale=0.5)
    ids = zipf_ids(r, n, V)
    x = oracle.affine_fwd([b, R, h])                    # (n, 1, V)
    loss_ref, z_ref = oracle.pnls_fwd(x[:, 0, :], ids)
    dE = randn(r, n)
    dx_ref = oracle.pnls_bwd(x[:, 0, :], ids, z_ref, dE, np.zeros((n, V), np.float32))
    g0 = [randn(r, *a.shape, scale=0.1) for a in (b, R, h)]
    want = [oracle.affine_bwd([b, R, h], dx_ref[:, None, :], i, g0[i].copy()) for i in range(3)]
    ctx = g.ctx()
    tb, tR, th_ = g.T(g.dev(b), [V], 1), g.T(g.dev(R), [V, H], 1), g.T(g.dev(h), [H], n)
    x_ = g.dev(np.zeros((n, V), np.float32))
    tx = g.T(x_, [V], n)
    ctx.fwd("affine_transform", [tb, tR, th_], tx)
    loss_, aux = g.dev(np.zeros(n, np.float32)), g.dev(np.zeros(3 * n, np.float32))
    ids_np, ids_p = g.u32(ids)
    at = capi.PickAttrs(ids_p, n)
    ctx.fwd("pickneglogsoftmax", [tx], g.T(loss_, [1], n), at, aux.data_ptr())
    tdE = g.T(g.dev(dE), [1], n)
    # node by node
    dx_ = g.dev(np.zeros((n, V), np.float32))
    ctx.bwd("pickneglogsoftmax", [tx], g.T(loss_, [1], n), tdE, 0, g.T(dx_, [V], n), at, aux.data_ptr())
    node = [g.dev(a) for a in g0]
    shapes = [([V], 1), ([V, H], 1), ([H], n)]
    for i in range(3):
        ctx.bwd("affine_transform", [tb, tR, th_], tx, g.T(dx_, [V], n), i, g.T(node[i], *shapes[i]))
    # fused
    fused = [g.dev(a) for a in g0]
    scratch = g.dev(np.full((n, V), 3.0, np.float32))
    ctx.softmax_output_bwd_fused(tx, th_, tR, tdE, aux.data_ptr(), g.T(fused[1], *shapes[1]), g.T(fused[0], *shapes[0]),
                                 g.T(fused[2], *shapes[2]), g.T(scratch, [V], n))
    assert np.array_equal(g.host(fused[1]), g.host(node[1]))
    assert np.array_equal(g.host(fused[2]), g.host(node[2]))
    for i, what in enumerate(("db", "dR", "dh")):
        scale = max(1e-2, float(np.abs(want[i]).max()) * 0.05)
        assert_close(g.host(fused[i]), want[i], TOL_REDUCE, floor=scale, what="fused " + what)
        assert_close(g.host(fused[i]), g.host(node[i]), 1e-5, floor=scale, what="fused vs nodes " + what)
    assert ctx.device_errors() == 0


def test_pickneglogsoftmax_errors(g, capi):
    x_ = g.dev(np.zeros((2, 5), np.float32))
    loss_, aux = g.dev(np.zeros(2, np.float32)), g.dev(np.zeros(6, np.float32))
    _, p = g.u32([0, 5])
    with pytest.raises(capi.InvalidArgument):  # index out of bounds (nodes-pickneglogsoftmax.cc:91,100)
        g.ctx().fwd("pickneglogsoftmax", [g.T(x_, [5], 2)], g.T(loss_, [1], 2), capi.PickAttrs(p, 2), aux.data_ptr())
    _, p = g.u32([0])
    with pytest.raises(capi.InvalidArgument):  # wrong number of ids
        g.ctx().fwd("pickneglogsoftmax", [g.T(x_, [5], 2)], g.T(loss_, [1], 2), capi.PickAttrs(p, 1), aux.data_ptr())
    _, p = g.u32([0, 1])
    with pytest.raises(capi.RuntimeErr):  # multiple columns: "not yet implemented" in the reference
        g.ctx().fwd("pickneglogsoftmax", [g.T(x_, [5, 2], 1)], g.T(loss_, [1], 1), capi.PickAttrs(p, 1), aux.data_ptr())


# ------------------------------------------------------------------ norms
@pytest.mark.parametrize("n", [9, 1000, 4096 * 3 + 1, 1024 * 4096])
def test_weight_norm(oracle, g, n):
    r = rng(130)
    w = randn(r, n) + 0.1
    gv = np.array([1.3], np.float32)
    y_ref = oracle.weight_norm_fwd(w, float(gv[0]))
    w_, g_, y_ = g.dev(w), g.dev(gv), g.dev(np.zeros_like(w))
    xs = [g.T(w_, [n], 1), g.T(g_, [1], 1)]
    g.ctx().fwd("weight_norm", xs, g.T(y_, [n], 1))
    assert_close(g.host(y_), y_ref, TOL_REDUCE, floor=1e-7, what="weight_norm fwd")
    dy = randn(r, n)
    for i, shape in ((0, n), (1, 1)):
        d0 = randn(r, shape)
        want = oracle.weight_norm_bwd(w, float(gv[0]), y_ref, dy, i, d0.copy())
        d_ = g.dev(d0)
        g.ctx().bwd("weight_norm", xs, g.T(g.dev(y_ref), [n], 1), g.T(g.dev(dy), [n], 1), i, g.T(d_, [shape], 1))
        assert_close(g.host(d_), want, TOL_REDUCE, floor=1e-2 if i == 1 else 1e-3, what="weight_norm bwd %d" % i)


def test_weight_norm_golden(g):
    c = GOLD["weight_norm_forward"]
    w = np.asarray(c["w"], np.float32)
    y_ = g.dev(np.zeros_like(w))
    g.ctx().fwd("weight_norm", [g.T(g.dev(w), [3, 3], 1), g.T(g.dev(np.array([c["g"]], np.float32)), [1], 1)], g.T(y_, [3, 3], 1))
    norm = float(np.sqrt((g.host(y_).astype(np.float64) ** 2).sum()))
    assert abs(norm - c["expect_norm"]) <= c["tol_rel"] * c["expect_norm"]


def test_moment_std_dim(oracle, g, capi):
    r = rng(131)
    # the layer_norm use: all non-batch dims reduced, batch kept
    for n, bd in [(3, 1), (10, 4), (4096, 6), (5003, 2)]:
        x = randn(r, bd, n) + 0.5
        x_ = g.dev(x)
        for order in (1, 2, 3):
            at = capi.MomentAttrs((C.c_uint32 * 2)(0, 0), 1, order, 0, 0)
            out = g.dev(np.zeros(bd, np.float32))
            g.ctx().fwd("moment_dim", [g.T(x_)], g.T(out, [1], bd), at)
            assert_close(g.host(out), oracle.moment_elems_fwd(x, order), TOL_REDUCE, what="moment %d" % order)
            dE, d0 = randn(r, bd), randn(r, bd, n)
            want = oracle.moment_elems_bwd(x, order, dE, d0.copy())
            d_ = g.dev(d0)
            g.ctx().bwd("moment_dim", [g.T(x_)], g.T(out, [1], bd), g.T(g.dev(dE), [1], bd), 0, g.T(d_), at)
            assert_close(g.host(d_), want, TOL_REDUCE, floor=ACC_FLOOR, what="moment bwd %d" % order)
        at = capi.MomentAttrs((C.c_uint32 * 2)(0, 0), 1, 0, 0, 0)
        out = g.dev(np.zeros(bd, np.float32))
        g.ctx().fwd("std_dim", [g.T(x_)], g.T(out, [1], bd), at)
        s_ref = oracle.std_elems_fwd(x)
        assert_close(g.host(out), s_ref, TOL_REDUCE, what="std")
        dE, d0 = randn(r, bd), randn(r, bd, n)
        want = oracle.std_elems_bwd(x, s_ref, dE, d0.copy())
        d_ = g.dev(d0)
        g.ctx().bwd("std_dim", [g.T(x_)], g.T(g.dev(s_ref), [1], bd), g.T(g.dev(dE), [1], bd), 0, g.T(d_), at)
        assert_close(g.host(d_), want, TOL_REDUCE, floor=ACC_FLOOR, what="std bwd")


def test_std_dim_value_golden(g, capi):
    c = GOLD["std_dim_value"]
    x = np.asarray(c["x"], np.float32).reshape(3, 3, 3)
    y = g.dev(np.zeros(3, np.float32))
    at = capi.MomentAttrs((C.c_uint32 * 2)(0, 0), 1, 0, 1, 0)   # std_dim(x, {0}, true)
    g.ctx().fwd("std_dim", [g.T(g.dev(x))], g.T(y, [3], 1), at)
    z = g.dev(np.zeros(1, np.float32))
    at2 = capi.MomentAttrs((C.c_uint32 * 2)(0, 0), 1, 1, 0, 0)  # mean_dim(y, {0}, false)
    g.ctx().fwd("moment_dim", [g.T(y, [3], 1)], g.T(z, [1], 1), at2)
    want = c["expect_mean_of_std_dim0_batch"]
    assert abs(float(g.host(z)[0]) - want) <= c["tol_rel"] * want


@pytest.mark.parametrize("n,bd", [(3, 1), (10, 1), (130, 5), (4096, 16), (4100, 3), (9001, 2),
                                  (128, 37), (256, 9), (640, 21), (1024, 300)])   # (the last four: a warp per column)
def test_layer_norm(oracle, g, n, bd):
    r = rng(132)
    x = randn(r, bd, n)
    gain = r.uniform(0.5, 1.5, n).astype(np.float32)
    bias = randn(r, n, scale=0.1)
    y_ref = oracle.layer_norm_fwd(x, gain, bias)
    x_, g_, b_ = g.dev(x), g.dev(gain), g.dev(bias)
    xs = [g.T(x_), g.T(g_, [n], 1), g.T(b_, [n], 1)]
    y_ = g.dev(np.zeros_like(x))
    g.ctx().fwd("layer_norm", xs, g.T(y_))
    assert_close(g.host(y_), y_ref, TOL_REDUCE, what="layer_norm fwd")
    dy = randn(r, bd, n)
    dx0, dg0, db0 = randn(r, bd, n), randn(r, n), randn(r, n)
    wx, wg, wb = oracle.layer_norm_bwd(x, gain, dy, dx0.copy(), dg0.copy(), db0.copy())
    dy_ = g.dev(dy)
    for i, (d0, want, dims, b) in enumerate(((dx0, wx, None, None), (dg0, wg, [n], 1), (db0, wb, [n], 1))):
        d_ = g.dev(d0)
        g.ctx().bwd("layer_norm", xs, g.T(y_), g.T(dy_), i, g.T(d_) if dims is None else g.T(d_, dims, b))
        assert_close(g.host(d_), want, TOL_REDUCE, floor=ACC_FLOOR, what="layer_norm bwd %d" % i)


def test_layer_norm_golden(g):
    c = GOLD["layer_norm_forward"]
    x = np.asarray(c["x"], np.float32).reshape(1, 3)
    y_ = g.dev(np.zeros_like(x))
    g.ctx().fwd("layer_norm", [g.T(g.dev(x)), g.T(g.dev(np.asarray(c["g"], np.float32)), [3], 1),
                               g.T(g.dev(np.asarray(c["b"], np.float32)), [3], 1)], g.T(y_))
    y = g.host(y_)
    assert abs(float(y.sum() / 3.0)) < c["expect_abs_mean_lt"]
    assert abs(float(np.sqrt((y.astype(np.float64) ** 2).sum() / 3.0)) - 1.0) <= c["tol_rel"]
    v = np.arange(10).astype(np.float32)
    y_ = g.dev(np.zeros((1, 10), np.float32))
    g.ctx().fwd("layer_norm", [g.T(g.dev(v.reshape(1, 10))), g.T(g.dev(v), [10], 1), g.T(g.dev(v), [10], 1)], g.T(y_))
    assert np.allclose(g.host(y_).ravel(), v / v.std() * (v - v.mean()) + v)


def test_layer_norm_composite_nodes(oracle, g, capi):
    """The 8-node composite of dynet/expr.cc:248-253 built from the drop-in nodes equals the fused kernel."""
    r = rng(133)
    n, bd = 64, 5
    x = randn(r, bd, n)
    gain, bias = r.uniform(0.5, 1.5, n).astype(np.float32), randn(r, n, scale=0.1)
    c = g.ctx()
    x_ = g.dev(x)
    at1 = capi.MomentAttrs((C.c_uint32 * 2)(0, 0), 1, 1, 0, 0)
    mu, sg = g.dev(np.zeros(bd, np.float32)), g.dev(np.zeros(bd, np.float32))
    c.fwd("moment_dim", [g.T(x_)], g.T(mu, [1], bd), at1)
    c.fwd("std_dim", [g.T(x_)], g.T(sg, [1], bd), at1)
    neg = -mu
    s2 = sg + np.float32(1e-8)
    xc, q, y1, y = (g.dev(np.zeros_like(x)) for _ in range(4))
    c.fwd("csum", [g.T(x_), g.T(neg, [1], bd)], g.T(xc))
    c.fwd("cdiv", [g.T(xc), g.T(s2, [1], bd)], g.T(q))
    c.fwd("cmult", [g.T(g.dev(gain), [n], 1), g.T(q)], g.T(y1))
    c.fwd("csum", [g.T(y1), g.T(g.dev(bias), [n], 1)], g.T(y))
    assert_close(g.host(y), oracle.layer_norm_fwd(x, gain, bias), TOL_REDUCE, what="composite layer_norm")


# ------------------------------------------------------------------ embedding
@pytest.mark.parametrize("E,V,n", [(4, 9, 5), (128, 1000, 300), (512, 5000, 4096), (6, 50, 77), (1028, 64, 33), (2048, 32, 40)])
@pytest.mark.parametrize("scale", [1.0, 0.75])
def test_lookup_gather_bit_exact(oracle, g, capi, E, V, n, scale):
    r = rng(140)
    table = randn(r, V, E)
    ids = zipf_ids(r, n, V)
    ids[0] = V - 1
    want = oracle.lookup_fwd(table, ids, scale)
    tab_, out_ = g.dev(table), g.dev(np.zeros((n, E), np.float32))
    aux = g.dev(np.zeros(n, np.float32))
    _, p = g.u32(ids)
    at = capi.LookupAttrs(tab_.data_ptr(), V, p, n, scale)
    g.ctx().fwd("lookup", [], g.T(out_, [E], n), at, aux.data_ptr())
    assert np.array_equal(g.host(out_), want)
    assert g.ctx().device_errors() == 0


def test_lookup_errors(g, capi):
    tab_, out_, aux = g.dev(np.zeros((9, 4), np.float32)), g.dev(np.zeros((2, 4), np.float32)), g.dev(np.zeros(2, np.float32))
    _, p = g.u32([1, 9])
    with pytest.raises(capi.InvalidArgument):
        g.ctx().fwd("lookup", [], g.T(out_, [4], 2), capi.LookupAttrs(tab_.data_ptr(), 9, p, 2, 1.0), aux.data_ptr())
    with pytest.raises(capi.InvalidArgument):
        g.ctx().fwd("lookup", [], g.T(out_, [4], 2), capi.LookupAttrs(tab_.data_ptr(), 9, p, 1, 1.0), aux.data_ptr())


@pytest.mark.parametrize("E,V,n", [(4, 9, 1), (4, 9, 5), (128, 1000, 512), (512, 5000, 4096), (6, 50, 77), (64, 300, 9000),
                                   (128, 2000, 50000)])   # (the last: 13 sorted runs merged, the most frequent id spans ~150 chunks)
def test_lookup_scatter_add(oracle, g, E, V, n):
    r = rng(141)
    ids = zipf_ids(r, n, V)
    grad = randn(r, n, E)
    acc0 = randn(r, V, E)
    want = oracle.lookup_accumulate_grads(acc0.copy(), ids, grad)
    acc_ = g.dev(acc0)
    ids_dev = g.dev(ids.view(np.float32)).view(dtype=__import__("torch").int32)
    g.ctx().lookup_accumulate_grads(ids, ids_dev.data_ptr(), g.dev(grad).data_ptr(), acc_.data_ptr(), E, V)
    got = g.host(acc_)
    # Rows of one id are added in ascending position.  An id whose run fits inside one 32-position chunk of
    # the sorted list is summed exactly as the CPU loop does (bit-exact); a frequent id (Zipf head) that
    # spans chunks is summed chunk-wise in a fixed tree, equal to the CPU's chain within rounding.
    counts = np.bincount(ids, minlength=V)
    rare = counts <= 1
    assert np.array_equal(got[rare], want[rare])
    assert_close(got, want, TOL_REDUCE, floor=max(1.0, float(np.sqrt(counts.max()))), what="scatter-add")
    # run to run reproducible
    acc2 = g.dev(acc0)
    g.ctx().lookup_accumulate_grads(ids, ids_dev.data_ptr(), g.dev(grad).data_ptr(), acc2.data_ptr(), E, V)
    assert np.array_equal(g.host(acc2), got)
    assert g.ctx().device_errors() == 0


# ------------------------------------------------------------------ fused LSTM nodes
def _gates_call(g, capi, xs, h, Wx, Wh, b, mx=None, mh=None, noise=0.0):
    B, H = h.shape
    d = [g.dev(x) for x in xs] + [g.dev(h), g.dev(Wx), g.dev(Wh), g.dev(b)]
    ts = [g.T(t) for t in d[:len(xs) + 1]]
    I = Wx.shape[0]
    ts += [g.T(d[-3], [4 * H, I], 1), g.T(d[-2], [4 * H, H], 1), g.T(d[-1], [4 * H], 1)]
    if mx is not None:
        d += [g.dev(mx), g.dev(mh)]
        ts += [g.T(d[-2]), g.T(d[-1])]
    at = capi.LstmGatesAttrs(1 if mx is not None else 0, noise, 1.0)
    return d, ts, at


@pytest.mark.parametrize("name", ["lstm_node_gates_fwd", "lstm_node_gates_dropout_fwd"])
def test_lstm_gates_golden(g, capi, name):
    c = GOLD[name]
    I, H, B = c["I"], c["H"], c["B"]
    f = lambda k, *s: np.asarray(c[k], np.float32).reshape(*s)
    mx = f("mask_x", B, I) if "mask_x" in c else None
    mh = f("mask_h", B, H) if "mask_h" in c else None
    d, ts, at = _gates_call(g, capi, [f("x_t", B, I)], f("h_tm1", B, H), f("Wx", I, 4 * H), f("Wh", H, 4 * H), f("b", 4 * H), mx, mh)
    fx = g.dev(np.zeros((B, 4 * H), np.float32))
    g.ctx().fwd("vanilla_lstm_gates", ts, g.T(fx), at)
    got = g.host(fx).ravel()
    for a, w in zip(got, c["expect"]):
        assert abs(a - w) <= c["tol_rel"] * abs(w), (a, w)


def test_lstm_c_h_golden(g):
    for name, node, key in (("lstm_node_c_fwd", "vanilla_lstm_c", "c_tm1"), ("lstm_node_h_fwd", "vanilla_lstm_h", "c_t")):
        c = GOLD[name]
        H, B = c["H"], c["B"]
        st = np.asarray(c[key], np.float32).reshape(B, H)
        gt = np.asarray(c["gates_t"], np.float32).reshape(B, 4 * H)
        out = g.dev(np.zeros((B, H), np.float32))
        g.ctx().fwd(node, [g.T(g.dev(st)), g.T(g.dev(gt))], g.T(out))
        for a, w in zip(g.host(out).ravel(), c["expect"]):
            assert abs(a - w) <= (c["tol_abs_zero"] if w == 0 else c["tol_rel"] * abs(w)), (name, a, w)


@pytest.mark.parametrize("I_list,H,B,masks", [([5], 3, 2, None), ([3, 2], 3, 2, "full"), ([128], 256, 32, None),
                                              ([128], 256, 32, "bd1"), ([96, 32], 64, 17, "full"), ([512], 128, 64, "full"),
                                              ([130], 66, 5, "bd1")])
def test_lstm_gates_vs_oracle(oracle, g, capi, I_list, H, B, masks):
    r = rng(150)
    I = sum(I_list)
    xs = [randn(r, B, i) for i in I_list]
    h = randn(r, B, H, scale=0.5)
    Wx, Wh = glorot(r, 4 * H, I), glorot(r, 4 * H, H)
    b = randn(r, 4 * H, scale=0.1)
    mx = mh = None
    if masks:
        mb = B if masks == "full" else 1
        mx = ((r.random((mb, I)) < 0.8) / 0.8).astype(np.float32)
        mh = ((r.random((mb, H)) < 0.8) / 0.8).astype(np.float32)
    fx_ref = oracle.lstm_gates_fwd(xs, h, Wx, Wh, b, mx, mh)
    d, ts, at = _gates_call(g, capi, xs, h, Wx, Wh, b, mx, mh)
    fx = g.dev(np.zeros((B, 4 * H), np.float32))
    g.ctx().fwd("vanilla_lstm_gates", ts, g.T(fx), at)
    assert_close(g.host(fx), fx_ref, TOL_REDUCE, floor=GEMM_FLOOR, what="gates fwd")
    dE = randn(r, B, 4 * H)
    fx_r, dE_ = g.dev(fx_ref), g.dev(dE)
    args = xs + [h, Wx, Wh, b]
    for i, arg in enumerate(args):
        d0 = randn(r, *arg.shape)
        want = oracle.lstm_gates_bwd(xs, h, Wx, Wh, fx_ref, dE, i, d0.copy(), mx, mh)
        d_ = g.dev(d0)
        g.ctx().bwd("vanilla_lstm_gates", ts, g.T(fx_r), g.T(dE_), i, capi.DyTensor.of(d_.data_ptr(), ts[i].d[:ts[i].nd], ts[i].bd), at)
        assert_close(g.host(d_), want, TOL_REDUCE, floor=ACC_FLOOR, what="gates bwd i=%d" % i)


def test_lstm_gates_weightnoise_and_errors(oracle, g, capi):
    r = rng(151)
    I, H, B = 6, 4, 3
    xs, h = [randn(r, B, I)], randn(r, B, H)
    Wx, Wh, b = glorot(r, 4 * H, I), glorot(r, 4 * H, H), randn(r, 4 * H)
    d, ts, at = _gates_call(g, capi, xs, h, Wx, Wh, b, noise=0.1)
    fx = g.dev(np.zeros((B, 4 * H), np.float32))
    g.ctx().fwd("vanilla_lstm_gates", ts, g.T(fx), at)   # reference skips both products (nodes-lstm.cc:200-219)
    assert_close(g.host(fx), oracle.lstm_gates_fwd(xs, h, Wx, Wh, b, skip_matmul=True), TOL_CWISE, what="weightnoise")
    d, ts, at = _gates_call(g, capi, xs, h, Wx, Wh, b)
    ts[2] = g.T(d[2], [4 * H + 1, I], 1)
    with pytest.raises(capi.InvalidArgument):
        g.ctx().fwd("vanilla_lstm_gates", ts, g.T(fx), at)


@pytest.mark.parametrize("H,B", [(3, 2), (256, 32), (1024, 9), (130, 7)])
def test_lstm_c_h_vs_oracle(oracle, g, H, B):
    r = rng(152)
    c_prev, gates = randn(r, B, H), r.uniform(0.05, 0.95, (B, 4 * H)).astype(np.float32)
    for node, fwd, bwd in (("vanilla_lstm_c", oracle.lstm_c_fwd, oracle.lstm_c_bwd), ("vanilla_lstm_h", oracle.lstm_h_fwd, oracle.lstm_h_bwd)):
        want = fwd(c_prev, gates)
        xs_d = [g.dev(c_prev), g.dev(gates)]
        xs = [g.T(t) for t in xs_d]
        out = g.dev(np.zeros_like(c_prev))
        g.ctx().fwd(node, xs, g.T(out))
        assert_close(g.host(out), want, TOL_CWISE, floor=5e-2, what=node)  # i*g + f*c cancels; terms are O(0.1)
        dE = randn(r, B, H)
        for i, arg in enumerate((c_prev, gates)):
            d0 = randn(r, *arg.shape)
            w = bwd(c_prev, gates, dE, i, d0.copy())
            d_ = g.dev(d0)
            g.ctx().bwd(node, xs, g.T(out), g.T(g.dev(dE)), i, g.T(d_))
            assert_close(g.host(d_), w, TOL_CWISE, floor=ACC_FLOOR, what="%s bwd %d" % (node, i))


@pytest.mark.parametrize("I,H,B,masks,first", [(5, 3, 2, None, False), (128, 256, 32, "full", False), (96, 64, 17, "bd1", True),
                                                (512, 1024, 64, "full", False), (130, 66, 5, None, False)])
def test_lstm_fused_entry_points_equal_node_chain(oracle, g, capi, I, H, B, masks, first):
    """dyb200_vanilla_lstm_{fwd,bwd}_fused against the oracle's gates -> c -> h node chain and its per-argument backward."""
    r = rng(154)
    x, h, c_prev = randn(r, B, I), randn(r, B, H, scale=0.5), randn(r, B, H, scale=0.5)
    Wx, Wh, b = glorot(r, 4 * H, I), glorot(r, 4 * H, H), randn(r, 4 * H, scale=0.1)
    mx = mh = None
    if masks:
        mb = B if masks == "full" else 1
        mx = ((r.random((mb, I)) < 0.8) / 0.8).astype(np.float32)
        mh = ((r.random((mb, H)) < 0.8) / 0.8).astype(np.float32)
    gates = oracle.lstm_gates_fwd([x], h, Wx, Wh, b, mx, mh)
    c_t = oracle.lstm_c_fwd(c_prev, gates)
    h_t = oracle.lstm_h_fwd(c_t, gates)
    dh, dc = randn(r, B, H), randn(r, B, H)
    # reference backward: H node, C node, gates node, each argument separately, into random starting gradients
    d0 = dict(x=randn(r, B, I), h=randn(r, B, H), c=randn(r, B, H), Wx=randn(r, I, 4 * H), Wh=randn(r, H, 4 * H), b=randn(r, 4 * H))
    want = {k: v.copy() for k, v in d0.items()}
    dc_tot = dc.copy()
    oracle.lstm_h_bwd(c_t, gates, dh, 0, dc_tot)
    dgates = np.zeros_like(gates)
    oracle.lstm_h_bwd(c_t, gates, dh, 1, dgates)
    oracle.lstm_c_bwd(c_prev, gates, dc_tot, 0, want["c"])
    oracle.lstm_c_bwd(c_prev, gates, dc_tot, 1, dgates)
    for i, k in enumerate(["x", "h", "Wx", "Wh", "b"]):
        oracle.lstm_gates_bwd([x], h, Wx, Wh, gates, dgates, i, want[k], mx, mh)
    at = capi.LstmGatesAttrs(1 if masks else 0, 0.0, 1.0)
    D = {k: g.dev(v) for k, v in dict(x=x, h=h, c=c_prev, Wx=Wx, Wh=Wh, b=b, dh=dh, dc=dc).items()}
    tm = (g.T(g.dev(mx)), g.T(g.dev(mh))) if masks else (None, None)
    tx, th_, tc_ = g.T(D["x"]), g.T(D["h"]), g.T(D["c"])
    tWx, tWh, tb = g.T(D["Wx"], [4 * H, I], 1), g.T(D["Wh"], [4 * H, H], 1), g.T(D["b"], [4 * H], 1)
    og, oc, oh = (g.dev(np.zeros_like(a)) for a in (gates, c_t, h_t))
    g.ctx().lstm_fwd_fused(tx, th_, tc_, tWx, tWh, tb, tm[0], tm[1], at, g.T(og), g.T(oc), g.T(oh))
    assert_close(g.host(og), gates, TOL_REDUCE, floor=GEMM_FLOOR, what="fused gates")
    assert_close(g.host(oc), c_t, TOL_REDUCE, floor=GEMM_FLOOR, what="fused c")
    assert_close(g.host(oh), h_t, TOL_REDUCE, floor=GEMM_FLOOR, what="fused h")
    G = {k: g.dev(v) for k, v in d0.items()}
    g.ctx().lstm_bwd_fused(tx, th_, tc_, tWx, tWh, tm[0], tm[1], g.T(g.dev(gates)), g.T(g.dev(c_t)), g.T(D["dh"]), g.T(D["dc"]),
                           g.T(G["x"]), None if first else g.T(G["h"]), None if first else g.T(G["c"]),
                           g.T(G["Wx"], [4 * H, I], 1), g.T(G["Wh"], [4 * H, H], 1), g.T(G["b"], [4 * H], 1), at)
    for k in ["x", "h", "c", "Wx", "Wh", "b"]:
        ref = d0[k] if (first and k in ("h", "c")) else want[k]   # skipped arguments must stay untouched
        assert_close(g.host(G[k]), ref, TOL_REDUCE, floor=ACC_FLOOR * (2.0 if k in ("Wx", "Wh", "b") else 1.0), what="fused d" + k)


def test_lstm_chain_fused_equals_builder_math(oracle, g, capi):
    """Config-1 shape (I=128, H=256, B=32), 5 steps: h_t / c_t through the fused chain on the GPU vs the oracle."""
    r = rng(153)
    I, H, B, T = 128, 256, 32, 5
    Wx, Wh, b = glorot(r, 4 * H, I), glorot(r, 4 * H, H), np.zeros(4 * H, np.float32)
    h = c = np.zeros((B, H), np.float32)
    hd, cd = g.dev(h), g.dev(c)
    for t in range(T):
        x = randn(r, B, I)
        gr = oracle.lstm_gates_fwd([x], h, Wx, Wh, b)
        c = oracle.lstm_c_fwd(c, gr)
        h = oracle.lstm_h_fwd(c, gr)
        d, ts, at = _gates_call(g, capi, [x], np.zeros_like(h), Wx, Wh, b)
        ts[1] = g.T(hd)
        gt = g.dev(np.zeros((B, 4 * H), np.float32))
        g.ctx().fwd("vanilla_lstm_gates", ts, g.T(gt), at)
        c2 = g.dev(np.zeros_like(c))
        g.ctx().fwd("vanilla_lstm_c", [g.T(cd), g.T(gt)], g.T(c2))
        h2 = g.dev(np.zeros_like(h))
        g.ctx().fwd("vanilla_lstm_h", [g.T(c2), g.T(gt)], g.T(h2))
        hd, cd = h2, c2
        assert_close(g.host(hd), h, TOL_REDUCE, floor=GEMM_FLOOR, what="h_%d" % t)
        assert_close(g.host(cd), c, TOL_REDUCE, floor=GEMM_FLOOR, what="c_%d" % t)


# ------------------------------------------------------------------ GEMM
# (the last three have more 128 x 128 / 128 x 64 tiles than a B200 has SMs: the persistent kernel, with a ragged last
# row / column block, two tiles per CTA on some SMs and one on others, and the 64-column tile)
@pytest.mark.parametrize("tA,tB,M,N,K", [(0, 0, 64, 32, 48), (1, 0, 70, 33, 129), (0, 1, 128, 65, 31), (0, 0, 1024, 32, 384),
                                         (1, 0, 384, 32, 1024), (0, 1, 1024, 384, 32), (0, 0, 256, 256, 512),
                                         (0, 0, 2000, 1500, 300), (1, 1, 1930, 2300, 70), (0, 0, 19300, 48, 96)])
def test_gemm(g, tA, tB, M, N, K):
    r = rng(160)
    A = randn(r, *((M, K) if tA else (K, M)))   # C-order (cols, rows) == column-major rows x cols
    Bm = randn(r, *((K, N) if tB else (N, K)))
    C0 = randn(r, N, M)
    opA = A.T.astype(np.float64) if not tA else A.astype(np.float64)       # M x K
    opB = Bm.T.astype(np.float64) if not tB else Bm.astype(np.float64)     # K x N
    ref = opA @ opB
    for acc in (0, 1):
        C_ = g.dev(C0)
        g.ctx().gemm(tA, tB, M, N, K, g.dev(A).data_ptr(), A.shape[1], g.dev(Bm).data_ptr(), Bm.shape[1], C_.data_ptr(), M, acc)
        want = ref.T + (C0 if acc else 0)
        assert_close(g.host(C_), want, TOL_REDUCE, floor=0.1 * K ** 0.5 + 1.0, what="gemm %d%d acc=%d" % (tA, tB, acc))


@pytest.mark.parametrize("M,N,K,acc", [(2048, 512, 4096, 1), (1536, 512, 4096, 1), (4096, 64, 2048, 0), (1024, 200, 1100, 1), (512, 96, 3000, 0)])
def test_gemm_cluster_split_equals_workspace_split(g, M, N, K, acc):
    """Products whose K is split: the cluster form (partial tiles reduced through distributed shared memory) and the
    workspace form (second kernel) add the partial tiles in the same order, so they agree bit for bit."""
    r = rng(M + N + K)
    A, Bm, C0 = randn(r, K, M), randn(r, N, K), randn(r, N, M)
    ctx = g.ctx()
    A_, B_ = g.dev(A), g.dev(Bm)
    outs = []
    try:
        for on in (1, 0):
            ctx.cluster_splitk(on)
            C_ = g.dev(C0)
            ctx.gemm(0, 0, M, N, K, A_.data_ptr(), M, B_.data_ptr(), K, C_.data_ptr(), M, acc)
            outs.append(g.host(C_).copy())
    finally:
        ctx.cluster_splitk(1)
    assert np.array_equal(outs[0], outs[1])
    ref = Bm.astype(np.float64) @ A.astype(np.float64) + (C0 if acc else 0)
    assert_close(outs[0], ref, TOL_REDUCE, floor=0.1 * K ** 0.5 + 1.0, what="split gemm")
    assert ctx.device_errors() == 0


def test_gemm_3xtf32_accuracy(g):
    """Error of the tensor-pipe GEMM against float64, relative to sum_k |a||b| (the scale of the
    reduction): 3xTF32 keeps it below 2e-6; one plain TF32 pass would sit near 5e-4."""
    r = rng(161)
    M, N, K = 512, 256, 1024
    A = randn(r, K, M)
    Bm = randn(r, N, K)
    C_ = g.dev(np.zeros((N, M), np.float32))
    g.ctx().gemm(0, 0, M, N, K, g.dev(A).data_ptr(), M, g.dev(Bm).data_ptr(), K, C_.data_ptr(), M, 0)
    ref = Bm.astype(np.float64) @ A.astype(np.float64)
    scale = np.abs(Bm).astype(np.float64) @ np.abs(A).astype(np.float64)
    rel = np.abs(g.host(C_) - ref) / scale
    assert rel.max() < 2e-6, rel.max()


@pytest.mark.parametrize("M,N0,N1", [(192, 96, 40), (77, 96, 40), (300, 33, 130)])
def test_deferred_weight_gradient(g, M, N0, N1):
    """dyb200_wgrad: T pushes of (A_t, B0_t .* mask, B1_t) then one flush == sum_t A_t B_t^T added to C (float64 reference).
    The accumulator keeps A MN-major in rows of M rounded up to 32: M = 77 and 300 leave padding in every row and a last
    group of 32 rows that is partly beyond M."""
    r = rng(162 + M)
    ks = [32, 32, 32, 32, 20]
    w = g.ctx().wgrad_create(M, N0, N1, sum(ks))
    C0, C1 = randn(r, N0, M), randn(r, N1, M)
    ref0, ref1 = C0.astype(np.float64), C1.astype(np.float64)
    for t, k in enumerate(ks):
        A, B0, B1 = randn(r, k, M), randn(r, k, N0), randn(r, k, N1)
        m0 = ((r.random((k, N0)) < 0.8) / 0.8).astype(np.float32)      # full-batch mask
        m1 = ((r.random((1, N1)) < 0.8) / 0.8).astype(np.float32)      # batch-1 mask
        g.ctx().wgrad_push(w, k, g.dev(A).data_ptr(), M, g.dev(B0).data_ptr(), N0, g.dev(m0).data_ptr(), 1,
                           g.dev(B1).data_ptr(), N1, g.dev(m1).data_ptr(), 0)
        ref0 += (B0 * m0).astype(np.float64).T @ A.astype(np.float64)
        ref1 += (B1 * m1).astype(np.float64).T @ A.astype(np.float64)
    C0_, C1_ = g.dev(C0), g.dev(C1)
    g.ctx().wgrad_flush(w, C0_.data_ptr(), M, C1_.data_ptr(), M)
    assert_close(g.host(C0_), ref0, TOL_REDUCE, floor=2.0, what="deferred dW0")
    assert_close(g.host(C1_), ref1, TOL_REDUCE, floor=2.0, what="deferred dW1")
    g.ctx().wgrad_flush(w, C0_.data_ptr(), M, C1_.data_ptr(), M)   # empty accumulator: no change
    assert_close(g.host(C0_), ref0, TOL_REDUCE, floor=2.0, what="deferred dW0 after empty flush")
    import torch
    torch.cuda.synchronize()
    g.ctx().wgrad_destroy(w)


# ------------------------------------------------------------------ ragged movers
def _tables(g, srcs, trgs, lens):
    import torch
    n = len(lens)
    sp = torch.tensor([t.data_ptr() for t in srcs], dtype=torch.int64, device="cuda")
    tp = torch.tensor([t.data_ptr() for t in trgs], dtype=torch.int64, device="cuda")
    ln = torch.tensor(lens, dtype=torch.int64, device="cuda")
    return n, sp, tp, ln


@pytest.mark.parametrize("n_seq", [1, 7, 300, 5000])
def test_parallel_memcpy(g, n_seq):
    import torch
    r = rng(170)
    lens = [int(v) for v in r.integers(1, 1100, n_seq)]
    src_all = g.dev(randn(r, sum(lens) + n_seq))
    dst_all = torch.zeros(sum(lens), device="cuda")
    srcs, trgs, off_s, off_d = [], [], 0, 0
    for k, L in enumerate(lens):
        srcs.append(src_all[off_s + 1:off_s + 1 + L])   # deliberately ragged alignment
        trgs.append(dst_all[off_d:off_d + L])
        off_s += L + 1
        off_d += L
    n, sp, tp, ln = _tables(g, srcs, trgs, lens)
    g.ctx().parallel_memcpy(n, max(lens), sp.data_ptr(), tp.data_ptr(), ln.data_ptr())
    want = torch.cat(srcs)
    assert torch.equal(dst_all, want)


@pytest.mark.parametrize("n_seq", [1, 9, 400, 4500])
def test_parallel_accumulate_with_shared_targets(g, n_seq):
    import torch
    r = rng(171)
    n_trg = max(1, n_seq // 3)
    L = [int(v) for v in r.integers(1, 600, n_trg)]
    L = [l - l % 4 if (k % 2 == 0 and l >= 4) else l for k, l in enumerate(L)]
    trg_bufs = [g.dev(randn(r, l)) for l in L]
    which = [int(v) for v in r.integers(0, n_trg, n_seq)]
    srcs = [g.dev(randn(r, L[w])) for w in which]
    want = [t.clone() for t in trg_bufs]
    for s, w in zip(srcs, which):      # ascending slice order, like the CPU loop (exec.cc:369-378)
        want[w] += s
    n, sp, tp, ln = _tables(g, srcs, [trg_bufs[w] for w in which], [L[w] for w in which])
    g.ctx().parallel_accumulate(n, max(L), sp.data_ptr(), tp.data_ptr(), ln.data_ptr())
    for a, b in zip(trg_bufs, want):   # later sort passes continue from the target's running value
        assert torch.equal(a, b)


# ------------------------------------------------------------------ MatrixMultiply / AffineTransform
# (bd, cols, rows) of {bias, A, B[, A2, B2]}; None = MatrixMultiply.  The first block are the shapes of the
# reference's gradient tests (tests/test-nodes.cc:431-505); the rest reach the tensor-pipe kernel.
AFFINE_SHAPES = {
    "multiply": [None, (1, 1, 3), (1, 3, 1)],
    "multiply_batch": [None, (1, 1, 3), (2, 3, 1)],
    "affine": [(1, 1, 3), (1, 1, 3), (1, 1, 1)],
    "affine_batch": [(1, 1, 3), (2, 1, 3), (1, 1, 1)],
    "affine_batch_col": [(1, 3, 1), (1, 1, 1), (2, 3, 1)],
    "affine_batch2": [(2, 3, 1), (1, 1, 1), (1, 3, 1)],
    "affine_batch3": [(1, 1, 3), (1, 3, 3), (2, 1, 3)],
    "two_products": [(1, 1, 4), (1, 3, 4), (3, 2, 3), (1, 5, 4), (3, 2, 5)],
    "both_batched": [(1, 1, 4), (3, 2, 4), (3, 5, 2)],
    "full_bias": [(5, 1, 130), (1, 70, 130), (5, 1, 70)],
    "projection": [(1, 1, 1000), (1, 256, 1000), (192, 1, 256)],          # b + R h, the output layer's shape class
    "projection_odd": [(1, 1, 1001), (1, 250, 1001), (67, 1, 250)],
    "projection_many_tiles": [(1, 1, 2100), (1, 200, 2100), (1700, 1, 200)],   # 17 x 14 tiles: the persistent kernel, bias epilogue
    "matmul_wide": [None, (1, 384, 512), (1, 640, 384)],
    "matmul_batched_left": [None, (3, 128, 256), (3, 130, 128)],
    "matrix_bias_tiled": [(1, 4, 256), (1, 128, 256), (6, 4, 128)],
}


@pytest.mark.parametrize("case", sorted(AFFINE_SHAPES))
def test_affine_matmul(oracle, g, capi, case):
    r = rng(sum(map(ord, case)))
    shapes = AFFINE_SHAPES[case]
    xs = [None if s is None else randn(r, *s, scale=0.5) for s in shapes]
    node = "matmul" if xs[0] is None else "affine_transform"
    args = xs[1:] if xs[0] is None else xs
    y_ref = oracle.affine_fwd(xs)
    dev_args = [g.dev(a) for a in args]
    ts = [g.T(d, [a.shape[2], a.shape[1]], a.shape[0]) for d, a in zip(dev_args, args)]
    y = g.dev(np.full_like(y_ref, 7.0))
    ty = g.T(y, [y_ref.shape[2], y_ref.shape[1]], y_ref.shape[0])
    g.ctx().fwd(node, ts, ty)
    assert_close(g.host(y), y_ref, TOL_REDUCE, floor=GEMM_FLOOR * 10, what=case + " fwd")
    dy = randn(r, *y_ref.shape)
    tdy = g.T(g.dev(dy), [dy.shape[2], dy.shape[1]], dy.shape[0])
    off = 1 if xs[0] is None else 0
    for i, a in enumerate(args):
        d0 = randn(r, *a.shape)
        want = oracle.affine_bwd(xs, dy, i + off, d0.copy())
        dx = g.dev(d0)
        g.ctx().bwd(node, ts, ty, tdy, i, g.T(dx, [a.shape[2], a.shape[1]], a.shape[0]))
        scale = max(1.0, float(np.abs(want).max()) * 0.05)
        assert_close(g.host(dx), want, TOL_REDUCE, floor=scale, what="%s bwd arg %d" % (case, i))
    assert g.ctx().device_errors() == 0


def test_affine_param_cache_matches_uncached(g, capi):
    """With the parameter cache on and the left operand flagged as a parameter, results are bitwise the same."""
    r = rng(77)
    R, h, b = randn(r, 1, 256, 1024, scale=0.1), randn(r, 128, 1, 256), randn(r, 1, 1, 1024)
    dev_args = [g.dev(a) for a in (b, R, h)]
    ts = [g.T(d, [a.shape[2], a.shape[1]], a.shape[0]) for d, a in zip(dev_args, (b, R, h))]
    y0, y1 = g.dev(np.zeros((128, 1, 1024), np.float32)), g.dev(np.zeros((128, 1, 1024), np.float32))
    g.ctx().fwd("affine_transform", ts, g.T(y0, [1024], 128))
    g.ctx().param_cache(True)
    try:
        at = capi.AffineAttrs(1)
        for _ in range(2):
            g.ctx().fwd("affine_transform", ts, g.T(y1, [1024], 128), at)
        assert np.array_equal(g.host(y0), g.host(y1))
    finally:
        g.ctx().param_cache(False)


def test_affine_rejects_bad_shapes(g, capi):
    r = rng(78)
    b, A, Bm = randn(r, 2, 1, 3), randn(r, 1, 4, 3), randn(r, 2, 5, 4)
    y = g.dev(np.zeros((2, 5, 3), np.float32))
    ts = [g.T(g.dev(a), [a.shape[2], a.shape[1]], a.shape[0]) for a in (b, A, Bm)]
    with pytest.raises(ValueError):     # mini-batched bias broadcast over columns: refused as on the CPU path
        g.ctx().fwd("affine_transform", ts, g.T(y, [3, 5], 2))
    with pytest.raises(ValueError):     # inner dimensions differ
        g.ctx().fwd("matmul", [ts[1], ts[1]], g.T(y, [3, 5], 2))


# ------------------------------------------------------------------ trainer update rules
TRAINER_HP = {
    "sgd": dict(lr=0.1), "momentum": dict(lr=0.01, momentum=0.9), "adagrad": dict(lr=0.1, eps=1e-20),
    "adadelta": dict(lr=1.0, eps=1e-6, rho=0.95), "rmsprop": dict(lr=0.1, eps=1e-20, rho=0.95),
    "adam": dict(lr=0.001, beta_1=0.9, beta_2=0.999, eps=1e-8), "amsgrad": dict(lr=0.001, beta_1=0.9, beta_2=0.999, eps=1e-8),
}
TRAINER_STATES = {"sgd": 0, "momentum": 1, "adagrad": 1, "adadelta": 2, "rmsprop": 1, "adam": 2, "amsgrad": 3}


@pytest.mark.parametrize("rule", sorted(TRAINER_HP))
@pytest.mark.parametrize("n,misalign", [(1, 0), (1003, 1), ((1 << 20) + 5, 0)])
def test_trainer_update(oracle, g, capi, rule, n, misalign):
    """Three consecutive updates (clipping active on the first) against the reference's statements on the CPU."""
    r = rng(500 + n)
    hp = TRAINER_HP[rule]
    p = randn(r, n)
    states = [np.abs(randn(r, n)) * 0.1 for _ in range(TRAINER_STATES[rule])]
    p_d = g.dev(p, misalign)
    s_d = [g.dev(s, misalign) for s in states]
    sumsq = g.dev(np.zeros(1, np.float32))
    for upd in range(3):
        grad = randn(r, n, scale=3.0 if upd == 0 else 0.01)
        g_d = g.dev(grad, misalign)
        gscale = oracle.clip_scale([grad], 5.0)
        oracle.trainer_update(rule, p, grad, states, gscale=gscale, wd=1.0, updates=upd, momentum=hp.get("momentum", 0.9),
                              eps=hp.get("eps", 1e-8), rho=hp.get("rho", 0.95), beta_1=hp.get("beta_1", 0.9),
                              beta_2=hp.get("beta_2", 0.999), lr=hp["lr"])
        hyper = capi.TrainerHyper(hp["lr"], 5.0, 1.0, hp.get("momentum", 0.9), hp.get("eps", 1e-8), hp.get("rho", 0.95),
                                  hp.get("beta_1", 0.9), hp.get("beta_2", 0.999), upd)
        g.ctx().squared_norm(g_d.data_ptr(), n, sumsq.data_ptr())
        g.ctx().trainer_update(rule, p_d.data_ptr(), g_d.data_ptr(), [s.data_ptr() for s in s_d], n, hyper, sumsq.data_ptr(),
                               zero_grads=(upd == 2))
        assert_close(g.host(p_d), p, 2e-5, floor=1.0, what="%s params after update %d" % (rule, upd))
        for k, s in enumerate(states):
            assert_close(g.host(s_d[k]), s, 2e-5, floor=0.1, what="%s state %d after update %d" % (rule, k, upd))
        if upd == 2:
            assert not g.host(g_d).any()
        elif rule not in ("sgd", "momentum"):
            assert_close(g.host(g_d), grad, 2e-5, floor=0.1, what="%s rewritten gradient" % rule)


# ------------------------------------------------------------------ glue nodes
def _t(g, d):
    """DyTensor of a torch tensor shaped (bd, ..., d1, d0)."""
    return g.T(d)


@pytest.mark.parametrize("shape,start,end,dim", [((4, 1, 8), 2, 6, 0), ((3, 5, 7), 1, 3, 1), ((2, 4, 130), 1, 129, 0),
                                                 ((64, 1, 4096), 1024, 2048, 0), ((2, 3, 4, 8), 1, 2, 2)])
def test_pick_range(oracle, g, capi, shape, start, end, dim):
    r = rng(610)
    x = randn(r, *shape)
    want = oracle.pick_range_fwd(x, start, end, dim)
    x_d, y_d = g.dev(x), g.dev(np.zeros_like(want))
    at = capi.PickRangeAttrs(start, end, dim)
    g.ctx().fwd("pick_range", [_t(g, x_d)], _t(g, y_d), at)
    assert np.array_equal(g.host(y_d), want)
    dy, dx0 = randn(r, *want.shape), randn(r, *shape)
    dx_d = g.dev(dx0)
    g.ctx().bwd("pick_range", [_t(g, x_d)], _t(g, y_d), _t(g, g.dev(dy)), 0, _t(g, dx_d), at)
    assert np.array_equal(g.host(dx_d), oracle.pick_range_bwd(shape, start, end, dim, dy, dx0.copy()))


@pytest.mark.parametrize("shapes,dimension", [([(4, 1, 8), (4, 1, 3)], 0), ([(3, 2, 4), (1, 5, 4)], 1),
                                              ([(32, 1, 512), (32, 1, 1024), (1, 1, 4)], 0), ([(2, 3, 4), (2, 3, 4)], 2)])
def test_concatenate(oracle, g, capi, shapes, dimension):
    r = rng(611)
    if dimension == 2:   # concatenating along a new trailing dimension: give the inputs an explicit size-1 axis
        shapes = [(s[0], 1) + s[1:] for s in shapes]
    xs = [randn(r, *s) for s in shapes]
    want = oracle.concatenate_fwd(xs, dimension)
    devs = [g.dev(x) for x in xs]
    y_d = g.dev(np.zeros_like(want))
    at = capi.DimAttrs(dimension)
    g.ctx().fwd("concatenate", [_t(g, d) for d in devs], _t(g, y_d), at)
    assert np.array_equal(g.host(y_d), want)
    dy = randn(r, *want.shape)
    dy_d = g.dev(dy)
    for i, x in enumerate(xs):
        d0 = randn(r, *x.shape)
        dx_d = g.dev(d0)
        g.ctx().bwd("concatenate", [_t(g, d) for d in devs], _t(g, y_d), _t(g, dy_d), i, _t(g, dx_d), at)
        assert_close(g.host(dx_d), oracle.concatenate_bwd(xs, dimension, dy, i, d0.copy()), TOL_REDUCE, floor=ACC_FLOOR,
                     what="concatenate bwd %d" % i)


@pytest.mark.parametrize("nargs,mixed", [(1, False), (2, False), (3, False), (4, False), (5, False), (7, False), (11, False), (50, False), (3, True)])
def test_sum_nary(oracle, g, capi, nargs, mixed):
    r = rng(612 + nargs)
    xs = [randn(r, 1 if (mixed and k == 1) else 4, 1, 300) for k in range(nargs)]
    want = oracle.sum_fwd(xs)
    devs = [g.dev(x) for x in xs]
    y_d = g.dev(np.zeros_like(want))
    g.ctx().fwd("sum", [_t(g, d) for d in devs], _t(g, y_d))
    if mixed:
        assert_close(g.host(y_d), want, TOL_CWISE, floor=1.0, what="sum mixed")
    else:
        assert np.array_equal(g.host(y_d), want)    # same grouping as the reference: bit-exact
    dy = randn(r, *want.shape)
    for i in (0, min(1, nargs - 1)):
        d0 = randn(r, *xs[i].shape)
        dx_d = g.dev(d0)
        g.ctx().bwd("sum", [_t(g, d) for d in devs], _t(g, y_d), _t(g, g.dev(dy)), i, _t(g, dx_d))
        assert_close(g.host(dx_d), oracle.sum_bwd(dy, d0.copy()), TOL_REDUCE, floor=ACC_FLOOR, what="sum bwd")


@pytest.mark.parametrize("shape,dims,ib", [((3, 4, 5), (0,), False), ((3, 4, 5), (1,), True), ((3, 4, 5), (0, 1), False),
                                           ((512, 1, 35), (), True), ((16, 1, 4096), (0,), False), ((2, 3, 4, 5), (2,), False),
                                           ((5, 2, 3), (0, 1), True)])
def test_sum_dim(oracle, g, capi, shape, dims, ib):
    r = rng(613)
    x = randn(r, *shape)
    want = oracle.sum_dim_fwd(x, dims, ib)
    x_d, y_d = g.dev(x), g.dev(np.zeros_like(want))
    at = capi.SumDimAttrs((C.c_uint * 2)(*(list(dims) + [0] * (2 - len(dims)))), len(dims), int(ib))
    nd = len(shape) - 1
    tx = g.T(x_d)
    ty = capi.DyTensor.of(y_d.data_ptr(), list(want.shape[1:][::-1]), want.shape[0])
    g.ctx().fwd("sum_dim", [tx], ty, at)
    assert_close(g.host(y_d), want, TOL_REDUCE, floor=1.0, what="sum_dim fwd")
    dy, d0 = randn(r, *want.shape), randn(r, *shape)
    dx_d = g.dev(d0)
    tdy = capi.DyTensor.of(g.dev(dy).data_ptr(), list(want.shape[1:][::-1]), want.shape[0])
    g.ctx().bwd("sum_dim", [tx], ty, tdy, 0, g.T(dx_d), at)
    assert_close(g.host(dx_d), oracle.sum_dim_bwd(shape, dims, ib, dy, d0.copy()), TOL_CWISE, floor=ACC_FLOOR, what="sum_dim bwd")


@pytest.mark.parametrize("shape", [(32, 1, 256), (1, 1, 1), (3, 7, 33), (2, 1, 100003)])
def test_squared_norm(oracle, g, capi, shape):
    r = rng(614)
    x = randn(r, *shape)
    want = oracle.squared_norm_fwd(x)
    x_d, y_d = g.dev(x), g.dev(np.zeros_like(want))
    g.ctx().fwd("squared_norm", [g.T(x_d)], g.T(y_d))
    assert_close(g.host(y_d), want, TOL_REDUCE, what="squared_norm fwd")
    dy, d0 = randn(r, *want.shape), randn(r, *shape)
    dx_d = g.dev(d0)
    g.ctx().bwd("squared_norm", [g.T(x_d)], g.T(y_d), g.T(g.dev(dy)), 0, g.T(dx_d))
    assert_close(g.host(dx_d), oracle.squared_norm_bwd(x, dy, d0.copy()), TOL_CWISE, floor=ACC_FLOOR, what="squared_norm bwd")


@pytest.mark.parametrize("name,c", [("negate", 0.0), ("constant_plus_x", 1e-8), ("constant_plus_x", 2.5), ("constant_minus_x", 1.0)])
def test_const_unary(g, capi, name, c):
    r = rng(615)
    x = randn(r, 3, 1001)
    want = {"negate": -x, "constant_plus_x": x + np.float32(c), "constant_minus_x": np.float32(c) - x}[name]
    x_d, y_d = g.dev(x), g.dev(np.zeros_like(x))
    at = None if name == "negate" else capi.ConstAttrs(c)
    g.ctx().fwd(name, [g.T(x_d)], g.T(y_d), at)
    assert np.array_equal(g.host(y_d), want)
    dy, d0 = randn(r, *x.shape), randn(r, *x.shape)
    dx_d = g.dev(d0)
    g.ctx().bwd(name, [g.T(x_d)], g.T(y_d), g.T(g.dev(dy)), 0, g.T(dx_d), at)
    assert np.array_equal(g.host(dx_d), d0 + dy if name == "constant_plus_x" else d0 - dy)


def test_random_bernoulli(g, capi):
    """Values are 0 or scale, the keep rate matches p, equal seeds repeat and different offsets differ."""
    n = 1 << 20
    y = g.dev(np.zeros((1, n + 3), np.float32))
    def draw(seed, offset, p=0.8, scale=1.25):
        g.ctx().fwd("random_bernoulli", [], g.T(y), capi.BernoulliAttrs(p, scale, seed, offset))
        return g.host(y).copy()
    a = draw(7, 0)
    assert set(np.unique(a)) == {0.0, 1.25}
    assert abs((a != 0).mean() - 0.8) < 4 * np.sqrt(0.8 * 0.2 / a.size)
    assert np.array_equal(a, draw(7, 0))
    b = draw(7, (n + 3 + 3) // 4)
    assert 0.6 < (a == b).mean() < 0.75          # independent draws agree with probability p^2 + (1-p)^2 = 0.68
    assert not np.array_equal(a, draw(8, 0))
    assert not draw(7, 0, p=0.0).any() and draw(7, 0, p=1.0, scale=2.0).min() == 2.0
    # neighbouring elements are uncorrelated
    k = (a[0, :-1] != 0).astype(np.float64); l = (a[0, 1:] != 0).astype(np.float64)
    assert abs(np.corrcoef(k, l)[0, 1]) < 0.01


@pytest.mark.parametrize("I,H,B,masks", [(512, 1024, 300, "full"), (256, 1024, 384, None), (512, 1024, 64, "full"), (256, 512, 96, None),
                                         (128, 1024, 700, "full")])
def test_lstm_fwd_fused_cell_epilogue(oracle, g, capi, I, H, B, masks):
    """The fused forward forms c and h in the epilogue of the gate product: inside the MMA kernel for shapes without a
    K split (the first two), in the split-K reduction for the next two, and in the persistent kernel for the last one
    (32 x 6 tiles, more than SMs).  Gates, c and h must equal the three nodes called one after the other bit for bit, and
    the oracle within the LSTM-state tolerance."""
    r = rng(155)
    x, h, c_prev = randn(r, B, I), randn(r, B, H, scale=0.5), randn(r, B, H, scale=0.5)
    Wx, Wh, b = glorot(r, 4 * H, I), glorot(r, 4 * H, H), randn(r, 4 * H, scale=0.1)
    mx = mh = None
    if masks:
        mx = ((r.random((B, I)) < 0.8) / 0.8).astype(np.float32)
        mh = ((r.random((B, H)) < 0.8) / 0.8).astype(np.float32)
    gates = oracle.lstm_gates_fwd([x], h, Wx, Wh, b, mx, mh)
    c_t = oracle.lstm_c_fwd(c_prev, gates)
    h_t = oracle.lstm_h_fwd(c_t, gates)
    at = capi.LstmGatesAttrs(1 if masks else 0, 0.0, 1.0)
    D = {k: g.dev(v) for k, v in dict(x=x, h=h, c=c_prev, Wx=Wx, Wh=Wh, b=b).items()}
    tm = [g.T(g.dev(mx)), g.T(g.dev(mh))] if masks else []
    tx, th_, tc_ = g.T(D["x"]), g.T(D["h"]), g.T(D["c"])
    tWx, tWh, tb = g.T(D["Wx"], [4 * H, I], 1), g.T(D["Wh"], [4 * H, H], 1), g.T(D["b"], [4 * H], 1)
    og, oc, oh = (g.dev(np.full_like(a, 9.0)) for a in (gates, c_t, h_t))
    g.ctx().lstm_fwd_fused(tx, th_, tc_, tWx, tWh, tb, tm[0] if masks else None, tm[1] if masks else None, at, g.T(og), g.T(oc), g.T(oh))
    ng, nc, nh = (g.dev(np.zeros_like(a)) for a in (gates, c_t, h_t))
    g.ctx().fwd("vanilla_lstm_gates", [tx, th_, tWx, tWh, tb] + tm, g.T(ng), at)
    g.ctx().fwd("vanilla_lstm_c", [tc_, g.T(ng)], g.T(nc))
    g.ctx().fwd("vanilla_lstm_h", [g.T(nc), g.T(ng)], g.T(nh))
    assert np.array_equal(g.host(og), g.host(ng))
    assert np.array_equal(g.host(oc), g.host(nc))
    assert np.array_equal(g.host(oh), g.host(nh))
    # K splits through a workspace and a second kernel instead of a cluster: the same bits
    wg, wc, wh = (g.dev(np.full_like(a, 5.0)) for a in (gates, c_t, h_t))
    try:
        g.ctx().cluster_splitk(0)
        g.ctx().lstm_fwd_fused(tx, th_, tc_, tWx, tWh, tb, tm[0] if masks else None, tm[1] if masks else None, at, g.T(wg), g.T(wc), g.T(wh))
    finally:
        g.ctx().cluster_splitk(1)
    assert np.array_equal(g.host(wg), g.host(og)) and np.array_equal(g.host(wc), g.host(oc)) and np.array_equal(g.host(wh), g.host(oh))
    assert_close(g.host(og), gates, TOL_REDUCE, floor=GEMM_FLOOR, what="gates")
    assert_close(g.host(oc), c_t, TOL_REDUCE, floor=GEMM_FLOOR, what="c")
    assert_close(g.host(oh), h_t, TOL_REDUCE, floor=GEMM_FLOOR, what="h")
    assert g.ctx().device_errors() == 0


@pytest.mark.parametrize("I,H,B", [(64, 64, 32), (128, 256, 64), (96, 64, 17)])
def test_lstm_fused_at_columns_equals_append(g, capi, I, H, B):
    """Two time steps through the *_fused_at pair (the forward call places the layer inputs at the step's columns of the
    accumulator, the backward call only the gate gradient, in reverse time order) give the weight gradients of the append
    form, in which every backward call pushes both."""
    r = rng(156)
    T = 2
    Wx, Wh, b = glorot(r, 4 * H, I), glorot(r, 4 * H, H), randn(r, 4 * H, scale=0.1)
    mx = ((r.random((B, I)) < 0.8) / 0.8).astype(np.float32)
    mh = ((r.random((B, H)) < 0.8) / 0.8).astype(np.float32)
    xs = [randn(r, B, I) for _ in range(T)]
    dhs = [randn(r, B, H) for _ in range(T)]
    at = capi.LstmGatesAttrs(1, 0.0, 1.0)
    D = {k: g.dev(v) for k, v in dict(Wx=Wx, Wh=Wh, b=b, mx=mx, mh=mh).items()}
    tWx, tWh, tb, tmx, tmh = g.T(D["Wx"], [4 * H, I], 1), g.T(D["Wh"], [4 * H, H], 1), g.T(D["b"], [4 * H], 1), g.T(D["mx"]), g.T(D["mh"])

    def run(mode):
        import torch
        w = g.ctx().wgrad_create(4 * H, I, H, T * B)
        try:
            h = [torch.zeros(B, H, device="cuda")] + [torch.empty(B, H, device="cuda") for _ in range(T)]
            c = [torch.zeros(B, H, device="cuda")] + [torch.empty(B, H, device="cuda") for _ in range(T)]
            gates = [torch.empty(B, 4 * H, device="cuda") for _ in range(T)]
            xd = [g.dev(x) for x in xs]
            for t in range(T):
                args = (g.T(xd[t]), g.T(h[t]), g.T(c[t]), tWx, tWh, tb, tmx, tmh, at, g.T(gates[t]), g.T(c[t + 1]), g.T(h[t + 1]))
                if mode == "at":
                    g.ctx().lstm_fwd_fused_at(*args, w, t * B)
                else:
                    g.ctx().lstm_fwd_fused(*args)
            dh = [g.dev(d) for d in dhs]
            dc = [torch.zeros(B, H, device="cuda") for _ in range(T)]
            dx = [torch.zeros(B, I, device="cuda") for _ in range(T)]
            db = torch.zeros(4 * H, device="cuda")
            for t in range(T - 1, -1, -1):
                args = (g.T(xd[t]), g.T(h[t]), g.T(c[t]), tWx, tWh, tmx, tmh, g.T(gates[t]), g.T(c[t + 1]), g.T(dh[t]), g.T(dc[t]), g.T(dx[t]),
                        None if t == 0 else g.T(dh[t - 1]), None if t == 0 else g.T(dc[t - 1]), None, None, g.T(db, [4 * H], 1), at)
                if mode == "at":
                    g.ctx().lstm_bwd_fused_at(*args, w, t * B)
                else:
                    g.ctx().lstm_bwd_fused(*args, w)
            dWx, dWh = torch.zeros(I, 4 * H, device="cuda"), torch.zeros(H, 4 * H, device="cuda")
            g.ctx().wgrad_flush(w, dWx.data_ptr(), 4 * H, dWh.data_ptr(), 4 * H)
            torch.cuda.synchronize()
            return [g.host(v) for v in (dWx, dWh, db, dx[0], dx[1], h[T], c[T])]
        finally:
            g.ctx().wgrad_destroy(w)

    a, p = run("at"), run("append")
    names = ["dWx", "dWh", "db", "dx0", "dx1", "h", "c"]
    for name, u, v in zip(names, a, p):
        if name in ("dWx", "dWh"):     # the steps sit in a different order along K: same sum, different association
            assert_close(u, v, TOL_REDUCE, floor=max(1.0, float(np.abs(v).max()) * 0.05), what=name)
        else:
            assert np.array_equal(u, v), name
    assert g.ctx().device_errors() == 0


@pytest.mark.parametrize("I,H,B,T,full", [(512, 1024, 256, 3, True), (256, 512, 64, 4, False), (128, 256, 32, 3, True)])
def test_lstm_presplit_inputs_equal_per_step_splits(g, capi, I, H, B, T, full):
    """dyb200_wgrad_pack_inputs (x of all steps split in one launch, h handed from epilogue to epilogue as operand planes)
    gives bitwise the states, gates and weight gradients of the same calls without it: tensor-pipe shapes with one tile
    per CTA, with K splits (batch 64) and a shape that takes the split through the workspace."""
    import torch
    r = rng(157)
    Wx, Wh, b = glorot(r, 4 * H, I), glorot(r, 4 * H, H), randn(r, 4 * H, scale=0.1)
    mB = B if full else 1
    mx = ((r.random((mB, I)) < 0.8) / 0.8).astype(np.float32)
    mh = ((r.random((mB, H)) < 0.8) / 0.8).astype(np.float32)
    xall = randn(r, T * B, I)
    dhs = [randn(r, B, H) for _ in range(T)]
    at = capi.LstmGatesAttrs(1, 0.0, 1.0)
    D = {k: g.dev(v) for k, v in dict(Wx=Wx, Wh=Wh, b=b, mx=mx, mh=mh, x=xall).items()}
    tWx, tWh, tb, tmx, tmh = g.T(D["Wx"], [4 * H, I], 1), g.T(D["Wh"], [4 * H, H], 1), g.T(D["b"], [4 * H], 1), g.T(D["mx"]), g.T(D["mh"])

    def run(presplit):
        ctx = g.ctx()
        w = ctx.wgrad_create(4 * H, I, H, T * B)
        try:
            launches0 = ctx.launches()
            if presplit:
                ctx.wgrad_pack_inputs(w, g.T(D["x"], [I], T * B), tmx, B)
            h = [torch.zeros(B, H, device="cuda")] + [torch.empty(B, H, device="cuda") for _ in range(T)]
            c = [torch.zeros(B, H, device="cuda")] + [torch.empty(B, H, device="cuda") for _ in range(T)]
            gates = [torch.empty(B, 4 * H, device="cuda") for _ in range(T)]
            xd = [D["x"][t * B:(t + 1) * B] for t in range(T)]
            for t in range(T):
                ctx.lstm_fwd_fused_at(g.T(xd[t]), g.T(h[t]), g.T(c[t]), tWx, tWh, tb, tmx, tmh, at, g.T(gates[t]), g.T(c[t + 1]), g.T(h[t + 1]), w, t * B)
            fwd_launches = ctx.launches() - launches0
            dh = [g.dev(d) for d in dhs]
            dc = [torch.zeros(B, H, device="cuda") for _ in range(T)]
            dx = [torch.zeros(B, I, device="cuda") for _ in range(T)]
            db = torch.zeros(4 * H, device="cuda")
            for t in range(T - 1, -1, -1):
                ctx.lstm_bwd_fused_at(g.T(xd[t]), g.T(h[t]), g.T(c[t]), tWx, tWh, tmx, tmh, g.T(gates[t]), g.T(c[t + 1]), g.T(dh[t]), g.T(dc[t]),
                                      g.T(dx[t]), None if t == 0 else g.T(dh[t - 1]), None if t == 0 else g.T(dc[t - 1]), None, None,
                                      g.T(db, [4 * H], 1), at, w, t * B)
            dWx, dWh = torch.zeros(I, 4 * H, device="cuda"), torch.zeros(H, 4 * H, device="cuda")
            ctx.wgrad_flush(w, dWx.data_ptr(), 4 * H, dWh.data_ptr(), 4 * H)
            torch.cuda.synchronize()
            return [g.host(v) for v in [dWx, dWh, db] + dx + h[1:] + c[1:] + gates], fwd_launches
        finally:
            ctx.wgrad_destroy(w)

    (a, la), (p, lp) = run(True), run(False)
    for k, (u, v) in enumerate(zip(a, p)):
        assert np.array_equal(u, v), k
    assert la < lp, (la, lp)          # fewer launches: no operand split per step after the first
    assert g.ctx().device_errors() == 0


def test_new_entry_points_reject_bad_arguments(g, capi):
    """Argument errors come back as the reference's exception class (std::invalid_argument), never as a fault."""
    r = rng(616)
    x = g.dev(randn(r, 2, 3, 5))
    y = g.dev(np.zeros((2, 3, 5), np.float32))
    with pytest.raises(ValueError):     # PickRange: end beyond the dimension (nodes-select.cc:208)
        g.ctx().fwd("pick_range", [g.T(x)], g.T(y), capi.PickRangeAttrs(2, 9, 0))
    with pytest.raises(ValueError):     # PickRange: empty range
        g.ctx().fwd("pick_range", [g.T(x)], g.T(y), capi.PickRangeAttrs(3, 3, 0))
    with pytest.raises(ValueError):     # Concatenate: the other dimensions differ
        g.ctx().fwd("concatenate", [g.T(x), g.T(g.dev(randn(r, 2, 4, 5)))], g.T(y), capi.DimAttrs(0))
    with pytest.raises(ValueError):     # Sum: mismatched input dimensions
        g.ctx().fwd("sum", [g.T(x), g.T(g.dev(randn(r, 2, 3, 4)))], g.T(y))
    with pytest.raises(ValueError):     # SumDimension: nothing to reduce
        g.ctx().fwd("sum_dim", [g.T(x)], g.T(y), capi.SumDimAttrs((C.c_uint * 2)(0, 0), 0, 0))
    with pytest.raises(ValueError):     # RandomBernoulli: p is not a probability
        g.ctx().fwd("random_bernoulli", [], g.T(y), capi.BernoulliAttrs(1.5, 1.0, 1, 0))
    p_, g_ = g.dev(randn(r, 16)), g.dev(randn(r, 16))
    hyper = capi.TrainerHyper(0.1, 5.0, 1.0, 0.9, 1e-8, 0.95, 0.9, 0.999, 0)
    with pytest.raises(ValueError):     # Adam without its two state buffers
        g.ctx().trainer_update("adam", p_.data_ptr(), g_.data_ptr(), [], 16, hyper)
    with pytest.raises(ValueError):     # a zero weight-decay divisor
        g.ctx().trainer_update("sgd", p_.data_ptr(), g_.data_ptr(), [], 16, capi.TrainerHyper(0.1, 5.0, 0.0, 0.9, 1e-8, 0.95, 0.9, 0.999, 0))
    assert g.ctx().device_errors() == 0


def test_two_devices_in_one_process(capi):
    """DyNet allows several devices per process (--dynet-devices).  What a context establishes on its device (shared-memory
    limits of the tensor-pipe kernels, cluster occupancy) must not leak to a second device: one tensor-path product on each."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = rng(1600)
    M, N, K = 512, 256, 2048
    A, Bm = randn(r, K, M), randn(r, N, K)
    ref = Bm.astype(np.float64) @ A.astype(np.float64)
    try:
        for dev in (0, 1):
            torch.cuda.set_device(dev)
            ctx = capi.Context(dev)
            A_, B_ = torch.from_numpy(A).cuda(dev), torch.from_numpy(Bm).cuda(dev)
            C_ = torch.zeros(N, M, device="cuda:%d" % dev)
            ctx.gemm(0, 0, M, N, K, A_.data_ptr(), M, B_.data_ptr(), K, C_.data_ptr(), M, 0)
            torch.cuda.synchronize(dev)
            assert_close(C_.cpu().numpy(), ref, TOL_REDUCE, floor=0.1 * K ** 0.5 + 1.0, what="product on device %d" % dev)
            assert ctx.device_errors() == 0
            ctx.close()
    finally:
        torch.cuda.set_device(0)
