"""Shape rules (dim_forward) of every node class the host layer mirrors, checked on the CPU against the rules of the
reference (read from its dim_forward bodies; the file:line of each rule is cited beside the cases).  The rules decide the
shape of every tensor a DyNet graph allocates, so a drop-in has to reproduce them exactly, error cases included."""
import ctypes as C

import pytest

from dynet_b200 import capi
from dynet_b200.lm import host_lib


def dim_forward(node, xs, iargs=()):
    """xs: list of (dims tuple, batch size).  Returns (dims tuple, batch size) or raises ValueError with the message."""
    L = host_lib()
    L.dyb200h_dim_forward.restype = C.c_int
    L.dyb200h_dim_forward.argtypes = [C.c_char_p, C.POINTER(capi.DyTensor), C.c_int, C.POINTER(C.c_int32), C.c_int,
                                      C.POINTER(capi.DyTensor), C.c_char_p, C.c_size_t]
    arr = (capi.DyTensor * max(1, len(xs)))(*[capi.DyTensor.of(None, d, b) for d, b in xs])
    ia = (C.c_int32 * max(1, len(iargs)))(*iargs)
    out = capi.DyTensor()
    err = C.create_string_buffer(512)
    rc = L.dyb200h_dim_forward(node.encode(), arr, len(xs), ia, len(iargs), C.byref(out), err, 512)
    if rc == capi.EINVAL:
        raise ValueError(err.value.decode())
    assert rc == 0, err.value.decode()
    return tuple(out.d[k] for k in range(out.nd)), out.bd


OK = [
    # unary nodes keep the shape (nodes-trig.cc, nodes-activations.cc, nodes-arith-unary.cc, nodes-arith-const.cc)
    ("Tanh", [((4, 3), 2)], (), ((4, 3), 2)),
    ("LogisticSigmoid", [((5,), 1)], (), ((5,), 1)),
    ("Rectify", [((2, 2, 2), 3)], (), ((2, 2, 2), 3)),
    ("ExponentialLinearUnit", [((7,), 4)], (), ((7,), 4)),
    ("Negate", [((3, 1), 2)], (), ((3, 1), 2)),
    ("ConstantPlusX", [((3,), 2)], (), ((3,), 2)),
    ("ConstantMinusX", [((3,), 2)], (), ((3,), 2)),
    # cwise binary with broadcasting (nodes-arith-cwise.cc:21-34, :168-182, :319-333)
    ("CwiseMultiply", [((4, 3), 2), ((4, 3), 2)], (), ((4, 3), 2)),
    ("CwiseMultiply", [((4, 3), 5), ((4, 1), 1)], (), ((4, 3), 5)),
    ("CwiseMultiply", [((1, 3), 1), ((4, 3), 2)], (), ((4, 3), 2)),
    ("CwiseSum", [((4,), 2), ((4, 3), 1)], (), ((4, 3), 2)),
    ("CwiseQuotient", [((4, 3), 2), ((1, 3), 1)], (), ((4, 3), 2)),
    # softmax family (nodes-softmaxes.cc:21-26, :144-148; nodes-logsumexp.cc:25-33, :112-121; nodes-pickneglogsoftmax.cc:32-44)
    ("Softmax", [((10, 4), 3)], (1,), ((10, 4), 3)),
    ("LogSoftmax", [((10,), 3)], (), ((10,), 3)),
    ("LogSumExp", [((6,), 1), ((6,), 4), ((6,), 1)], (), ((6,), 4)),
    ("LogSumExpDimension", [((5, 7), 2)], (0,), ((7,), 2)),
    ("LogSumExpDimension", [((5, 7), 2)], (1,), ((5,), 2)),
    ("LogSumExpDimension", [((5,), 2)], (0,), ((1,), 2)),          # Dim::delete_dim of the only dimension (dim.h:212-228)
    ("PickNegLogSoftmax", [((45,), 8)], (8,), ((1,), 8)),
    # normalisation (nodes-normalization.cc:20-24; nodes-moments.cc:166-179, :419-431; dim.h:234-256)
    ("WeightNormalization", [((16, 8), 1), ((1,), 1)], (), ((16, 8), 1)),
    ("MomentDimension", [((4096,), 32)], (1, 0, 0), ((1,), 32)),
    ("MomentDimension", [((3, 4, 5), 2)], (2, 0, 0, 2), ((4,), 2)),
    ("MomentDimension", [((3, 4), 6)], (1, 1), ((3, 4), 1)),
    ("StdDimension", [((3, 4), 6)], (0, 1), ((3,), 6)),
    ("StdDimension", [((3, 4), 6)], (1, 0, 1), ((1,), 1)),
    ("LayerNormFused", [((64,), 5), ((64,), 1), ((64,), 1)], (), ((64,), 5)),
    # embedding and fused LSTM (param-nodes.cc:164-166; nodes-lstm.cc:24-59, :541-548, :629-636)
    ("LookupNode", [], (512, 17), ((512,), 17)),
    ("VanillaLSTMGates", [((3,), 2), ((5,), 2), ((20, 3), 1), ((20, 5), 1), ((20,), 1)], (0,), ((20,), 2)),
    ("VanillaLSTMGates", [((2,), 2), ((1,), 2), ((5,), 2), ((20, 3), 1), ((20, 5), 1), ((20,), 1)], (0,), ((20,), 2)),
    ("VanillaLSTMGates", [((3,), 2), ((5,), 2), ((20, 3), 1), ((20, 5), 1), ((20,), 1), ((3,), 2), ((5,), 1)], (1,), ((20,), 2)),
    ("VanillaLSTMC", [((5,), 2), ((20,), 2)], (), ((5,), 2)),
    ("VanillaLSTMH", [((5,), 2), ((20,), 2)], (), ((5,), 2)),
    # glue (nodes-select.cc:206-212; nodes-concat.cc:25-40; nodes-arith-sum.cc:22-33, :182-193; nodes-norms.cc:22-25)
    ("PickRange", [((20,), 3)], (5, 10, 0), ((5,), 3)),
    ("PickRange", [((4, 6), 1)], (2, 6, 1), ((4, 4), 1)),
    ("Concatenate", [((3,), 2), ((4,), 1), ((1,), 2)], (0,), ((8,), 2)),
    ("Concatenate", [((3, 2), 1), ((3, 5), 1)], (1,), ((3, 7), 1)),
    ("Concatenate", [((3,), 1), ((3,), 1)], (1,), ((3, 2), 1)),
    ("Sum", [((3, 2), 1), ((3, 2), 4)], (), ((3, 2), 4)),
    ("SumDimension", [((3, 4), 5)], (0, 1), ((3,), 5)),
    ("SumDimension", [((3, 4), 5)], (1,), ((3, 4), 1)),
    ("SumDimension", [((3, 4), 5)], (1, 0, 1), ((1,), 1)),
    ("SquaredNorm", [((9, 2), 3)], (), ((1,), 3)),
    # products (nodes-matrixmultiply.cc:21-27; nodes-affinetransform.cc:23-38)
    ("MatrixMultiply", [((4, 3), 1), ((3,), 5)], (), ((4,), 5)),
    ("MatrixMultiply", [((4, 3), 2), ((3, 6), 1)], (), ((4, 6), 2)),
    ("AffineTransform", [((4,), 1), ((4, 3), 1), ((3,), 7)], (), ((4,), 7)),
    ("AffineTransform", [((4,), 1), ((4, 3), 1), ((3, 2), 1), ((4, 5), 1), ((5, 2), 3)], (), ((4, 2), 3)),
    ("AffineTransform", [((4,), 2)], (), ((4,), 2)),
]


@pytest.mark.parametrize("node,xs,iargs,want", OK, ids=["%s-%d" % (c[0], k) for k, c in enumerate(OK)])
def test_dim_forward_follows_the_reference(node, xs, iargs, want):
    assert dim_forward(node, xs, iargs) == want


BAD = [
    ("Tanh", [((3,), 1), ((3,), 1)], (), "input count"),
    ("CwiseMultiply", [((4, 3), 1), ((4, 2), 1)], (), "needs to match or equal 1"),
    ("CwiseSum", [((4,), 2), ((4,), 3)], (), "batch size"),
    ("CwiseQuotient", [((1, 3), 1), ((4, 3), 1)], (), "CwiseQuotient"),          # only the right side may broadcast
    ("CwiseQuotient", [((4, 3), 1), ((4, 3), 2)], (), "batch size"),
    ("Softmax", [((2, 3, 4), 1)], (0,), "2 or fewer"),
    ("Softmax", [((5,), 1)], (1,), "reduction dimension"),
    ("LogSoftmax", [((2, 3, 4), 1)], (), "2 or fewer"),
    ("LogSumExp", [((6,), 1), ((5,), 1)], (), "Mismatched"),
    ("LogSumExpDimension", [((5, 7), 1)], (2,), "smaller than"),
    ("PickNegLogSoftmax", [((45, 2), 8)], (8,), "Bad input dimensions"),
    ("PickNegLogSoftmax", [((45,), 8)], (7,), "number of IDs"),
    ("WeightNormalization", [((4, 4), 1), ((2,), 1)], (), "gain"),
    ("MomentDimension", [((3, 4), 1)], (0, 0, 0), "Order of moment"),
    ("MomentDimension", [((3, 4), 1)], (1, 0), "At least one dimension"),
    ("MomentDimension", [((3, 4), 1)], (1, 0, 2), "out of bounds"),
    ("StdDimension", [((2, 2, 2, 2), 1)], (0, 0), "order 3"),
    ("VanillaLSTMGates", [((3,), 2), ((5,), 2), ((20, 4), 1), ((20, 5), 1), ((20,), 1)], (0,), "inconsistent dimension"),
    ("VanillaLSTMGates", [((3,), 2), ((5,), 2), ((16, 3), 1), ((20, 5), 1), ((20,), 1)], (0,), "Wx dim 0"),
    ("VanillaLSTMGates", [((3,), 2), ((5,), 3), ((20, 3), 1), ((20, 5), 1)], (0,), "input count"),
    ("VanillaLSTMC", [((5,), 2), ((19,), 2)], (), "4 times"),
    ("VanillaLSTMH", [((10,), 2), ((20,), 4)], (), "equal batch size"),       # (sizes agree, batch sizes do not)
    ("PickRange", [((20,), 1)], (5, 25, 0), "PickRange"),
    ("PickRange", [((20,), 1)], (5, 5, 0), "PickRange"),
    ("Concatenate", [((3, 2), 1), ((4, 5), 1)], (1,), "Concatenate"),
    ("Sum", [((3,), 1), ((4,), 1)], (), "Mismatched"),
    ("SumDimension", [((3, 4), 5)], (0,), "At least one dimension"),
    ("SumDimension", [((3, 4), 5)], (0, 2), "out of bounds"),
    ("MatrixMultiply", [((4, 3), 1), ((2, 6), 1)], (), "Mismatched"),
    ("AffineTransform", [((4,), 1), ((4, 3), 1)], (), "Bad number of inputs"),
    ("AffineTransform", [((5,), 1), ((4, 3), 1), ((3,), 1)], (), "Bad dimensions"),
]


@pytest.mark.parametrize("node,xs,iargs,msg", BAD, ids=["%s-%d" % (c[0], k) for k, c in enumerate(BAD)])
def test_dim_forward_rejects_what_the_reference_rejects(node, xs, iargs, msg):
    with pytest.raises(ValueError, match=msg):
        dim_forward(node, xs, iargs)
