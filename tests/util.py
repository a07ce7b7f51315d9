"""Shared helpers for the parity tests."""
import os

import numpy as np

# Parity classes (relative, with an absolute floor so values near zero such as
# sigma(-18) ~ 1.5e-8 do not demand sub-ulp agreement):
TOL_CWISE = 1e-5      # elementwise ops
TOL_REDUCE = 1e-4     # reductions, LSTM states, gradients


# Measured errors, for the log: test id -> (worst |err| / bound, its |err|, label).  tests/conftest.py prints one line per
# test at the end of the run, so the margin of every comparison can be read off a passing log.
RECORDS = {}


def _record(what, ratio, err):
    test = os.environ.get("PYTEST_CURRENT_TEST", "?").split(" ")[0]
    old = RECORDS.get(test)
    if old is None or ratio > old[0]:
        RECORDS[test] = (float(ratio), float(err), what)


def assert_close(got, want, tol, floor=1e-3, what=""):
    """|got - want| <= tol * max(|want|, floor) element-wise.  `floor` may be an array that broadcasts against `want`
    (a scale per row, see row_floor)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.all(np.isfinite(got)), what + ": non-finite values"
    err = np.abs(got - want)
    bound = tol * np.maximum(np.abs(want), floor)
    if err.size:
        with np.errstate(divide="ignore", invalid="ignore"):
            ratio = np.where(bound > 0, err / np.where(bound > 0, bound, 1.0), np.where(err > 0, np.inf, 0.0))
        k = int(np.argmax(ratio))
        _record(what, ratio.flat[k], err.flat[k])
    bad = err > bound
    if bad.any():
        k = int(np.argmax(ratio))
        raise AssertionError(
            "%s: %d/%d outside tol %g; worst idx %s got %r want %r (err %g, bound %g)"
            % (what, bad.sum(), bad.size, tol, np.unravel_index(k, got.shape), got.flat[k],
               want.flat[k], err.flat[k], np.broadcast_to(bound, err.shape).flat[k]))


def row_floor(want, axis, rel=0.0):
    """Per-row comparison scale for a 2-D gradient: max |want| along `axis` (kept as a broadcastable array), so that every
    row (an embedding row, a gate row) is held to its own magnitude and a row that must stay zero has to be exactly
    zero.  `rel` > 0 adds that fraction of the global maximum as a lower limit for every row."""
    want = np.asarray(want, np.float64)
    f = np.abs(want).max(axis=axis, keepdims=True)
    if rel > 0.0:
        f = np.maximum(f, rel * float(np.abs(want).max()))
    return f


def lm_grad_floors(grads_ref, shapes, rel=1e-3):
    """Comparison scales for the gradient tensors of the LSTM language model (flat, column-major, in parameter order:
    embedding table (E, V), per layer Wx (4H, I), Wh (4H, H), b, then R (V, H), bias): per embedding row, per gate row,
    per vocabulary row (never below `rel` of the tensor's largest element, except that an all-zero row must stay exactly
    zero); vectors keep one scale.  Returns (reshaped want, floor) pairs."""
    out = []
    for k, (w, (rows, cols)) in enumerate(zip(grads_ref, shapes)):
        if cols == 1:
            out.append((w, max(1e-6, float(np.abs(w).max()))))
            continue
        w2 = np.asarray(w).reshape(cols, rows)            # C order (cols, rows) == column-major rows x cols
        axis = 1 if k == 0 else 0                          # embedding: one scale per column (= per id); else per row
        f = row_floor(w2, axis)
        out.append((w2, np.where(f > 0, np.maximum(f, rel * float(np.abs(w2).max())), 0.0)))
    return out


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def randn(r, *shape, scale=1.0):
    return (r.standard_normal(shape) * scale).astype(np.float32)


def zipf_ids(r, n, vocab, s=1.1):
    """n draws from p(k) ~ k^-s over ranks 1..vocab (inverse CDF), as 0-based ids."""
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** (-s))
    cdf /= cdf[-1]
    u = r.random(n)
    return np.minimum(np.searchsorted(cdf, u), vocab - 1).astype(np.uint32)


def glorot(r, rows, cols):
    """DyNet's default ParameterInitGlorot for a matrix: U(+-sqrt(6/(r+c)))."""
    a = np.sqrt(6.0 / (rows + cols))
    return r.uniform(-a, a, size=(cols, rows)).astype(np.float32)  # (cols, rows) C-order == column-major rows x cols
