"""Shared helpers for the parity tests."""
import numpy as np

# Parity classes (relative, with an absolute floor so values near zero such as
# sigma(-18) ~ 1.5e-8 do not demand sub-ulp agreement):
TOL_CWISE = 1e-5      # elementwise ops
TOL_REDUCE = 1e-4     # reductions, LSTM states, gradients


def assert_close(got, want, tol, floor=1e-3, what=""):
    """|got - want| <= tol * max(|want|, floor) element-wise."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.all(np.isfinite(got)), what + ": non-finite values"
    err = np.abs(got - want)
    bound = tol * np.maximum(np.abs(want), floor)
    bad = err > bound
    if bad.any():
        k = np.argmax(err / bound)
        raise AssertionError(
            "%s: %d/%d outside tol %g; worst idx %s got %r want %r (err %g, bound %g)"
            % (what, bad.sum(), bad.size, tol, np.unravel_index(k, got.shape), got.flat[k],
               want.flat[k], err.flat[k], bound.flat[k]))


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
