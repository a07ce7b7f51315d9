"""GPU parity at the sizes of the benchmark configuration (2-layer LSTM language model, V = 10 000, E = 512, H = 1024,
T = 35): the code paths that only those sizes reach.

* The four long products of a training step, each through the C ABI at its full shape, against a float64 product formed
  on the device for a few hundred sampled rows and columns: the output layer (10 000 x 17 920 x 1 024 with the bias
  epilogue: persistent kernel, grouped tile order), the gradient of the output matrix (10 000 x 1 024 x 17 920,
  accumulate: persistent kernel with the partly filled last round run apart), a weight gradient of an LSTM layer
  (4 096 x 1 024 x 17 920, accumulate: accumulation chains of 560 k-blocks) and the gradient of the top-layer states
  (1 024 x 17 920 x 10 000, accumulate).
* One full-width training step (all 35 time steps, dropout masks fed in) at a per-GPU batch of 64 through the fused driver
  and its CUDA graph, against the CPU oracle: loss and every gradient tensor, each row held to its own scale.

The measured worst errors are printed at the end of the run (tests/conftest.py)."""
import numpy as np
import pytest

from util import assert_close, lm_grad_floors

pytestmark = pytest.mark.gpu

V, E, H, L, T = 10000, 512, 1024, 2, 35
NCOLS = 512 * T   # 17 920 columns: all time steps of the global batch


@pytest.fixture(scope="module")
def ctx():
    from dynet_b200 import capi
    c = capi.Context(0)
    yield c
    c.close()


def _sampled_check(torch, At, Bt, C_got, C0, bias, what):
    """At: (K, M), Bt: (N, K), C_got / C0: (N, M) device tensors (C order == column-major M x K, K x N, M x N).
    want = Bt @ At (+ C0) (+ bias per m), in float64 for 192 sampled rows m and 192 sampled columns n."""
    K, M = At.shape
    N = Bt.shape[0]
    gen = torch.Generator(device="cpu").manual_seed(7)
    rows = torch.randperm(M, generator=gen)[:192].sort().values.cuda()
    cols = torch.randperm(N, generator=gen)[:192].sort().values.cuda()
    # edges of the tile grid on purpose: first / last rows and columns
    rows[0], rows[-1] = 0, M - 1
    cols[0], cols[-1] = 0, N - 1
    want_r = Bt.double() @ At[:, rows].double()                    # (N, |rows|)
    want_c = Bt[cols].double() @ At.double()                       # (|cols|, M)
    if C0 is not None:
        want_r += C0[:, rows].double()
        want_c += C0[cols].double()
    if bias is not None:
        want_r += bias[rows].double()[None, :]
        want_c += bias.double()[None, :]
    rms = float(want_c.pow(2).mean().sqrt())
    for name, got, want in (("sampled rows", C_got[:, rows], want_r), ("sampled columns", C_got[cols], want_c)):
        g, w = got.double().cpu().numpy(), want.cpu().numpy()
        # 1e-4 class with the result's rms as the floor (an element of a K-term sum of products that cancel to ~0 cannot be
        # held to its own magnitude)
        assert_close(g, w, 1e-4, floor=rms, what="%s, %s (rms %.3g)" % (what, name, rms))


@pytest.mark.parametrize("shape", ["output_layer_bias", "dR_accumulate", "dW_lstm_accumulate", "dh_top_accumulate"])
def test_long_products_of_the_training_step(ctx, shape):
    import torch
    from dynet_b200 import capi
    gen = torch.Generator(device="cuda").manual_seed(hash(shape) % 1000 + 5)
    randn = lambda *s: torch.randn(*s, generator=gen, device="cuda", dtype=torch.float32)
    ctx.param_cache(True)
    try:
        if shape == "output_layer_bias":
            # r = bias + R * h over all columns: AffineTransform with R flagged as a parameter (as the driver does)
            M, N, K = V, NCOLS, H
            At, Bt, bias = randn(K, M) * 0.05, randn(N, K), randn(M)
            C = torch.empty(N, M, device="cuda")
            ts = [capi.DyTensor.of(bias.data_ptr(), [M], 1), capi.DyTensor.of(At.data_ptr(), [M, K], 1),
                  capi.DyTensor.of(Bt.data_ptr(), [K], N)]
            ctx.fwd("affine_transform", ts, capi.DyTensor.of(C.data_ptr(), [M], N), capi.AffineAttrs(1))
            torch.cuda.synchronize()
            _sampled_check(torch, At, Bt, C, None, bias, shape)
        else:
            M, N, K = {"dR_accumulate": (V, H, NCOLS), "dW_lstm_accumulate": (4 * H, H, NCOLS),
                       "dh_top_accumulate": (H, NCOLS, V)}[shape]
            At, Bt, C0 = randn(K, M), randn(N, K), randn(N, M)
            C = C0.clone()
            ctx.gemm(0, 0, M, N, K, At.data_ptr(), M, Bt.data_ptr(), K, C.data_ptr(), M, 1)
            torch.cuda.synchronize()
            _sampled_check(torch, At, Bt, C, C0, None, shape)
        assert ctx.device_errors() == 0
    finally:
        ctx.param_cache(False)


def test_full_width_lm_step_at_batch_64_matches_oracle(oracle):
    """Every kernel of the benchmark step at its real width (the 8-GPU share of the global batch): eager step, then the
    captured graph; the graph's loss and gradients against the oracle."""
    import torch
    from dynet_b200 import lm
    B = 64
    dims = dict(V=V, E=E, H=H, L=L, T=T, B=B)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        model = lm.LstmLm(device=0, seed=3, lr=0.1, clip=5.0, dropout=True, stream=stream.cuda_stream, **dims)
        tokens, masks = lm.synthetic_batch(dims, seed=4, dropout=0.2)
        params = model.params_host()
        loss_eager = model.forward_backward(tokens, masks)
        g_eager = model.grads_host()
        model.grads.zero_()
        model.set_graph(True)
        loss = model.forward_backward(tokens, masks)
        grads = model.grads_host()
        assert model.ctx.device_errors() == 0
        assert loss == loss_eager
        for a, b in zip(grads, g_eager):
            assert np.array_equal(a, b)
        model.close()
    g_ref = [np.zeros_like(p) for p in params]
    loss_ref, _ = oracle.lstm_lm_fwdbwd((V, E, H, L, T, B), params, g_ref, tokens, masks[0], masks[1])
    assert abs(loss - loss_ref) <= 1e-4 * abs(loss_ref), (loss, loss_ref)
    shapes = lm.param_shapes(V, E, H, L)
    names = ["C"] + [n + str(l + 1) for l in range(L) for n in ("Wx", "Wh", "b")] + ["R", "bias"]
    for name, got, (want, floor) in zip(names, grads, lm_grad_floors(g_ref, shapes)):
        assert_close(np.asarray(got).reshape(np.shape(want)), want, 1e-4, floor=floor, what="gradient of %s (per-row scale)" % name)
