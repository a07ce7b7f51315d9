"""The sequence-persistent LSTM kernels (one launch per layer and direction for all time steps) against the per-step calls
they replace: gates, cell and hidden states of every step, dE/dx, dE/dh and dE/dc of every step, the bias gradient and the
weight gradients that the recorded operand planes produce must agree BIT FOR BIT, and the forward values must match the CPU
oracle (the backward values of the per-step calls are checked against it in test_gpu_parity.py / test_gpu_lm.py).
Shapes: one tile per CTA (batch 512 and 384), K splits reduced inside a thread-block cluster with 128-column tiles (batch 256:
2 splits, batch 128: 4) and with 64-column tiles (batch 64), batch-1 masks, a layer whose input is narrower than its state,
and shapes the kernels decline (per-step calls inside)."""
import numpy as np
import pytest

from util import assert_close, glorot, randn, rng

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


def _run(g, capi, D, I, H, B, T, dropout, seq, dhs):
    """Forward over T steps (seq: one dyb200_vanilla_lstm_seq_fwd call; else pack_inputs + T per-step calls), then the
    per-step backward calls and the deferred weight-gradient products.  Returns host copies of everything."""
    import torch
    ctx = g.ctx()
    at = capi.LstmGatesAttrs(1 if dropout else 0, 0.0, 1.0)
    tWx, tWh, tb = g.T(D["Wx"], [4 * H, I], 1), g.T(D["Wh"], [4 * H, H], 1), g.T(D["b"], [4 * H], 1)
    tmx = g.T(D["mx"]) if dropout else None
    tmh = g.T(D["mh"]) if dropout else None
    w = ctx.wgrad_create(4 * H, I, H, T * B)
    try:
        zeros = torch.zeros(B, H, device="cuda")
        hs, cs, gates = (torch.full((T * B, H), 7.0, device="cuda"), torch.full((T * B, H), 7.0, device="cuda"),
                         torch.full((T * B, 4 * H), 7.0, device="cuda"))
        l0 = ctx.launches()
        if seq:
            ctx.lstm_seq_fwd(g.T(D["x"], [I], T * B), g.T(zeros), g.T(zeros), tWx, tWh, tb, tmx, tmh, at,
                             g.T(gates, [4 * H], T * B), g.T(cs, [H], T * B), g.T(hs, [H], T * B), w, T)
        else:
            ctx.wgrad_pack_inputs(w, g.T(D["x"], [I], T * B), tmx, B)
            for t in range(T):
                sl = slice(t * B, (t + 1) * B)
                hp = zeros if t == 0 else hs[(t - 1) * B:t * B]
                cp = zeros if t == 0 else cs[(t - 1) * B:t * B]
                ctx.lstm_fwd_fused_at(g.T(D["x"][sl]), g.T(hp), g.T(cp), tWx, tWh, tb, tmx, tmh, at, g.T(gates[sl]), g.T(cs[sl]),
                                      g.T(hs[sl]), w, t * B)
        fwd_launches = ctx.launches() - l0
        dh = g.dev(np.concatenate(dhs))                      # dE/dh_t of every step, step t in rows [t B, (t + 1) B)
        dc = torch.zeros(T * B, H, device="cuda")
        dx = torch.zeros(T * B, I, device="cuda")
        db = torch.zeros(4 * H, device="cuda")
        l1 = ctx.launches()
        if seq:
            ctx.lstm_seq_bwd(g.T(D["x"], [I], T * B), g.T(zeros), g.T(zeros), tWx, tWh, tmx, tmh, at, g.T(gates, [4 * H], T * B),
                             g.T(cs, [H], T * B), g.T(hs, [H], T * B), g.T(dh, [H], T * B), g.T(dc, [H], T * B), g.T(dx, [I], T * B),
                             None, None, g.T(db, [4 * H], 1), w, T)
        else:
            for t in range(T - 1, -1, -1):
                sl, pr = slice(t * B, (t + 1) * B), slice((t - 1) * B, t * B)
                hp = zeros if t == 0 else hs[pr]
                cp = zeros if t == 0 else cs[pr]
                ctx.lstm_bwd_fused_at(g.T(D["x"][sl]), g.T(hp), g.T(cp), tWx, tWh, tmx, tmh, g.T(gates[sl]), g.T(cs[sl]), g.T(dh[sl]),
                                      g.T(dc[sl]), g.T(dx[sl]), None if t == 0 else g.T(dh[pr]), None if t == 0 else g.T(dc[pr]), None, None,
                                      g.T(db, [4 * H], 1), at, w, t * B)
        bwd_launches = ctx.launches() - l1
        dWx, dWh = torch.zeros(I, 4 * H, device="cuda"), torch.zeros(H, 4 * H, device="cuda")
        ctx.wgrad_flush(w, dWx.data_ptr(), 4 * H, dWh.data_ptr(), 4 * H)
        torch.cuda.synchronize()
        out = dict(gates=g.host(gates), c=g.host(cs), h=g.host(hs), dWx=g.host(dWx), dWh=g.host(dWh), db=g.host(db),
                   dx=g.host(dx), dh=g.host(dh), dc=g.host(dc))
        return out, (fwd_launches, bwd_launches)
    finally:
        ctx.wgrad_destroy(w)


def _same(seq, per):
    """Everything the sequence calls produce, bit for bit what the per-step calls produce (the per-step backward call uses the
    sequence kernel's K splits for shapes the kernel takes, so both add the same partial sums in the same order)."""
    bad = ["%s (max |diff| %.3g)" % (k, float(np.abs(seq[k] - per[k]).max())) for k in sorted(seq) if not np.array_equal(seq[k], per[k])]
    assert not bad, "the sequence calls differ from the per-step calls in " + ", ".join(bad)


@pytest.mark.parametrize("I,H,B,T,dropout,full,one_kernel,bwd_kernel", [
    (512, 1024, 512, 4, True, True, True, True),      # benchmark layer 1 on one GPU: one tile per CTA, 128 CTAs
    (1024, 1024, 64, 6, True, True, True, True),      # benchmark layer 2 on 8 GPUs: 64-column tiles, 4 K splits per cluster
    (512, 1024, 64, 5, True, False, True, True),      # layer 1 on 8 GPUs, batch-1 masks
    (1024, 1024, 128, 3, True, True, True, True),     # 4 GPUs: 128-column tiles, 4 K splits per cluster
    (512, 1024, 256, 3, False, True, True, True),     # 2 GPUs: 2 K splits per cluster, no dropout
    (256, 1024, 384, 3, True, True, True, True),      # three column blocks, one tile per CTA
    (256, 512, 384, 3, True, True, False, True),      # 3 K splits: 48 clusters of 3 do not fit on the GPU at once -> per-step calls
    (128, 256, 96, 3, True, True, False, False),       # 96 columns are not whole tiles: per-step calls inside
    (32, 64, 8, 3, True, True, False, False),          # far below the tensor path
])
def test_sequence_calls_equal_per_step_calls(oracle, g, capi, I, H, B, T, dropout, full, one_kernel, bwd_kernel):
    r = rng(700 + B + I)
    Wx, Wh, b = glorot(r, 4 * H, I), glorot(r, 4 * H, H), randn(r, 4 * H, scale=0.1)
    mB = B if full else 1
    mx = ((r.random((mB, I)) < 0.8) / 0.8).astype(np.float32)
    mh = ((r.random((mB, H)) < 0.8) / 0.8).astype(np.float32)
    xall = randn(r, T * B, I)
    dhs = [randn(r, B, H) for _ in range(T)]
    D = {k: g.dev(v) for k, v in dict(Wx=Wx, Wh=Wh, b=b, mx=mx, mh=mh, x=xall).items()}
    ctx = g.ctx()
    ctx.param_cache(True)
    try:
        per, l_per = _run(g, capi, D, I, H, B, T, dropout, False, dhs)     # (first: it also fills the parameter cache)
        seq, l_seq = _run(g, capi, D, I, H, B, T, dropout, True, dhs)
        ctx.sequence_kernels(False)
        off, l_off = _run(g, capi, D, I, H, B, T, dropout, True, dhs)      # the entry point with the kernel switched off
    finally:
        ctx.sequence_kernels(True)
        ctx.param_cache(False)
    assert ctx.device_errors() == 0
    _same(seq, per)
    for k in sorted(seq):
        assert np.array_equal(off[k], per[k]), "%s: the sequence call (kernel off) differs from the per-step calls" % k
    if one_kernel:
        assert l_seq[0] == 3 < l_per[0], (l_seq, l_per)   # operand split of x, of h0 (the counter reset is a memset), one kernel
    else:
        assert l_seq[0] <= l_per[0]
    if bwd_kernel:
        # the kernel, the sum of its bias-gradient partials, and the per-step form of step 0
        assert l_seq[1] < l_per[1] and l_seq[1] <= 2 + 4, (l_seq, l_per)
    else:
        assert l_seq[1] <= l_per[1]
    # and the values themselves: the oracle's node chain
    h = np.zeros((B, H), np.float32)
    c = np.zeros((B, H), np.float32)
    for t in range(T):
        gt = oracle.lstm_gates_fwd([xall[t * B:(t + 1) * B]], h, Wx, Wh, b, mask_x=mx if dropout else None, mask_h=mh if dropout else None)
        c = oracle.lstm_c_fwd(c, gt)
        h = oracle.lstm_h_fwd(c, gt)
        assert_close(seq["h"][t * B:(t + 1) * B], h, 1e-4, floor=0.1, what="h_%d" % t)
        assert_close(seq["c"][t * B:(t + 1) * B], c, 1e-4, floor=0.1, what="c_%d" % t)
        assert_close(seq["gates"][t * B:(t + 1) * B], gt, 1e-4, floor=0.1, what="gates_%d" % t)


def test_sequence_forward_twice_in_a_row_and_many_steps(g, capi):
    """35 steps (the benchmark's sequence length), called twice: the hand-over counters start from zero every time."""
    I, H, B, T = 512, 1024, 64, 35
    r = rng(735)
    Wx, Wh, b = glorot(r, 4 * H, I), glorot(r, 4 * H, H), randn(r, 4 * H, scale=0.1)
    mx = ((r.random((B, I)) < 0.8) / 0.8).astype(np.float32)
    mh = ((r.random((B, H)) < 0.8) / 0.8).astype(np.float32)
    xall = randn(r, T * B, I)
    dhs = [randn(r, B, H) for _ in range(T)]
    D = {k: g.dev(v) for k, v in dict(Wx=Wx, Wh=Wh, b=b, mx=mx, mh=mh, x=xall).items()}
    ctx = g.ctx()
    ctx.param_cache(True)
    try:
        a, _ = _run(g, capi, D, I, H, B, T, True, True, dhs)
        b2, _ = _run(g, capi, D, I, H, B, T, True, True, dhs)
        per, _ = _run(g, capi, D, I, H, B, T, True, False, dhs)
    finally:
        ctx.param_cache(False)
    assert ctx.device_errors() == 0
    _same(a, per)
    _same(b2, per)
