"""Config-5 parity case: the BiLSTM tagger of examples/tagger/train_tag-bilstm.cc:60-117 over ragged sentences.

CPU side: every sentence on its own, node by node through the oracle (batch size 1), as the reference's CPU build
runs it.  GPU side: what the autobatching executor makes of the same graph (dynet/exec.cc:481-725) - nodes of equal
depth are batched over the sentences that are still running, so the batch shrinks with the time step, the hidden
states of all tokens are collected into one token-major matrix with the ragged copy (combine_tensors ->
gpu::parallel_memcpy), the tag layer runs once over all tokens, and the gradients flow back through the ragged
accumulate (accumulate_tensors -> gpu::parallel_accumulate).  Everything goes through the C ABI."""
import ctypes as C

import numpy as np
import pytest

from util import TOL_REDUCE, assert_close, glorot, randn, rng, row_floor, zipf_ids

pytestmark = pytest.mark.gpu


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


def _mat(a):
    """(rows, cols) parameter stored column-major -> the oracle's (bd=1, cols, rows) view of the same memory."""
    return a.reshape(1, a.shape[0], a.shape[1])


def oracle_tagger(oracle, P, sents, tags):
    """Loss and gradients, one sentence at a time.  P: dict of parameters (numpy, column-major as (cols, rows))."""
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
                x = oracle.lookup_fwd(P["emb"], np.array([sent[t]], np.uint32))
                gates = oracle.lstm_gates_fwd([x], h, P["Wx_" + d], P["Wh_" + d], P["b_" + d])
                c_new = oracle.lstm_c_fwd(c, gates)
                h_new = oracle.lstm_h_fwd(c_new, gates)
                states[(d, t)] = (x, h, c, gates, c_new, h_new)
                h, c = h_new, c_new
        dh_tok = {}
        for t in range(n):
            hf, hr = states[("f", t)][5], states[("r", t)][5]
            xs1 = [P["thbias"].reshape(1, 1, -1), _mat(P["l2th"]), hf.reshape(1, 1, H), _mat(P["r2th"]), hr.reshape(1, 1, H)]
            pre = oracle.affine_fwd(xs1)
            th = oracle.unary_fwd("tanh", pre)
            xs2 = [P["tbias"].reshape(1, 1, -1), _mat(P["th2t"]), th]
            logits = oracle.affine_fwd(xs2)
            ids = np.array([tg[t]], np.uint32)
            l, z = oracle.pnls_fwd(logits.reshape(1, -1), ids)
            loss += float(l[0])
            dlog = oracle.pnls_bwd(logits.reshape(1, -1), ids, z, np.ones(1, np.float32), np.zeros((1, logits.size), np.float32))
            dlog = dlog.reshape(logits.shape)
            oracle.affine_bwd(xs2, dlog, 0, G["tbias"].reshape(1, 1, -1))
            oracle.affine_bwd(xs2, dlog, 1, _mat(G["th2t"]))
            dth = oracle.affine_bwd(xs2, dlog, 2, np.zeros_like(th))
            dpre = oracle.unary_bwd("tanh", pre, th, dth, np.zeros_like(pre))
            oracle.affine_bwd(xs1, dpre, 0, G["thbias"].reshape(1, 1, -1))
            oracle.affine_bwd(xs1, dpre, 1, _mat(G["l2th"]))
            oracle.affine_bwd(xs1, dpre, 3, _mat(G["r2th"]))
            dh_tok[("f", t)] = oracle.affine_bwd(xs1, dpre, 2, np.zeros((1, 1, H), np.float32)).reshape(1, H)
            dh_tok[("r", t)] = oracle.affine_bwd(xs1, dpre, 4, np.zeros((1, 1, H), np.float32)).reshape(1, H)
        for d in ("f", "r"):
            order = list(range(n)) if d == "f" else list(range(n - 1, -1, -1))
            dh_c = np.zeros((1, H), np.float32)
            dc_c = np.zeros((1, H), np.float32)
            for t in reversed(order):
                x, h_prev, c_prev, gates, c_new, h_new = states[(d, t)]
                dh = dh_tok[(d, t)] + dh_c
                dc = dc_c.copy()
                oracle.lstm_h_bwd(c_new, gates, dh, 0, dc)
                dg = np.zeros_like(gates)
                oracle.lstm_h_bwd(c_new, gates, dh, 1, dg)
                dc_c = oracle.lstm_c_bwd(c_prev, gates, dc, 0, np.zeros((1, H), np.float32))
                oracle.lstm_c_bwd(c_prev, gates, dc, 1, dg)
                dx = oracle.lstm_gates_bwd([x], h_prev, P["Wx_" + d], P["Wh_" + d], gates, dg, 0, np.zeros_like(x))
                dh_c = oracle.lstm_gates_bwd([x], h_prev, P["Wx_" + d], P["Wh_" + d], gates, dg, 1, np.zeros((1, H), np.float32))
                oracle.lstm_gates_bwd([x], h_prev, P["Wx_" + d], P["Wh_" + d], gates, dg, 2, G["Wx_" + d])
                oracle.lstm_gates_bwd([x], h_prev, P["Wx_" + d], P["Wh_" + d], gates, dg, 3, G["Wh_" + d])
                oracle.lstm_gates_bwd([x], h_prev, P["Wx_" + d], P["Wh_" + d], gates, dg, 4, G["b_" + d])
                oracle.lookup_accumulate_grads(G["emb"], np.array([sent[t]], np.uint32), dx)
    return loss, G


def _tables(torch, ptrs_src, ptrs_trg, n, length):
    sp = torch.tensor(ptrs_src, dtype=torch.int64, device="cuda")
    tp = torch.tensor(ptrs_trg, dtype=torch.int64, device="cuda")
    ln = torch.full((n,), length, dtype=torch.int64, device="cuda")
    return sp, tp, ln


def gpu_tagger(g, capi, P, sents, tags):
    """The same loss and gradients with time-step batching; sentences are sorted by length (longest first), so the
    sentences still running at step k are the first B_k of the batch."""
    import torch
    ctx = g.ctx()
    E, H = P["emb"].shape[1], P["b_f"].size // 4
    TH, NT, V = P["thbias"].size, P["tbias"].size, P["emb"].shape[0]
    S, lens = len(sents), [len(s) for s in sents]
    assert lens == sorted(lens, reverse=True)
    Lmax = lens[0]
    D = {k: g.dev(v) for k, v in P.items()}
    Gd = {k: g.dev(np.zeros_like(v)) for k, v in P.items()}
    keep = []   # pointer tables and id arrays must outlive the asynchronous kernels
    zeros = torch.zeros(S, H, device="cuda")
    at = capi.LstmGatesAttrs(0, 0.0, 1.0)
    f32 = dict(dtype=torch.float32, device="cuda")
    steps = {}
    for d in ("f", "r"):
        tWx, tWh, tb = g.T(D["Wx_" + d], [4 * H, E], 1), g.T(D["Wh_" + d], [4 * H, H], 1), g.T(D["b_" + d], [4 * H], 1)
        for k in range(Lmax):
            B = sum(1 for n in lens if n > k)
            ids = np.array([sents[s][k if d == "f" else lens[s] - 1 - k] for s in range(B)], np.uint32)
            st = dict(B=B, ids=ids, x=torch.empty(B, E, **f32), gates=torch.empty(B, 4 * H, **f32), c=torch.empty(B, H, **f32),
                      h=torch.empty(B, H, **f32), dh=torch.zeros(B, H, **f32), dc=torch.zeros(B, H, **f32), dx=torch.zeros(B, E, **f32),
                      aux=torch.empty(B, **f32))
            steps[(d, k)] = st
            _, p = g.u32(ids)
            keep.append(p)
            ctx.fwd("lookup", [], g.T(st["x"], [E], B), capi.LookupAttrs(D["emb"].data_ptr(), V, p, B, 1.0), st["aux"].data_ptr())
            hp = zeros if k == 0 else steps[(d, k - 1)]["h"]
            cp = zeros if k == 0 else steps[(d, k - 1)]["c"]
            ctx.lstm_fwd_fused(g.T(st["x"], [E], B), g.T(hp, [H], B), g.T(cp, [H], B), tWx, tWh, tb, None, None, at,
                               g.T(st["gates"], [4 * H], B), g.T(st["c"], [H], B), g.T(st["h"], [H], B))
    # token-major matrices of the hidden states: token n = (sentence s, position t)
    toks = [(s, t) for s in range(S) for t in range(lens[s])]
    N = len(toks)
    hf, hr = torch.empty(N, H, **f32), torch.empty(N, H, **f32)
    dhf, dhr = torch.zeros(N, H, **f32), torch.zeros(N, H, **f32)

    def slot(d, s, t, what):
        k = t if d == "f" else lens[s] - 1 - t
        return steps[(d, k)][what].data_ptr() + 4 * H * s

    for d, dst in (("f", hf), ("r", hr)):
        sp, tp, ln = _tables(torch, [slot(d, s, t, "h") for s, t in toks], [dst.data_ptr() + 4 * H * n for n in range(N)], N, H)
        keep += [sp, tp, ln]
        ctx.parallel_memcpy(N, H, sp.data_ptr(), tp.data_ptr(), ln.data_ptr())
    # tag layer over all tokens at once
    pre, th, logits = torch.empty(N, TH, **f32), torch.empty(N, TH, **f32), torch.empty(N, NT, **f32)
    xs1 = [g.T(D["thbias"], [TH], 1), g.T(D["l2th"], [TH, H], 1), g.T(hf, [H], N), g.T(D["r2th"], [TH, H], 1), g.T(hr, [H], N)]
    ctx.fwd("affine_transform", xs1, g.T(pre, [TH], N))
    ctx.fwd("tanh", [g.T(pre, [TH], N)], g.T(th, [TH], N))
    xs2 = [g.T(D["tbias"], [NT], 1), g.T(D["th2t"], [NT, TH], 1), g.T(th, [TH], N)]
    ctx.fwd("affine_transform", xs2, g.T(logits, [NT], N))
    tag_ids = np.array([tags[s][t] for s, t in toks], np.uint32)
    _, tp_ = g.u32(tag_ids)
    keep.append(tp_)
    errs, aux = torch.empty(N, 1, **f32), torch.empty(3 * N, **f32)
    pat = capi.PickAttrs(tp_, N)
    ctx.fwd("pickneglogsoftmax", [g.T(logits, [NT], N)], g.T(errs, [1], N), pat, aux.data_ptr())
    total = torch.empty(1, 1, **f32)
    ctx.fwd("sum_dim", [g.T(errs, [1], N)], g.T(total, [1], 1), capi.SumDimAttrs((C.c_uint * 2)(0, 0), 0, 1))
    # backward
    ones, dlog = torch.ones(N, 1, **f32), torch.zeros(N, NT, **f32)
    ctx.bwd("pickneglogsoftmax", [g.T(logits, [NT], N)], g.T(errs, [1], N), g.T(ones, [1], N), 0, g.T(dlog, [NT], N), pat, aux.data_ptr())
    dth, dpre = torch.zeros(N, TH, **f32), torch.zeros(N, TH, **f32)
    ctx.bwd("affine_transform", xs2, g.T(logits, [NT], N), g.T(dlog, [NT], N), 0, g.T(Gd["tbias"], [NT], 1))
    ctx.bwd("affine_transform", xs2, g.T(logits, [NT], N), g.T(dlog, [NT], N), 1, g.T(Gd["th2t"], [NT, TH], 1))
    ctx.bwd("affine_transform", xs2, g.T(logits, [NT], N), g.T(dlog, [NT], N), 2, g.T(dth, [TH], N))
    ctx.bwd("tanh", [g.T(pre, [TH], N)], g.T(th, [TH], N), g.T(dth, [TH], N), 0, g.T(dpre, [TH], N))
    for i, out in ((0, g.T(Gd["thbias"], [TH], 1)), (1, g.T(Gd["l2th"], [TH, H], 1)), (2, g.T(dhf, [H], N)),
                   (3, g.T(Gd["r2th"], [TH, H], 1)), (4, g.T(dhr, [H], N))):
        ctx.bwd("affine_transform", xs1, g.T(pre, [TH], N), g.T(dpre, [TH], N), i, out)
    for d, src in (("f", dhf), ("r", dhr)):
        sp, tp, ln = _tables(torch, [src.data_ptr() + 4 * H * n for n in range(N)], [slot(d, s, t, "dh") for s, t in toks], N, H)
        keep += [sp, tp, ln]
        ctx.parallel_accumulate(N, H, sp.data_ptr(), tp.data_ptr(), ln.data_ptr())
    for d in ("f", "r"):
        tWx, tWh = g.T(D["Wx_" + d], [4 * H, E], 1), g.T(D["Wh_" + d], [4 * H, H], 1)
        gWx, gWh, gb = g.T(Gd["Wx_" + d], [4 * H, E], 1), g.T(Gd["Wh_" + d], [4 * H, H], 1), g.T(Gd["b_" + d], [4 * H], 1)
        for k in range(Lmax - 1, -1, -1):
            st = steps[(d, k)]
            B = st["B"]
            prev = steps.get((d, k - 1))
            hp = zeros if k == 0 else prev["h"]
            cp = zeros if k == 0 else prev["c"]
            ctx.lstm_bwd_fused(g.T(st["x"], [E], B), g.T(hp, [H], B), g.T(cp, [H], B), tWx, tWh, None, None, g.T(st["gates"], [4 * H], B),
                               g.T(st["c"], [H], B), g.T(st["dh"], [H], B), g.T(st["dc"], [H], B), g.T(st["dx"], [E], B),
                               None if k == 0 else g.T(prev["dh"], [H], B), None if k == 0 else g.T(prev["dc"], [H], B), gWx, gWh, gb, at)
            ids_dev = torch.from_numpy(st["ids"].view(np.int32)).cuda()
            keep.append(ids_dev)
            ctx.lookup_accumulate_grads(st["ids"], ids_dev.data_ptr(), st["dx"].data_ptr(), Gd["emb"].data_ptr(), E, V)
    torch.cuda.synchronize()
    assert ctx.device_errors() == 0
    return float(total.item()), {k: g.host(v) for k, v in Gd.items()}, N


def tagger_floor(name, want):
    """Comparison scale of a tagger gradient: per embedding row (numpy (V, E): axis 1), per row of a weight matrix (numpy
    (cols, rows): axis 0), never below 1 % of the tensor's largest entry; vectors: 5 % of their largest entry."""
    if want.ndim == 2:
        return row_floor(want, 1 if name == "emb" else 0, rel=1e-2)
    return max(float(np.abs(want).max()) * 0.05, 1e-6)


@pytest.mark.parametrize("dims", [dict(V=50, E=16, H=8, TH=6, NT=5, S=7, lo=1, hi=6),
                                  dict(V=2000, E=128, H=256, TH=32, NT=45, S=64, lo=5, hi=30)])
def test_bilstm_tagger_autobatched_vs_per_sentence(oracle, g, capi, dims):
    r = rng(500 + dims["S"])
    V, E, H, TH, NT, S = (dims[k] for k in ("V", "E", "H", "TH", "NT", "S"))
    lens = sorted((int(v) for v in r.integers(dims["lo"], dims["hi"] + 1, S)), reverse=True)
    sents = [[int(v) for v in zipf_ids(r, n, V)] for n in lens]
    tags = [[int(v) for v in r.integers(0, NT, n)] for n in lens]
    P = {"emb": glorot(r, E, V)}   # Dim({E}, V): numpy (V, E)
    for d in ("f", "r"):
        P["Wx_" + d], P["Wh_" + d], P["b_" + d] = glorot(r, 4 * H, E), glorot(r, 4 * H, H), randn(r, 4 * H, scale=0.1)
    P["l2th"], P["r2th"], P["thbias"] = glorot(r, TH, H), glorot(r, TH, H), randn(r, TH, scale=0.1)
    P["th2t"], P["tbias"] = glorot(r, NT, TH), randn(r, NT, scale=0.1)
    want_loss, want = oracle_tagger(oracle, P, sents, tags)
    got_loss, got, n_tok = gpu_tagger(g, capi, P, sents, tags)
    assert n_tok == sum(lens)
    assert abs(got_loss - want_loss) <= 1e-4 * abs(want_loss)
    for k in sorted(want):
        assert_close(got[k], want[k], TOL_REDUCE, floor=tagger_floor(k, want[k]), what="d" + k + " (per-row scale)")
