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


def oracle_tagger(oracle, P, sents, tags):
    return oracle.tagger_fwdbwd(P, sents, tags)


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


# ------------------------------------------------------------------ the C++ driver (host/tagger.cc)
def _params(r, V, E, H, TH, NT):
    P = {"emb": glorot(r, E, V)}
    for d in ("f", "r"):
        P["Wx_" + d], P["Wh_" + d], P["b_" + d] = glorot(r, 4 * H, E), glorot(r, 4 * H, H), randn(r, 4 * H, scale=0.1)
    P["l2th"], P["r2th"], P["thbias"] = glorot(r, TH, H), glorot(r, TH, H), randn(r, TH, scale=0.1)
    P["th2t"], P["tbias"] = glorot(r, NT, TH), randn(r, NT, scale=0.1)
    return P


def _driver(tg, P, dims, S, N, Lmax):
    V, E, H, TH, NT = dims
    return tg.Tagger(V, E, H, TH, NT, max_sentences=S, max_tokens=N, max_len=Lmax, device=0, params=[P[k] for k in tg.NAMES])


def _split(lens, words, tags):
    off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    return ([[int(v) for v in words[off[s]:off[s + 1]]] for s in range(len(lens))],
            [[int(v) for v in tags[off[s]:off[s + 1]]] for s in range(len(lens))])


@pytest.mark.parametrize("dims,S,lo,hi", [((50, 16, 8, 6, 5), 7, 1, 6), ((2000, 128, 256, 32, 45), 48, 5, 30)])
def test_tagger_driver_matches_per_sentence_oracle(oracle, dims, S, lo, hi):
    """The C++ driver (autobatched schedule, deferred weight-gradient products, folded embedding scatter) against the oracle
    running every sentence on its own: loss and all 12 gradient tensors, every row at its own scale.  Two passes in a row:
    gradients accumulate, the second pass reuses every buffer."""
    from dynet_b200 import tagger as tg
    V, E, H, TH, NT = dims
    r = rng(800 + S)
    P = _params(r, V, E, H, TH, NT)
    lens, words, tags = tg.synthetic_corpus(S, V, NT, seed=5 + S, lo=lo, hi=hi)
    sents, tgs = _split(lens, words, tags)
    want_loss, want = oracle.tagger_fwdbwd(P, sents, tgs)
    m = _driver(tg, P, dims, S, int(lens.sum()), int(lens[0]))
    loss = m.forward_backward(lens, words, tags)
    got = m.grads_host()
    assert abs(loss - want_loss) <= 1e-4 * abs(want_loss)
    for k in sorted(want):
        assert_close(got[k].reshape(want[k].shape), want[k], TOL_REDUCE, floor=tagger_floor(k, want[k]), what="d" + k + " (per-row scale)")
    loss2 = m.forward_backward(lens, words, tags)          # accumulates: twice the gradient
    assert loss2 == loss
    got2 = m.grads_host()
    for k in sorted(want):
        assert_close(got2[k].reshape(want[k].shape), 2.0 * want[k], TOL_REDUCE, floor=2.0 * tagger_floor(k, want[k]), what="2 x d" + k)
    assert m.ctx.device_errors() == 0
    m.close()


def test_tagger_driver_at_the_benchmark_size(oracle):
    """2 048 sentences of 5 .. 100 words, V = 20 000, E = 128, H = 256, 45 tags in ONE pass (107 k tokens).  The oracle would
    need minutes for that, so: (1) parity on a sample of 24 of the sentences run as their own mini-batch; (2) additivity,
    which does not depend on the size: the loss and gradients of the full batch equal those of its even- plus its
    odd-numbered sentences (each half still sorted by length), to the 1e-4 class."""
    from dynet_b200 import tagger as tg
    dims = (20000, 128, 256, 32, 45)
    V, E, H, TH, NT = dims
    S = 2048
    r = rng(900)
    P = _params(r, V, E, H, TH, NT)
    lens, words, tags = tg.synthetic_corpus(S, V, NT, seed=77)
    N, Lmax = int(lens.sum()), int(lens[0])
    off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)

    def subset(idx):
        idx = np.asarray(idx)
        return (np.ascontiguousarray(lens[idx]), np.ascontiguousarray(np.concatenate([words[off[s]:off[s + 1]] for s in idx])),
                np.ascontiguousarray(np.concatenate([tags[off[s]:off[s + 1]] for s in idx])))

    m = _driver(tg, P, dims, S, N, Lmax)
    loss_full = m.forward_backward(lens, words, tags)
    g_full = m.grads_host()
    assert m.ctx.device_errors() == 0
    m.grads.zero_()
    halves = [subset(np.arange(0, S, 2)), subset(np.arange(1, S, 2))]
    loss_sum = sum(m.forward_backward(*h) for h in halves)          # gradients accumulate over the two passes
    g_sum = m.grads_host()
    assert abs(loss_full - loss_sum) <= 1e-4 * abs(loss_full)
    for k in sorted(g_full):
        shape = (-1, g_full[k].size) if g_full[k].ndim == 1 else g_full[k].shape
        a, b = g_full[k].reshape(shape), g_sum[k].reshape(shape)
        assert_close(a, b, TOL_REDUCE, floor=max(float(np.abs(b).max()) * 0.01, 1e-6), what="additivity of d" + k)
    # parity on a sample
    m.grads.zero_()
    idx = np.sort(rng(901).choice(S, 24, replace=False))
    sl, sw, st = subset(idx)
    loss_s = m.forward_backward(sl, sw, st)
    got = m.grads_host()
    sents, tgs = _split(sl, sw, st)
    want_loss, want = oracle.tagger_fwdbwd(P, sents, tgs)
    assert abs(loss_s - want_loss) <= 1e-4 * abs(want_loss)
    for k in sorted(want):
        assert_close(got[k].reshape(want[k].shape), want[k], TOL_REDUCE, floor=tagger_floor(k, want[k]), what="sample: d" + k)
    ms, host_ms = m.mover_ms()
    assert m.ctx.device_errors() == 0
    m.close()


def test_tagger_driver_rejects_bad_input():
    from dynet_b200 import capi, tagger as tg
    dims = (50, 16, 8, 6, 5)
    m = tg.Tagger(*dims, max_sentences=4, max_tokens=16, max_len=8, device=0, seed=1)
    lens = np.array([2, 3], np.uint32)                                 # not sorted, longest first
    words = np.zeros(5, np.uint32)
    with pytest.raises(capi.InvalidArgument, match="sorted"):
        m.launch_forward_backward(lens, words, words.copy())
    lens = np.array([3, 2], np.uint32)
    bad = words.copy(); bad[1] = 50
    with pytest.raises(capi.InvalidArgument, match="Out-of-bounds"):
        m.launch_forward_backward(lens, bad, words.copy())
    with pytest.raises(capi.InvalidArgument, match="tokens"):
        m.launch_forward_backward(np.array([8, 8, 8], np.uint32), np.zeros(24, np.uint32), np.zeros(24, np.uint32))
    m.close()
