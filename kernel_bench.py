"""Per-kernel timing of the memory-bound nodes at the sizes of BASELINE configs 2 and 3.

    python kernel_bench.py [--only NAME] [--iters 20] [--small]

Each case is called through the C ABI `iters` times on ROTATING buffer sets whose total footprint
exceeds the 126 MB L2 (so every call reads its inputs from HBM).  The calls are captured once into a
CUDA graph on the library's stream and the graph launch is timed with CUDA events after warm-up, so
the figure is device time of the kernels back to back, free of per-call host overhead.  Output: one JSON line per case with the algorithmic bytes of one call,
the average duration, achieved GB/s and its fraction of the measured copy bandwidth (MEASURED_PEAKS.json,
fallback 6650 GB/s) and of the nominal 8000 GB/s.  `--small` shrinks every case to a few hundred MB total so
that a profiler capture of one launch ends quickly.
"""
import argparse
import ctypes as C
import json
import os

import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from dynet_b200 import capi  # noqa: E402

L2_BYTES = 126 * 1024 * 1024


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class Case:
    def __init__(self, name, nbytes, make, call, footprint):
        self.name, self.nbytes, self.make, self.call, self.footprint = name, nbytes, make, call, footprint


def T(t, dims, bd):
    return capi.DyTensor.of(t.data_ptr(), dims, bd)


def build_cases(torch, ctx, small):
    cases = []
    dev = "cuda"
    R, Ccols = (1024, 4096)              # config 3: [1024, 4096] tensors; row-wise ops see Dim({4096}, 1024)
    n = R * Ccols
    S = 4 * n

    def unary(name, attrs=None):
        def make():
            return dict(x=torch.randn(R, Ccols, device=dev), y=torch.empty(R, Ccols, device=dev),
                        dy=torch.randn(R, Ccols, device=dev), dx=torch.zeros(R, Ccols, device=dev))
        def fwd(b):
            ctx.fwd(name, [T(b["x"], [Ccols], R)], T(b["y"], [Ccols], R), attrs)
        def bwd(b):
            ctx.bwd(name, [T(b["x"], [Ccols], R)], T(b["y"], [Ccols], R), T(b["dy"], [Ccols], R), 0, T(b["dx"], [Ccols], R), attrs)
        cases.append(Case(name + "_fwd", 2 * S, make, fwd, 4 * S))
        cases.append(Case(name + "_bwd", 4 * S, make, bwd, 4 * S))

    unary("tanh"); unary("logistic"); unary("rectify"); unary("elu", capi.EluAttrs(1.0, 1.0))
    # yardstick, not a library kernel: a plain device copy of one config-3 tensor (what 2S of traffic can reach at this size;
    # the 6551 GB/s peak was measured on 2 GB buffers)
    def mk_copy():
        return dict(x=torch.randn(R, Ccols, device=dev), y=torch.empty(R, Ccols, device=dev))
    cases.append(Case("copy_reference_1024x4096", 2 * S, mk_copy, lambda b: b["y"].copy_(b["x"]), 2 * S))

    # the same kernels on 8x larger tensors ([8192, 4096], 134 MB each): launch ramp-up and tail no longer dominate
    RL = 8 * R
    SLg = 4 * RL * Ccols
    def mk_large():
        return dict(x=torch.randn(RL, Ccols, device=dev), y=torch.empty(RL, Ccols, device=dev))
    cases.append(Case("tanh_fwd_8192x4096", 2 * SLg, mk_large,
                      lambda b: ctx.fwd("tanh", [T(b["x"], [Ccols], RL)], T(b["y"], [Ccols], RL)), 2 * SLg))
    cases.append(Case("softmax_rows4096_fwd_8192x4096", 2 * SLg, mk_large,
                      lambda b: ctx.fwd("softmax", [T(b["x"], [Ccols], RL)], T(b["y"], [Ccols], RL), capi.DimAttrs(0)), 2 * SLg))
    def mk_large_ln():
        d = mk_large()
        d.update(g=torch.rand(Ccols, device=dev) + 0.5, b=torch.randn(Ccols, device=dev) * 0.1)
        return d
    cases.append(Case("layer_norm_fwd_8192x4096", 2 * SLg, mk_large_ln,
                      lambda b: ctx.fwd("layer_norm", [T(b["x"], [Ccols], RL), T(b["g"], [Ccols], 1), T(b["b"], [Ccols], 1)],
                                        T(b["y"], [Ccols], RL)), 2 * SLg))

    def mk_cmult():
        return dict(a=torch.randn(R, Ccols, device=dev), b=torch.randn(R, Ccols, device=dev), y=torch.empty(R, Ccols, device=dev),
                    dy=torch.randn(R, Ccols, device=dev), da=torch.zeros(R, Ccols, device=dev))
    cases.append(Case("cmult_fwd", 3 * S, mk_cmult,
                      lambda b: ctx.fwd("cmult", [T(b["a"], [Ccols], R), T(b["b"], [Ccols], R)], T(b["y"], [Ccols], R)), 5 * S))
    cases.append(Case("cmult_bwd_arg0", 4 * S, mk_cmult,
                      lambda b: ctx.bwd("cmult", [T(b["a"], [Ccols], R), T(b["b"], [Ccols], R)], T(b["y"], [Ccols], R),
                                        T(b["dy"], [Ccols], R), 0, T(b["da"], [Ccols], R)), 5 * S))

    sm0 = capi.DimAttrs(0)
    sm1 = capi.DimAttrs(1)
    def mk_sm():
        return dict(x=torch.randn(R, Ccols, device=dev), y=torch.empty(R, Ccols, device=dev),
                    dy=torch.randn(R, Ccols, device=dev), dx=torch.zeros(R, Ccols, device=dev))
    cases.append(Case("softmax_rows4096_fwd", 2 * S, mk_sm,
                      lambda b: ctx.fwd("softmax", [T(b["x"], [Ccols], R)], T(b["y"], [Ccols], R), sm0), 4 * S))
    cases.append(Case("softmax_rows4096_bwd", 4 * S, mk_sm,
                      lambda b: ctx.bwd("softmax", [T(b["x"], [Ccols], R)], T(b["y"], [Ccols], R), T(b["dy"], [Ccols], R), 0,
                                        T(b["dx"], [Ccols], R), sm0), 4 * S))
    # Dim({1024, 4096}) reduced along dim 1 (strided)
    cases.append(Case("softmax_dim1_1024x4096_fwd", 2 * S, mk_sm,
                      lambda b: ctx.fwd("softmax", [T(b["x"], [R, Ccols], 1)], T(b["y"], [R, Ccols], 1), sm1), 4 * S))

    def mk_ln():
        return dict(x=torch.randn(R, Ccols, device=dev), g=torch.rand(Ccols, device=dev) + 0.5, b=torch.randn(Ccols, device=dev) * 0.1,
                    y=torch.empty(R, Ccols, device=dev), dy=torch.randn(R, Ccols, device=dev), dx=torch.zeros(R, Ccols, device=dev))
    def ln_xs(b):
        return [T(b["x"], [Ccols], R), T(b["g"], [Ccols], 1), T(b["b"], [Ccols], 1)]
    cases.append(Case("layer_norm_fwd", 2 * S, mk_ln, lambda b: ctx.fwd("layer_norm", ln_xs(b), T(b["y"], [Ccols], R)), 4 * S))
    cases.append(Case("layer_norm_bwd_x", 4 * S, mk_ln,
                      lambda b: ctx.bwd("layer_norm", ln_xs(b), T(b["y"], [Ccols], R), T(b["dy"], [Ccols], R), 0, T(b["dx"], [Ccols], R)), 4 * S))
    # the same 16.8 MB tensor as 4096 columns of 1024 elements (a hidden layer of 1024 units, 4096 batch columns): a warp per column
    def mk_ln2():
        return dict(x=torch.randn(Ccols, R, device=dev), g=torch.rand(R, device=dev) + 0.5, b=torch.randn(R, device=dev) * 0.1,
                    y=torch.empty(Ccols, R, device=dev), dy=torch.randn(Ccols, R, device=dev), dx=torch.zeros(Ccols, R, device=dev))
    def ln2_xs(b):
        return [T(b["x"], [R], Ccols), T(b["g"], [R], 1), T(b["b"], [R], 1)]
    cases.append(Case("layer_norm_fwd_cols1024", 2 * S, mk_ln2, lambda b: ctx.fwd("layer_norm", ln2_xs(b), T(b["y"], [R], Ccols)), 4 * S))
    cases.append(Case("layer_norm_bwd_x_cols1024", 4 * S, mk_ln2,
                      lambda b: ctx.bwd("layer_norm", ln2_xs(b), T(b["y"], [R], Ccols), T(b["dy"], [R], Ccols), 0, T(b["dx"], [R], Ccols)), 4 * S))

    def mk_wn():
        return dict(w=torch.randn(R, Ccols, device=dev), g=torch.full((1,), 1.3, device=dev), y=torch.empty(R, Ccols, device=dev),
                    dy=torch.randn(R, Ccols, device=dev), dw=torch.zeros(R, Ccols, device=dev))
    cases.append(Case("weight_norm_fwd", 2 * S, mk_wn,
                      lambda b: ctx.fwd("weight_norm", [T(b["w"], [R, Ccols], 1), T(b["g"], [1], 1)], T(b["y"], [R, Ccols], 1)), 4 * S))
    cases.append(Case("weight_norm_bwd_w", 4 * S, mk_wn,
                      lambda b: ctx.bwd("weight_norm", [T(b["w"], [R, Ccols], 1), T(b["g"], [1], 1)], T(b["y"], [R, Ccols], 1),
                                        T(b["dy"], [R, Ccols], 1), 0, T(b["dw"], [R, Ccols], 1)), 4 * S))

    # config 2: vocab 50,000, embed 512, 4,096 Zipf(1.1) ids
    V, E, N = (50000, 512, 4096) if not small else (50000, 512, 4096)
    rng = np.random.Generator(np.random.PCG64(7))
    ranks = np.arange(1, V + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** -1.1); cdf /= cdf[-1]
    ids = np.minimum(np.searchsorted(cdf, rng.random(N)), V - 1).astype(np.uint32)
    ids_p = ids.ctypes.data_as(C.POINTER(C.c_uint32))
    uniq = len(np.unique(ids))
    def mk_lookup():
        return dict(table=torch.randn(V, E, device=dev), out=torch.empty(N, E, device=dev), aux=torch.zeros(N, dtype=torch.int32, device=dev),
                    ids_dev=torch.from_numpy(ids.view(np.int32)).to(dev), g=torch.randn(N, E, device=dev), grads=torch.zeros(V, E, device=dev),
                    keep=ids)
    cases.append(Case("lookup_gather_N4096_E512", 2 * N * E * 4 + 4 * N, mk_lookup,
                      lambda b: ctx.fwd("lookup", [], T(b["out"], [E], N), capi.LookupAttrs(b["table"].data_ptr(), V, None, N, 1.0),
                                        b["ids_dev"].data_ptr()), 2 * V * E * 4))
    cases.append(Case("lookup_scatter_add_N4096_E512", N * E * 4 + 2 * uniq * E * 4 + 16 * N, mk_lookup,
                      lambda b: ctx.lookup_accumulate_grads([], b["ids_dev"].data_ptr(), b["g"].data_ptr(), b["grads"].data_ptr(), E, V, n=N),
                      2 * V * E * 4))

    # config 2 logits: Dim({50000}, 4096) = 819 MB (already > L2, one buffer set is enough)
    Vr, Bc = (50000, 4096) if not small else (50000, 1024)
    tgt = np.minimum(np.searchsorted(cdf, rng.random(Bc)), V - 1).astype(np.uint32)
    tgt_p = tgt.ctypes.data_as(C.POINTER(C.c_uint32))
    SL = 4 * Vr * Bc
    def mk_pnls():
        aux = torch.zeros(3 * Bc, device=dev)
        aux[2 * Bc:].view(torch.int32).copy_(torch.from_numpy(tgt.view(np.int32)))   # ids already in aux_mem on the device
        return dict(x=torch.randn(Bc, Vr, device=dev), loss=torch.empty(Bc, device=dev), aux=aux,
                    dE=torch.ones(Bc, device=dev), dx=torch.zeros(Bc, Vr, device=dev), z=torch.empty(Bc, device=dev), keep=tgt)
    pa = capi.PickAttrs(None, Bc)
    cases.append(Case("pickneglogsoftmax_fwd_50000x%d" % Bc, SL, mk_pnls,
                      lambda b: ctx.fwd("pickneglogsoftmax", [T(b["x"], [Vr], Bc)], T(b["loss"], [1], Bc), pa, b["aux"].data_ptr()), 2 * SL))
    cases.append(Case("pickneglogsoftmax_bwd_50000x%d" % Bc, 3 * SL, mk_pnls,
                      lambda b: ctx.bwd("pickneglogsoftmax", [T(b["x"], [Vr], Bc)], T(b["loss"], [1], Bc), T(b["dE"], [1], Bc), 0,
                                        T(b["dx"], [Vr], Bc), pa, b["aux"].data_ptr()), 2 * SL))
    cases.append(Case("logsumexp_dim0_50000x%d" % Bc, SL, mk_pnls,
                      lambda b: ctx.fwd("logsumexp_dim", [T(b["x"], [Vr], Bc)], T(b["z"], [1], Bc), capi.DimAttrs(0)), 2 * SL))

    # LSTM C / H nodes at config 4 size (H = 1024, B = 512)
    Hh, Bb = 1024, 512
    def mk_ch():
        return dict(c=torch.randn(Bb, Hh, device=dev), gates=torch.rand(Bb, 4 * Hh, device=dev), out=torch.empty(Bb, Hh, device=dev))
    cases.append(Case("vanilla_lstm_c_fwd_H1024_B512", 20 * Hh * Bb, mk_ch,
                      lambda b: ctx.fwd("vanilla_lstm_c", [T(b["c"], [Hh], Bb), T(b["gates"], [4 * Hh], Bb)], T(b["out"], [Hh], Bb)), 24 * Hh * Bb))
    cases.append(Case("vanilla_lstm_h_fwd_H1024_B512", 12 * Hh * Bb, mk_ch,
                      lambda b: ctx.fwd("vanilla_lstm_h", [T(b["c"], [Hh], Bb), T(b["gates"], [4 * Hh], Bb)], T(b["out"], [Hh], Bb)), 24 * Hh * Bb))
    # tensor-bound: the gate GEMM (layer-2 shape of config 4: 4H = 4096, I = H = 1024, B = 512) and a weight-gradient product
    Ig = Hh
    def mk_gates():
        sc = (6.0 / (4 * Hh + Ig)) ** 0.5
        return dict(x=torch.randn(Bb, Ig, device=dev), h=torch.randn(Bb, Hh, device=dev) * 0.5,
                    Wx=(torch.rand(Ig, 4 * Hh, device=dev) * 2 - 1) * sc, Wh=(torch.rand(Hh, 4 * Hh, device=dev) * 2 - 1) * sc,
                    b=torch.zeros(4 * Hh, device=dev), mx=(torch.rand(Bb, Ig, device=dev) < 0.8).float() / 0.8,
                    mh=(torch.rand(Bb, Hh, device=dev) < 0.8).float() / 0.8, out=torch.empty(Bb, 4 * Hh, device=dev),
                    dW=torch.zeros(Ig, 4 * Hh, device=dev), dg=torch.randn(Bb, 4 * Hh, device=dev))
    gat = capi.LstmGatesAttrs(1, 0.0, 1.0)
    def gates_fwd(b):
        xs = [T(b["x"], [Ig], Bb), T(b["h"], [Hh], Bb), T(b["Wx"], [4 * Hh, Ig], 1), T(b["Wh"], [4 * Hh, Hh], 1), T(b["b"], [4 * Hh], 1),
              T(b["mx"], [Ig], Bb), T(b["mh"], [Hh], Bb)]
        ctx.fwd("vanilla_lstm_gates", xs, T(b["out"], [4 * Hh], Bb), gat)
    fl_g = 2.0 * 4 * Hh * (Ig + Hh) * Bb
    cases.append(Case("lstm_gates_fwd_gemm_4096x512x2048", 0, mk_gates, gates_fwd, 10 ** 9))
    cases[-1].flops = fl_g
    def dw_gemm(b):   # dWx += dgate * x^T : M = 4H, N = I, K = B
        ctx.gemm(0, 1, 4 * Hh, Ig, Bb, b["dg"].data_ptr(), 4 * Hh, b["x"].data_ptr(), Ig, b["dW"].data_ptr(), 4 * Hh, 1)
    cases.append(Case("gemm_dW_4096x1024x512_accumulate", 0, mk_gates, dw_gemm, 10 ** 9))
    cases[-1].flops = 2.0 * 4 * Hh * Ig * Bb
    # the same step through the fused entry point: one kernel forms gates, c and h (c / h update in the GEMM epilogue)
    def mk_fused():
        b = mk_gates()
        b.update(c_prev=torch.randn(Bb, Hh, device=dev) * 0.5, c=torch.empty(Bb, Hh, device=dev), hh=torch.empty(Bb, Hh, device=dev))
        return b
    def fused_fwd(b):
        ctx.lstm_fwd_fused(T(b["x"], [Ig], Bb), T(b["h"], [Hh], Bb), T(b["c_prev"], [Hh], Bb), T(b["Wx"], [4 * Hh, Ig], 1),
                           T(b["Wh"], [4 * Hh, Hh], 1), T(b["b"], [4 * Hh], 1), T(b["mx"], [Ig], Bb), T(b["mh"], [Hh], Bb), gat,
                           T(b["out"], [4 * Hh], Bb), T(b["c"], [Hh], Bb), T(b["hh"], [Hh], Bb))
    cases.append(Case("lstm_fwd_fused_gates_c_h_4096x512x2048", 0, mk_fused, fused_fwd, 10 ** 9))
    cases[-1].flops = fl_g
    # a whole LSTM layer over T = 35 time steps in one call (layer 2 of config 4: I = H = 1024) at the per-GPU batches of 1 and
    # 8 GPUs: one sequence-persistent kernel, or (--per-step) the 35 per-step products it replaces
    Tt = 35 if not small else 4
    for Bq in (512, 64):
        def mk_seq(Bq=Bq):
            sc = (6.0 / (4 * Hh + Ig)) ** 0.5
            d = dict(x=torch.randn(Tt * Bq, Ig, device=dev), z=torch.zeros(Bq, Hh, device=dev),
                     Wx=(torch.rand(Ig, 4 * Hh, device=dev) * 2 - 1) * sc, Wh=(torch.rand(Hh, 4 * Hh, device=dev) * 2 - 1) * sc,
                     b=torch.zeros(4 * Hh, device=dev), mx=(torch.rand(Bq, Ig, device=dev) < 0.8).float() / 0.8,
                     mh=(torch.rand(Bq, Hh, device=dev) < 0.8).float() / 0.8, gates=torch.empty(Tt * Bq, 4 * Hh, device=dev),
                     c=torch.empty(Tt * Bq, Hh, device=dev), h=torch.empty(Tt * Bq, Hh, device=dev))
            d["w"] = ctx.wgrad_create(4 * Hh, Ig, Hh, Tt * Bq)
            return d
        def seq_fwd(b, Bq=Bq):
            ctx.lstm_seq_fwd(T(b["x"], [Ig], Tt * Bq), T(b["z"], [Hh], Bq), T(b["z"], [Hh], Bq), T(b["Wx"], [4 * Hh, Ig], 1),
                             T(b["Wh"], [4 * Hh, Hh], 1), T(b["b"], [4 * Hh], 1), T(b["mx"], [Ig], Bq), T(b["mh"], [Hh], Bq), gat,
                             T(b["gates"], [4 * Hh], Tt * Bq), T(b["c"], [Hh], Tt * Bq), T(b["h"], [Hh], Tt * Bq), b["w"], Tt)
        cases.append(Case("lstm_seq_fwd_I1024_H1024_B%d_T%d" % (Bq, Tt), 0, mk_seq, seq_fwd, 10 ** 9))
        cases[-1].flops = 2.0 * 4 * Hh * (Ig + Hh) * Bq * Tt

    # the backward pass of the same layer over all time steps in one call: one sequence-persistent kernel for steps T-1 .. 1
    # (cell pass + [Wx; Wh]^T dgates product per step) + the per-step form of step 0, or (--per-step) T per-step calls
    for Bq in (512, 64):
        def mk_seqb(Bq=Bq):
            sc = (6.0 / (4 * Hh + Ig)) ** 0.5
            d = dict(x=torch.randn(Tt * Bq, Ig, device=dev), z=torch.zeros(Bq, Hh, device=dev),
                     Wx=(torch.rand(Ig, 4 * Hh, device=dev) * 2 - 1) * sc, Wh=(torch.rand(Hh, 4 * Hh, device=dev) * 2 - 1) * sc,
                     mx=(torch.rand(Bq, Ig, device=dev) < 0.8).float() / 0.8, mh=(torch.rand(Bq, Hh, device=dev) < 0.8).float() / 0.8,
                     gates=torch.rand(Tt * Bq, 4 * Hh, device=dev), c=torch.randn(Tt * Bq, Hh, device=dev) * 0.5,
                     h=torch.randn(Tt * Bq, Hh, device=dev) * 0.5, dh=torch.randn(Tt * Bq, Hh, device=dev) * 0.01,
                     dc=torch.zeros(Tt * Bq, Hh, device=dev), dx=torch.zeros(Tt * Bq, Ig, device=dev), db=torch.zeros(4 * Hh, device=dev))
            d["w"] = ctx.wgrad_create(4 * Hh, Ig, Hh, Tt * Bq)
            return d
        def seq_bwd(b, Bq=Bq):
            ctx.lstm_seq_bwd(T(b["x"], [Ig], Tt * Bq), T(b["z"], [Hh], Bq), T(b["z"], [Hh], Bq), T(b["Wx"], [4 * Hh, Ig], 1),
                             T(b["Wh"], [4 * Hh, Hh], 1), T(b["mx"], [Ig], Bq), T(b["mh"], [Hh], Bq), gat, T(b["gates"], [4 * Hh], Tt * Bq),
                             T(b["c"], [Hh], Tt * Bq), T(b["h"], [Hh], Tt * Bq), T(b["dh"], [Hh], Tt * Bq), T(b["dc"], [Hh], Tt * Bq),
                             T(b["dx"], [Ig], Tt * Bq), None, None, T(b["db"], [4 * Hh], 1), b["w"], Tt)
        cases.append(Case("lstm_seq_bwd_I1024_H1024_B%d_T%d" % (Bq, Tt), 0, mk_seqb, seq_bwd, 10 ** 9))
        cases[-1].flops = 2.0 * 4 * Hh * (Ig + Hh) * Bq * Tt

    # one backward time step of an LSTM layer (layer 2 of config 4) through the fused entry point: the tiled cell pass
    # (H, C and gate derivatives, operand planes of the gate gradient) + the product for dx and dh_tm1
    for Bq in (512, 64):
        def mk_bwd(Bq=Bq):
            d = mk_gates()
            d.update(x=torch.randn(Bq, Ig, device=dev), h=torch.randn(Bq, Hh, device=dev) * 0.5, c_prev=torch.randn(Bq, Hh, device=dev) * 0.5,
                     c=torch.randn(Bq, Hh, device=dev) * 0.5, gates=torch.rand(Bq, 4 * Hh, device=dev), dh=torch.randn(Bq, Hh, device=dev),
                     dc=torch.randn(Bq, Hh, device=dev), dx=torch.zeros(Bq, Ig, device=dev), dhp=torch.zeros(Bq, Hh, device=dev),
                     dcp=torch.zeros(Bq, Hh, device=dev), db=torch.zeros(4 * Hh, device=dev),
                     mx=(torch.rand(Bq, Ig, device=dev) < 0.8).float() / 0.8, mh=(torch.rand(Bq, Hh, device=dev) < 0.8).float() / 0.8)
            d["w"] = ctx.wgrad_create(4 * Hh, Ig, Hh, Bq)
            return d
        def bwd_step(b, Bq=Bq):
            ctx.lstm_bwd_fused_at(T(b["x"], [Ig], Bq), T(b["h"], [Hh], Bq), T(b["c_prev"], [Hh], Bq), T(b["Wx"], [4 * Hh, Ig], 1),
                                  T(b["Wh"], [4 * Hh, Hh], 1), T(b["mx"], [Ig], Bq), T(b["mh"], [Hh], Bq), T(b["gates"], [4 * Hh], Bq),
                                  T(b["c"], [Hh], Bq), T(b["dh"], [Hh], Bq), T(b["dc"], [Hh], Bq), T(b["dx"], [Ig], Bq), T(b["dhp"], [Hh], Bq),
                                  T(b["dcp"], [Hh], Bq), None, None, T(b["db"], [4 * Hh], 1), gat, b["w"], 0)
        cases.append(Case("lstm_bwd_fused_step_I1024_H1024_B%d" % Bq, 0, mk_bwd, bwd_step, 10 ** 9))
        cases[-1].flops = 2.0 * 4 * Hh * (Ig + Hh) * Bq

    # output layer of config 4 over all time steps: r = bias + R h, M = V = 10000, N = T*B = 17920, K = H = 1024
    Vv, TB = 10000, 17920
    def mk_aff():
        return dict(R=torch.randn(Hh, Vv, device=dev) * 0.02, h=torch.randn(TB, Hh, device=dev) * 0.5, b=torch.zeros(Vv, device=dev),
                    r=torch.empty(TB, Vv, device=dev))
    def aff_fwd(b):
        ctx.fwd("affine_transform", [T(b["b"], [Vv], 1), T(b["R"], [Vv, Hh], 1), T(b["h"], [Hh], TB)], T(b["r"], [Vv], TB))
    cases.append(Case("affine_transform_fwd_10000x17920x1024", 0, mk_aff, aff_fwd, 10 ** 9))
    cases[-1].flops = 2.0 * Vv * TB * Hh

    # backward of the same output layer in one call: PickNegLogSoftmax gradient written as the operands of dR and dh
    # (k_softmax_bwd_split: 4 V n bytes in, 8 V n bytes out), then the two products
    nB = TB if not small else 4096
    def mk_outbwd():
        tgt = rng.integers(0, Vv, size=nB).astype(np.uint32)
        aux = torch.zeros(3 * nB, device=dev)
        aux[:nB] = 9.3                                                     # logsumexp of each column (any plausible value)
        aux[2 * nB:].view(torch.int32).copy_(torch.from_numpy(tgt.view(np.int32)))
        return dict(x=torch.randn(nB, Vv, device=dev), h=torch.randn(nB, Hh, device=dev) * 0.5, R=torch.randn(Hh, Vv, device=dev) * 0.02,
                    dE=torch.ones(nB, device=dev), aux=aux, dR=torch.zeros(Hh, Vv, device=dev), db=torch.zeros(Vv, device=dev),
                    dh=torch.zeros(nB, Hh, device=dev))
    def outbwd(b):
        ctx.softmax_output_bwd_fused(T(b["x"], [Vv], nB), T(b["h"], [Hh], nB), T(b["R"], [Vv, Hh], 1), T(b["dE"], [1], nB), b["aux"].data_ptr(),
                                     T(b["dR"], [Vv, Hh], 1), T(b["db"], [Vv], 1), T(b["dh"], [Hh], nB))
    cases.append(Case("softmax_output_bwd_fused_10000x%dx1024" % nB, 0, mk_outbwd, outbwd, 10 ** 9))
    cases[-1].flops = 4.0 * Vv * nB * Hh

    # autobatch movers at the tagger's size (config 5): 2048 slices of 256 floats (one hidden state per token) gathered
    # from ragged positions into a token-major matrix and scattered back with +=; and the same kernels on 65536 slices of
    # 1024 floats, where the transfer (268 MB each way) is long enough to show what they sustain
    for (nsl, ln, tag) in ([(2048, 256, "tagger_2048x256"), (65536, 1024, "65536x1024")] if not small else [(2048, 256, "tagger_2048x256")]):
        def mk_ragged(nsl=nsl, ln=ln):
            pool = torch.randn(2 * nsl, ln, device=dev)                 # slices sit at every other row (ragged source positions)
            dense = torch.zeros(nsl, ln, device=dev)
            perm = torch.randperm(nsl, device=dev)
            src = (pool.data_ptr() + (2 * perm.to(torch.int64)) * (4 * ln))
            trg = (dense.data_ptr() + torch.arange(nsl, device=dev, dtype=torch.int64) * (4 * ln))
            lens = torch.full((nsl,), ln, dtype=torch.int64, device=dev)
            return dict(pool=pool, dense=dense, src=src, trg=trg, lens=lens)
        nb = 4 * nsl * ln
        cases.append(Case("parallel_memcpy_" + tag, 2 * nb + 24 * nsl, mk_ragged,
                          lambda b, nsl=nsl, ln=ln: ctx.parallel_memcpy(nsl, ln, b["src"].data_ptr(), b["trg"].data_ptr(), b["lens"].data_ptr()), 3 * nb))
        # accumulate the other way round: dense rows added into the ragged positions (distinct targets, the autobatch case)
        cases.append(Case("parallel_accumulate_" + tag, 3 * nb + 24 * nsl, mk_ragged,
                          lambda b, nsl=nsl, ln=ln: ctx.parallel_accumulate(nsl, ln, b["trg"].data_ptr(), b["src"].data_ptr(), b["lens"].data_ptr()), 3 * nb))

    # trainer update rules over the config-4 parameter buffer (30.06 M floats)
    NP = 30_060_000 if not small else 1 << 20
    def mk_tr():
        return dict(p=torch.randn(NP, device=dev), g=torch.randn(NP, device=dev) * 0.01, m=torch.zeros(NP, device=dev),
                    v=torch.zeros(NP, device=dev), ss=torch.ones(1, device=dev))
    hyp = capi.TrainerHyper(0.001, 5.0, 1.0, 0.9, 1e-8, 0.95, 0.9, 0.999, 3)
    cases.append(Case("trainer_sgd_clip_zero_30M", 16 * NP, mk_tr,
                      lambda b: ctx.trainer_update("sgd", b["p"].data_ptr(), b["g"].data_ptr(), [], NP, hyp, b["ss"].data_ptr(), True), 16 * NP))
    cases.append(Case("trainer_adam_clip_zero_30M", 32 * NP, mk_tr,
                      lambda b: ctx.trainer_update("adam", b["p"].data_ptr(), b["g"].data_ptr(), [b["m"].data_ptr(), b["v"].data_ptr()], NP, hyp,
                                                   b["ss"].data_ptr(), True), 32 * NP))
    cases.append(Case("squared_norm_30M", 4 * NP, mk_tr,
                      lambda b: ctx.squared_norm(b["g"].data_ptr(), NP, b["ss"].data_ptr()), 4 * NP))
    # glue nodes at LSTM-builder sizes: concatenate(h_fwd, h_bwd) and pick_range of the gates, 4096 x 4096
    Rg, Bg = (4096, 4096) if not small else (256, 256)
    def mk_glue():
        return dict(a=torch.randn(Bg, Rg, device=dev), b=torch.randn(Bg, Rg, device=dev), cat=torch.empty(Bg, 2 * Rg, device=dev),
                    part=torch.empty(Bg, Rg // 4, device=dev), s=torch.empty(1, Rg, device=dev), msk=torch.empty(Bg, Rg, device=dev))
    SG = 4 * Rg * Bg
    cases.append(Case("concatenate_2x4096_B4096", 4 * SG, mk_glue,
                      lambda b: ctx.fwd("concatenate", [T(b["a"], [Rg], Bg), T(b["b"], [Rg], Bg)], T(b["cat"], [2 * Rg], Bg), capi.DimAttrs(0)), 4 * SG))
    cases.append(Case("pick_range_quarter_of_4096_B4096", SG // 2, mk_glue,
                      lambda b: ctx.fwd("pick_range", [T(b["a"], [Rg], Bg)], T(b["part"], [Rg // 4], Bg), capi.PickRangeAttrs(Rg // 4, Rg // 2, 0)), SG))
    cases.append(Case("sum_batches_4096_B4096", SG, mk_glue,
                      lambda b: ctx.fwd("sum_dim", [T(b["a"], [Rg], Bg)], T(b["s"], [Rg], 1),
                                        capi.SumDimAttrs((C.c_uint * 2)(0, 0), 0, 1)), SG))
    cases.append(Case("random_bernoulli_4096_B4096", SG, mk_glue,
                      lambda b: ctx.fwd("random_bernoulli", [], T(b["msk"], [Rg], Bg), capi.BernoulliAttrs(0.8, 1.25, 7, 0)), SG))
    return cases


def run(only=None, iters=20, small=False, out=None, graph_mode=True, quiet=False, device=0, skip_tensor_bound=False, per_step=False):
    import torch
    stream = torch.cuda.Stream()
    ctx = capi.Context(device, stream.cuda_stream)
    if per_step:
        ctx.sequence_kernels(0 if per_step is True else per_step)
    ctx.param_cache(True)   # as in training: weight matrices are split once (during warm-up), not in every timed call
    peak, src = peaks()
    results = []
    for case in build_cases(torch, ctx, small):
        if only and only not in case.name:
            continue
        if skip_tensor_bound and getattr(case, "flops", None):
            continue
        nsets = max(2, min(24, int(np.ceil(2.0 * L2_BYTES / max(case.footprint, 1)))))
        if small or getattr(case, "flops", None):
            nsets = 2
        with torch.cuda.stream(stream):
            sets = [case.make() for _ in range(nsets)]
            for k in range(3):
                case.call(sets[k % nsets])
            stream.synchronize()
            l0 = ctx.launches()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            graph = None
            if graph_mode:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for k in range(iters):
                        case.call(sets[k % nsets])
                launches = ctx.launches() - l0
                graph.replay()
                stream.synchronize()
                e0.record(stream)
                graph.replay()
                e1.record(stream)
            else:   # eager calls (what a profiler capture of single launches wants)
                e0.record(stream)
                for k in range(iters):
                    case.call(sets[k % nsets])
                e1.record(stream)
                launches = ctx.launches() - l0
            stream.synchronize()
        ms = e0.elapsed_time(e1) / iters
        gbs = case.nbytes / (ms * 1e-3) / 1e9
        rec = {"kernel": case.name, "algorithmic_bytes": int(case.nbytes), "ms": ms, "GBps": gbs,
               "frac_of_%s_copy_peak" % src: gbs / peak, "frac_of_8000": gbs / 8000.0,
               "launches_per_call": launches / iters, "buffer_sets": nsets}
        if getattr(case, "flops", None):
            rec["useful_TFLOPs"] = case.flops / (ms * 1e-3) / 1e12   # whole call, operand packing included
        results.append(rec)
        if not quiet:
            print(json.dumps(rec), flush=True)
        del sets, graph
        torch.cuda.empty_cache()
    assert ctx.device_errors() == 0
    ctx.close()
    if out:
        with open(out, "w") as f:
            json.dump(results, f, indent=1)
    return results


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--out", default=None)
    ap.add_argument("--eager", action="store_true", help="no CUDA graph: plain launches (for profiler captures)")
    ap.add_argument("--per-step", action="store_true", help="sequence entry points issue one call per time step (dyb200_ctx_sequence_kernels off)")
    ap.add_argument("--plain-launch", action="store_true", help="sequence kernels without the cooperative-launch attribute (for ncu)")
    a = ap.parse_args()
    run(a.only, a.iters, a.small, a.out, graph_mode=not a.eager, per_step=(True if a.per_step else (2 if a.plain_launch else False)))
