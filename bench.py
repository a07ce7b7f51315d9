#!/usr/bin/env python
"""Benchmark of the hot path: training steps of the 2-layer LSTM language model built from the fused
nodes (embedding gather, vanilla_lstm_gates/_c/_h with dropout masks, output projection,
PickNegLogSoftmax, their backward, deterministic embedding scatter-add, gradient all-reduce, clipped SGD).

  python bench.py --gpus N --steps K --warmup W            # this implementation, one rank per GPU
  python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU algorithm on the host cores

Prints ONE JSON line (rank 0).  `value` = tokens/s with the token ids already resident in HBM;
`e2e` = tokens/s through the same public step call with the ids copied from pinned host memory and the
loss read back every step.  Data are synthetic: Zipf(1.1) token ids, Glorot-uniform weights.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The configuration the metric is quoted on: 2-layer LSTM-LM, vocab 10k, embed 512, hidden 1024,
# dropout 0.2, sequence length 35, global batch 512 sharded over the GPUs.
WORKLOAD = dict(V=10000, E=512, H=1024, L=2, T=35)
GLOBAL_BATCH = 512
DROPOUT = 0.2
METRIC = "LSTM-LM training tokens/sec (2-layer LSTM, V=10k E=512 H=1024 T=35, global batch 512, fwd+bwd+allreduce+SGD)"


def config_dict(world, graph=True):
    """The `config` object of the JSON line: the same for this implementation and for the reference arm."""
    V, E, H, L, T = (WORKLOAD[k] for k in "VEHLT")
    return {"workload": "lstm_lm_2x1024_v10k_t35", "global_batch": GLOBAL_BATCH, "per_gpu_batch": GLOBAL_BATCH // world,
            "seq_len": T, "vocab": V, "embed": E, "hidden": H, "layers": L, "dropout": DROPOUT,
            "parallelism": "dp%d" % world, "l2": "per-step working set (~2.5 GB of activations) exceeds the 126 MB L2",
            "cuda_graph": bool(graph)}


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.lower().startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown CPU"


FLOPS_PER_TOKEN = None   # filled below (useful FLOPs of fwd + bwd per token of the workload)


def flops_per_step(B):
    V, E, H, L, T = (WORKLOAD[k] for k in "VEHLT")
    fwd = 0
    for l in range(L):
        fwd += 2 * 4 * H * ((E if l == 0 else H) + H) * B
    fwd += 2 * V * H * B
    return 3 * fwd * T   # backward = 2x forward


FLOPS_PER_TOKEN = flops_per_step(1) / WORKLOAD["T"]


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d.get("hbm_gbs"), "bf16_tflops": d.get("bf16_tflops"),
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def measure_tf32_peak(torch):
    """cuBLAS TF32 dense GEMM, 8192^3, run back to back for about a second (the 3xTF32 roofline
    denominator is this figure / 3; the peaks file only carries bf16)."""
    n = 8192
    a = torch.randn(n, n, device="cuda")
    b = torch.randn(n, n, device="cuda")
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        for _ in range(3):
            torch.matmul(a, b)
        torch.cuda.synchronize()
        reps = 40
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch.matmul(a, b)
        e1.record()
        torch.cuda.synchronize()
        return 2.0 * n ** 3 * reps / (e0.elapsed_time(e1) * 1e-3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
        del a, b


def cpu_baseline_sample(threads, seqs_per_thread, steps=1):
    """The CPU oracle (a port of the reference's single-threaded Eigen path) on a bounded sample of
    the same workload: `threads` independent shards of `seqs_per_thread` sequences, full model size."""
    import oracle
    from dynet_b200 import lm
    oracle.build()
    V, E, H, L, T = (WORKLOAD[k] for k in "VEHLT")
    params = lm.init_params(V, E, H, L, seed=1)
    dims = dict(WORKLOAD, B=seqs_per_thread)
    work = []
    for k in range(threads):
        tokens, masks = lm.synthetic_batch(dims, seed=100 + k, dropout=DROPOUT)
        grads = [np.zeros_like(p) for p in params]
        work.append((tokens, masks, grads))

    def run(k):
        tokens, masks, grads = work[k]
        oracle.lstm_lm_fwdbwd((V, E, H, L, T, seqs_per_thread), params, grads, tokens, masks[0], masks[1])

    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        ths = [threading.Thread(target=run, args=(k,)) for k in range(threads)]
        [t.start() for t in ths]
        [t.join() for t in ths]
        # gradient sum over shards + clipped SGD on one thread, as rank 0 does in dynet/mp.h
        total = [sum(w[2][i] for w in work) for i in range(len(params))]
        oracle.sgd_update([p.copy() for p in params], total, 0.1, 5.0)
        times.append(time.perf_counter() - t0)
    tokens_per_step = threads * seqs_per_thread * T
    sec = float(np.mean(times))
    return tokens_per_step / sec, sec, tokens_per_step


def cpu_baseline_record(single_seqs, steps, multi=True):
    """The reference's CPU path is single-threaded (Eigen DefaultDevice, no OpenMP in its build, dynet/devices.cc:150), so
    the baseline is ONE host thread running the oracle port on a bounded sample of the step (single_seqs of the 512
    sequences, all 35 time steps, full model size); tokens/s scales linearly in the sequences.  A second, labelled figure
    uses all host threads as independent shards (the reference's dynet/mp.h process-level data parallelism)."""
    ncpu = os.cpu_count() or 1
    tps, sec, toks = cpu_baseline_sample(1, single_seqs, steps=steps)
    rec = {"value": tps, "unit": "tokens/s", "cores": 1, "kind": "port", "cpu_model": cpu_model(), "nproc": ncpu,
           "sample": "1 host thread x %d sequences x T=35 per step (of the 512-sequence batch; tokens/s is linear in the sequences), "
                     "fwd+bwd+update at full model size, %.1f s per step" % (single_seqs, sec),
           "gflops_per_thread": tps * FLOPS_PER_TOKEN / 1e9,
           "note": "oracle port of the reference's CPU algorithm (the reference itself needs Eigen b2e267dc99d4, absent here); its "
                   "matrix products are plain blocked loops without FMA contraction, several times slower than Eigen's GEBP kernel"}
    if multi and ncpu > 1:
        threads = min(ncpu, 32)
        mtps, msec, _ = cpu_baseline_sample(threads, 16, steps=1)
        rec["multi_thread"] = {"value": mtps, "unit": "tokens/s", "cores": threads,
                               "sample": "%d host threads x 16 sequences each, one step, %.1f s" % (threads, msec)}
    return rec


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    seqs = 8    # per step: ~2 s of one core, so that K steps stay within a few minutes
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_baseline_sample(1, 1, steps=1)           # builds the oracle, touches memory
    rec = cpu_baseline_record(seqs, max(1, args.steps))
    tps = rec["value"]
    world = max(1, args.gpus)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": GLOBAL_BATCH * WORKLOAD["T"] / tps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_dict(world),
        "ms_per_step_note": "the full 512-sequence step extrapolated linearly from the sample",
        "cpu_baseline": rec,
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from dynet_b200 import dp, lm

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback for this arm")
    rank, world = dp.init_process_group("nccl") if int(os.environ.get("WORLD_SIZE", "1")) > 1 else (0, 1)
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world != args.gpus and world > 1:
        raise SystemExit("--gpus %d does not match WORLD_SIZE %d" % (args.gpus, world))
    if GLOBAL_BATCH % world:
        raise SystemExit("global batch %d is not divisible by %d ranks" % (GLOBAL_BATCH, world))
    B = GLOBAL_BATCH // world
    dims = dict(WORKLOAD, B=B)
    V, E, H, L, T = (WORKLOAD[k] for k in "VEHLT")
    stream = torch.cuda.Stream()          # a capturable (non-legacy) stream for the whole step
    torch.cuda.set_stream(stream)
    model = lm.LstmLm(device=local_rank, seed=1, lr=0.1, clip=5.0, dropout=True, stream=stream.cuda_stream, **dims)
    if args.plain_launch:
        model.ctx.sequence_kernels(2)

    # synthetic corpus: a few global batches of Zipf(1.1) ids; this rank keeps its columns
    n_batches = 4
    host_tokens, dev_tokens = [], []
    for k in range(n_batches):
        tokens, _ = lm.synthetic_batch(dict(WORKLOAD, B=GLOBAL_BATCH), seed=1000 + k, dropout=0.0)
        tok, _ = dp.shard_batch(tokens, None, rank, world)
        pinned = torch.from_numpy(tok.view(np.int32)).pin_memory()
        host_tokens.append(pinned)
        dev_tokens.append(pinned.cuda())
    keep = 1.0 - DROPOUT
    masks = model.mask_buffers()          # the driver's own buffers: fixed addresses, so the step can be a CUDA graph
    mask_step = [0]

    def draw_masks():
        # RandomBernoulli(keep) * 1/keep per layer, fixed over the sequence (dynet/lstm.cc:964-982), drawn every step
        model.draw_masks(keep, 1234 + rank, mask_step[0])
        mask_step[0] += 1

    def step(tokens):
        draw_masks()
        # forward + backward; with several ranks the gradient buckets are summed on a side stream as they become final
        model.launch_forward_backward_overlapped(tokens, masks)
        model.update()

    closed = [False]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(K, source, read_loss):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        losses = []
        for k in range(K):
            step(source[k % n_batches])
            if read_loss:
                losses.append(float(model.loss_dev.item()))   # D2H read of the step's result
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, losses

    # warm-up: eager steps (they size the scratch arena and the parameter cache), then the graph capture + replays
    l0 = model.ctx.launches()
    for k in range(max(3, args.warmup)):
        step(dev_tokens[k % n_batches])
    torch.cuda.synchronize()
    launches_per_step = (model.ctx.launches() - l0) // max(3, args.warmup)
    if not args.no_graph:
        model.set_graph(True)
        for k in range(2):
            step(dev_tokens[k % n_batches])
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, _ = timed(args.steps, dev_tokens, read_loss=False)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e, losses = timed(args.steps, host_tokens, read_loss=True)
    # roofline pass: the same K steps issued launch by launch, every GEMM bracketed by CUDA events
    model.set_graph(False)
    model.ctx.profile_begin(1 << 16)
    ms_prof, _ = timed(args.steps, dev_tokens, read_loss=False)
    per_launch = model.ctx.profile_launches()      # (M, N, K, epilogue mode, path, ms, flops) of every product
    prof = model.ctx.profile_end()
    errs = model.ctx.device_errors()
    launches = launches_per_step * args.steps
    # where a step's time goes (this rank, 5 more steps, CUDA events between the phases; not part of any headline number)
    if not args.no_graph:
        model.set_graph(True)
    phases = np.zeros(4)
    for k in range(5):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record(stream)
        draw_masks()
        ev[1].record(stream)
        model._after_last_phase = None
        model.launch_forward_backward_overlapped(dev_tokens[k % n_batches], masks)
        ev[2].record(stream)
        model.update()
        ev[3].record(stream)
        torch.cuda.synchronize()
        mid = model._after_last_phase           # recorded after the last backward phase, before the waits for the sums
        fb = ev[1].elapsed_time(mid) if mid is not None else ev[1].elapsed_time(ev[2])
        ar = mid.elapsed_time(ev[2]) if mid is not None else 0.0
        phases += [ev[0].elapsed_time(ev[1]), fb, ar, ev[2].elapsed_time(ev[3])]
    phases /= 5

    # replicas must hold bit-identical parameters after the same number of updates (deterministic kernels, the same reduced
    # gradient on every rank): max over ranks and elements of |theta_r - theta_0|
    replica_diff = 0.0
    if world > 1:
        ref = model.params.clone()
        dist.broadcast(ref, src=0)
        d = (model.params - ref).abs().max().reshape(1)
        dist.all_reduce(d, op=dist.ReduceOp.MAX)
        replica_diff = float(d.item())
        del ref

    tokens_per_step = GLOBAL_BATCH * T
    value = tokens_per_step * args.steps / (ms * 1e-3)
    e2e = tokens_per_step * args.steps / (ms_e2e * 1e-3)

    if rank == 0:
        peaks = measured_peaks()
        tf32 = measure_tf32_peak(torch)
        # dominant kernel = the GEMM behind the gates, the projection and their backward products
        which = "tensor" if prof["tensor"][1] >= prof["simt"][1] and prof["tensor"][1] > 0 else "simt"
        g_ms, g_n, g_fl = prof[which]
        achieved = g_fl / (g_ms * 1e-3) / 1e12 if g_ms > 0 else 0.0
        peak = tf32 / 3.0
        # per shape: launches per step, device time, useful TFLOP/s, and the bytes one launch has to move at least (the split
        # operand planes once, the result once; read-modify-write for the accumulating epilogues)
        shapes = {}
        for (M_, N_, K_, mode, path, t_ms, fl) in per_launch:
            rec = shapes.setdefault((M_, N_, K_, mode), [0, 0.0, 0.0])
            rec[0] += 1; rec[1] += t_ms; rec[2] += fl
        by_shape = []
        for (M_, N_, K_, mode), (cnt, t_ms, fl) in sorted(shapes.items(), key=lambda kv: -kv[1][1]):
            operand = 8.0 * K_ * (M_ + N_)
            result = 4.0 * M_ * N_ * (2 if mode in (1, 3) else 1) * (5.0 / 4.0 if mode == 5 else 1.0)   # LSTM epilogue: + c and h
            by_shape.append({"M": M_, "N": N_, "K": K_, "epilogue": int(mode), "launches_per_step": cnt / args.steps,
                             "us_per_launch": 1e3 * t_ms / cnt, "useful_tflops": fl / (t_ms * 1e-3) / 1e12 if t_ms > 0 else None,
                             "algorithmic_bytes_per_launch": operand + result})
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak if peak else None,
                    # DRAM bytes are a per-launch quantity of ONE shape, and this figure averages some ten shapes: the captured
                    # traffic is therefore given per shape below, next to the bytes that shape has to move at least
                    "traffic": None,
                    "traffic_captured_per_launch": {
                        "output_layer_M10000_N17920_K1024": 1.54e9,
                        "note": "dram__bytes_read.sum + dram__bytes_write.sum of one launch from the committed ncu summaries "
                                "(0.82 GB read + 0.72 GB written; algorithmic 0.83 GB); tensor-bound kernels, DRAM at 15-19 % of peak"},
                    "kernel": "gemm_3xtf32_tcgen05" if which == "tensor" else "gemm_fp32_cuda_core",
                    "launches": g_n, "share_of_step_time": g_ms / ms_prof if ms_prof else None,
                    "by_shape": by_shape[:12],
                    "measured_over": "the same %d steps issued launch by launch (%.2f ms/step) right after the timed region, "
                                     "which replays them as one CUDA graph" % (args.steps, ms_prof / args.steps),
                    "peak_source": "cuBLAS TF32 8192^3 measured in this run (%.0f TFLOP/s) / 3; bf16 peak of %s: %s TFLOP/s"
                                   % (tf32, peaks["source"], peaks["bf16_tflops"]),
                    "useful_tflop_per_step": flops_per_step(B) * world / 1e12}
        cpu_rec = None if args.no_cpu_baseline else cpu_baseline_record(32, 1)
        # the memory-bound kernels one by one (CUDA-graph timed, rotating buffers): the other half of the metric
        hbm = None
        if world == 1 and not args.no_hbm_kernels:
            import kernel_bench
            model.close()
            closed[0] = True
            res = kernel_bench.run(iters=10, quiet=True, device=local_rank, skip_tensor_bound=True)
            hbm = {"peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"],
                   "kernels": [{"name": r_["kernel"], "algorithmic_bytes": r_["algorithmic_bytes"], "us": 1e3 * r_["ms"],
                                "GBps": r_["GBps"], "frac": r_["GBps"] / peaks["hbm_gbs"]} for r_ in res]}
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": config_dict(world, not args.no_graph),
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": int((T + 1) * B * 4 * world),
                    "d2h_bytes_per_step": 4 * world, "ms_per_step": ms_e2e / args.steps, "last_loss": losses[-1] if losses else None},
            "gpu_launches": int(launches),
            "phases_ms": {"mask_draw": float(phases[0]), "fwd_bwd": float(phases[1]), "allreduce": float(phases[2]),
                          "clip_update": float(phases[3]),
                          "note": "rank 0, 5 extra steps after the timed regions; allreduce = what is left of the gradient sums after the "
                                  "last backward phase (the buckets of the output layer and of the upper LSTM layers are reduced on a side "
                                  "stream while the backward pass continues)"},
            "replica_max_abs_diff": replica_diff,
            "roofline": roofline,
            "cpu_baseline": cpu_rec,
            "hbm_kernels": hbm,
            "device_error_flags": errs,
        }
        print(json.dumps(line), flush=True)
    if not closed[0]:
        model.close()
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------------
# Second workload (--workload tagger): the autobatched BiLSTM tagger, 2 048 ragged sentences per step.
TAGGER = dict(V=20000, E=128, H=256, TH=32, NT=45, sentences=2048, lo=5, hi=100)
TAGGER_METRIC = ("BiLSTM tagger training tokens/sec (autobatched: 2048 sentences of 5..100 words per step, V=20k E=128 H=256/direction, "
                 "45 tags, fwd+bwd+allreduce+SGD)")


def tagger_config(world):
    c = dict(TAGGER)
    c.update({"workload": "bilstm_tagger_autobatch_2048x5-100", "parallelism": "dp%d" % world, "sentences_per_gpu": TAGGER["sentences"] // world,
              "l2": "per-step working set (~1.5 GB of step-major activations at one GPU) exceeds the 126 MB L2"})
    return c


def tagger_cpu_record(n_sent=96):
    """The oracle runs the tagger as the reference's CPU build does: sentence by sentence, batch size 1, one thread."""
    import oracle
    from dynet_b200 import tagger as tg
    oracle.build()
    V, E, H, TH, NT = (TAGGER[k] for k in ("V", "E", "H", "TH", "NT"))
    shapes = tg.param_shapes(V, E, H, TH, NT)
    flat = tg.init_params(V, E, H, TH, NT, seed=1)
    P = {n: a.reshape(cols, rows) if cols > 1 else a for n, a, (rows, cols) in zip(tg.NAMES, flat, shapes)}
    lens, words, tags = tg.synthetic_corpus(TAGGER["sentences"], V, NT, seed=2000, lo=TAGGER["lo"], hi=TAGGER["hi"])
    off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    idx = np.linspace(0, len(lens) - 1, n_sent).astype(int)           # long, medium and short sentences
    sents = [[int(v) for v in words[off[s]:off[s + 1]]] for s in idx]
    tgs = [[int(v) for v in tags[off[s]:off[s + 1]]] for s in idx]
    oracle.tagger_fwdbwd(P, sents[:1], tgs[:1])
    t0 = time.perf_counter()
    oracle.tagger_fwdbwd(P, sents, tgs)
    sec = time.perf_counter() - t0
    toks = sum(len(x) for x in sents)
    return {"value": toks / sec, "unit": "tokens/s", "cores": 1, "kind": "port", "cpu_model": cpu_model(), "nproc": os.cpu_count() or 1,
            "sample": "1 host thread, %d of the 2048 sentences (%d tokens), sentence by sentence at batch size 1 as the reference's CPU "
                      "build runs this example, %.1f s" % (n_sent, toks, sec),
            "note": "oracle port driven node by node from Python (the reference itself needs Eigen b2e267dc99d4, absent here)"}


def run_tagger_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    recs = [tagger_cpu_record() for _ in range(max(1, min(args.steps, 3)))]
    rec = recs[-1]
    tps = float(np.mean([r_["value"] for r_ in recs]))
    rec["value"] = tps
    world = max(1, args.gpus)
    ntok = float(np.mean([sum(range(TAGGER["lo"], TAGGER["hi"] + 1)) / (TAGGER["hi"] - TAGGER["lo"] + 1)])) * TAGGER["sentences"]
    print(json.dumps({"impl": "reference", "metric": TAGGER_METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": ntok / tps * 1e3, "higher_is_better": True, "scaling": "strong",
                      "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": tagger_config(world),
                      "ms_per_step_note": "the full 2048-sentence step extrapolated linearly from the sample", "cpu_baseline": rec,
                      "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)


def run_tagger_gpu(args):
    import torch
    import torch.distributed as dist
    from dynet_b200 import dp, tagger as tg
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback for this arm")
    rank, world = dp.init_process_group("nccl") if int(os.environ.get("WORLD_SIZE", "1")) > 1 else (0, 1)
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    V, E, H, TH, NT = (TAGGER[k] for k in ("V", "E", "H", "TH", "NT"))
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    # synthetic corpus: a few batches of 2048 sentences; this rank takes every world-th sentence of the length-sorted batch
    batches, total_tokens = [], []
    for k in range(3):
        lens, words, tags = tg.synthetic_corpus(TAGGER["sentences"], V, NT, seed=2000 + k, lo=TAGGER["lo"], hi=TAGGER["hi"])
        off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        mine = np.arange(rank, len(lens), world)
        batches.append((np.ascontiguousarray(lens[mine]), np.ascontiguousarray(np.concatenate([words[off[i]:off[i + 1]] for i in mine])),
                        np.ascontiguousarray(np.concatenate([tags[off[i]:off[i + 1]] for i in mine]))))
        total_tokens.append(int(lens.sum()))
    max_tok = max(int(b[0].sum()) for b in batches)
    model = tg.Tagger(V, E, H, TH, NT, max_sentences=len(batches[0][0]), max_tokens=max_tok, max_len=TAGGER["hi"], device=local_rank,
                      seed=1, lr=0.1, clip=5.0, stream=stream.cuda_stream)

    def step(k, read_loss=False):
        model.launch_forward_backward(*batches[k % len(batches)])
        model.allreduce_grads()
        model.update()
        return float(model.loss_dev.item()) if read_loss else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(K, read_loss):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        toks, last = 0, None
        for k in range(K):
            last = step(k, read_loss)
            toks += total_tokens[k % len(batches)]
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, toks, last

    l0 = model.launches()
    W = max(3, args.warmup)
    for k in range(W):
        step(k)
    torch.cuda.synchronize()
    launches_per_step = (model.launches() - l0) // W
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, toks, _ = timed(args.steps, read_loss=False)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e, toks_e2e, last_loss = timed(args.steps, read_loss=True)
    # the ragged movers, bracketed by CUDA events on the launch stream in a few extra passes
    model.time_movers(True)
    mv = np.zeros(4)
    host_ms = 0.0
    reps = 3
    for k in range(reps):
        model.launch_forward_backward(*batches[k % len(batches)])
        m4, hm = model.mover_ms()
        mv += m4
        host_ms += hm
        model.grads.zero_()
    model.time_movers(False)
    mv /= reps
    host_ms /= reps
    errs = model.device_errors()
    n_local = float(np.mean([int(b[0].sum()) for b in batches]))
    replica_diff = 0.0
    if world > 1:
        ref = model.params.clone()
        dist.broadcast(ref, src=0)
        d = (model.params - ref).abs().max().reshape(1)
        dist.all_reduce(d, op=dist.ReduceOp.MAX)
        replica_diff = float(d.item())
    if rank == 0:
        peaks = measured_peaks()
        slice_bytes = 4.0 * H * n_local
        algo = 2 * (2 * slice_bytes) + 2 * (3 * slice_bytes)         # two copies (read + write), two accumulates (2 reads + write)
        t_mv = float(mv.sum()) * 1e-3
        achieved = algo / t_mv / 1e9 if t_mv > 0 else 0.0
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                    "traffic": None, "kernel": "k_ragged_copy_warp; k_ragged_probe + k_ragged_accumulate_direct (the autobatch movers)",
                    "algorithmic_bytes": algo, "us": {"copy_fwd_dir": 1e3 * mv[0], "copy_bwd_dir": 1e3 * mv[1], "accumulate_fwd_dir": 1e3 * mv[2],
                                                      "accumulate_bwd_dir": 1e3 * mv[3]},
                    "note": "%d slices of %d floats per call (%.1f MB each way), timed with CUDA events around the four mover calls of a "
                            "step: a copy moves 2x and an accumulate 3x those bytes; the accumulate also runs the probe that checks its "
                            "targets for repeats (5 launches per call); the same kernels on 268 MB slices of 4 KB are in hbm_kernels of "
                            "the LSTM-LM line" % (int(n_local), H, slice_bytes / 1e6),
                    "peak_source": peaks["source"]}
        cpu_rec = None if args.no_cpu_baseline else tagger_cpu_record()
        tok_step = float(np.mean(total_tokens))
        line = {"metric": TAGGER_METRIC, "value": toks / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": W,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": tagger_config(world), "clocks": clocks,
                "e2e": {"value": toks_e2e / (ms_e2e * 1e-3), "unit": "tokens/s",
                        "h2d_bytes_per_step": int(world * n_local * (8 * 8 + 8 + 3 * 4)), "d2h_bytes_per_step": 4 * world,
                        "ms_per_step": ms_e2e / args.steps, "last_loss": last_loss,
                        "note": "every pass takes host arrays (lengths, word ids, tags): the pointer tables of the movers and the ids are "
                                "built on the host and copied to the device inside the timed region in both figures; e2e also reads the loss back"},
                "gpu_launches": int(launches_per_step * args.steps), "tokens_per_step": tok_step,
                "host_schedule_ms_per_step": host_ms, "replica_max_abs_diff": replica_diff,
                "roofline": roofline, "cpu_baseline": cpu_rec, "device_error_flags": errs}
        print(json.dumps(line), flush=True)
    model.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="dyb200", choices=["dyb200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-hbm-kernels", action="store_true", help="skip the per-kernel pass over the memory-bound kernels (N = 1 only)")
    ap.add_argument("--no-graph", action="store_true", help="issue every launch from the host instead of replaying a CUDA graph")
    ap.add_argument("--plain-launch", action="store_true",
                    help="launch the sequence-persistent kernels without the cooperative attribute (profilers that cannot replay such launches)")
    ap.add_argument("--workload", default="lm", choices=["lm", "tagger"],
                    help="lm: the 2-layer LSTM language model the headline metric is quoted on; tagger: the autobatched BiLSTM tagger")
    args = ap.parse_args()
    if args.workload == "tagger":
        run_tagger_reference(args) if args.impl == "reference" else run_tagger_gpu(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
