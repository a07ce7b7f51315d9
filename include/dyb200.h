/*
 * dyb200 — C ABI of the B200 (sm_100a) kernels that replace the Device_GPU
 * instantiations of DyNet's fused-layer nodes.
 *
 * Every node of the reference declares
 *     template<class MyDevice> void forward_dev_impl(const MyDevice&, const std::vector<const Tensor*>& xs, Tensor& fx) const;
 *     template<class MyDevice> void backward_dev_impl(const MyDevice&, const std::vector<const Tensor*>& xs,
 *                                                     const Tensor& fx, const Tensor& dEdf, unsigned i, Tensor& dEdxi) const;
 * (dynet/nodes-def-macros.h:44-62).  For each node in scope this header exports
 * one <node>_fwd and one <node>_bwd with exactly those arguments flattened to C:
 * tensors become dyb200_tensor views, the node's constructor arguments become a
 * small `attrs` struct, `aux_mem` is the node's aux_storage_size() block.
 *
 * Conventions (all identical to the reference):
 *  - tensors are column-major float32 on the device, the batch is the slowest
 *    axis (dynet/tensor-eigen.h:21-224); a dyb200_tensor does not own memory;
 *  - backward ACCUMULATES into dEdxi (dEdxi += ...), once per argument index i
 *    (dynet/exec.cc:262-271);
 *  - every call returns a status; nothing aborts, traps or throws.  The C++ shim
 *    maps DYB200_EINVAL to std::invalid_argument (DYNET_ARG_CHECK, dynet/except.h:41-46),
 *    DYB200_ERUNTIME to std::runtime_error (dynet/except.h:60-70), DYB200_ECUDA
 *    to dynet::cuda_exception (dynet/cuda.h:20-43) and DYB200_ENOMEM to
 *    dynet::out_of_memory (dynet/except.h:11-14);
 *  - kernels are launched on the context's stream (DyNet uses the legacy default
 *    stream, dynet/devices.cc:113-114) and the call returns without synchronising
 *    unless stated otherwise.
 */
#ifndef DYB200_H_
#define DYB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DYB200_OK 0
#define DYB200_EINVAL 1   /* bad shape / index / argument (reference: std::invalid_argument) */
#define DYB200_ERUNTIME 2 /* unsupported configuration (reference: std::runtime_error) */
#define DYB200_ECUDA 3    /* CUDA runtime failure, or a bounded device wait ran out */
#define DYB200_ENOMEM 4   /* scratch arena could not grow */

/* Mirror of dynet::Dim + the data pointer of dynet::Tensor (dynet/dim.h:24,301-303;
 * dynet/tensor.h:44-130).  d[k] for k >= nd is ignored (treated as 1). */
typedef struct dyb200_tensor {
  float* v;
  uint32_t d[7];
  uint32_t nd;
  uint32_t bd;
} dyb200_tensor;

/* Per-device state: device id, stream, a grow-only scratch arena owned by the
 * library (stands in for the SCS pool use of the reference nodes, e.g.
 * dynet/nodes-lstm.cc:125,234), the last error text. Not thread-safe, like the
 * reference (one ComputationGraph per process, dynet/dynet.cc:76-79). */
typedef struct dyb200_ctx dyb200_ctx;

/* Creates the context for `device` (cudaSetDevice) using `stream` (NULL = legacy
 * default stream, the one dynet/devices.cc:113-114 uses). */
int dyb200_ctx_create(int device, void* stream, dyb200_ctx** out);
int dyb200_ctx_destroy(dyb200_ctx* ctx);
/* Text of the last non-OK status returned through this context ("" if none). */
const char* dyb200_last_error(const dyb200_ctx* ctx);
/* Reads (and clears) the device-side error word set by kernels that clamp an
 * index or give up a bounded wait; synchronises the stream.  0 = clean. */
int dyb200_ctx_check_device_errors(dyb200_ctx* ctx, uint32_t* flags_out);
/* Number of kernels this library has launched through `ctx` so far. */
uint64_t dyb200_ctx_launch_count(const dyb200_ctx* ctx);
/* Per-launch timing of the GEMM kernels for the benchmark's roofline: between begin and end every
 * GEMM launch (up to `capacity`) is bracketed by CUDA events on the context's stream.  end()
 * synchronises and returns, for index 0 = CUDA-core kernel and 1 = tensor-pipe kernel, the summed
 * device time in ms, the launch count and the useful FLOPs (2*M*N*K per product). */
int dyb200_ctx_profile_begin(dyb200_ctx* ctx, int capacity);
int dyb200_ctx_profile_end(dyb200_ctx* ctx, double ms_out[2], uint64_t launches_out[2], double flops_out[2]);
/* Between begin and end: the number of GEMM launches recorded so far, and launch k of them: shape = {M, N, sum of K,
 * epilogue mode}, path = 1 for the tensor-pipe kernels, its device time (waits for that launch) and its useful FLOPs. */
int dyb200_ctx_profile_count(const dyb200_ctx* ctx);
int dyb200_ctx_profile_launch(dyb200_ctx* ctx, int k, uint32_t shape_out[4], int* path_out, float* ms_out, double* flops_out);
/* Parameter cache for the tensor-pipe GEMM (off by default).  The GEMM splits every operand into
 * TF32 hi/lo planes first; with the cache on, the planes of a PARAMETER matrix (the LSTM's Wx / Wh, or
 * the A operand of dyb200_gemm called with DYB200_GEMM_A_IS_PARAM) are kept and reused until the
 * parameters change.  The caller must call dyb200_ctx_params_changed after every in-place update of
 * parameter values (dyb200_sgd_update does it itself); in a DyNet tree that is the end of
 * Trainer::update (dynet/training.cc:195-265).  Costs up to 2x the size of each cached matrix. */
int dyb200_ctx_param_cache(dyb200_ctx* ctx, int enable);
/* Programmatic dependent launch (off by default).  When on, every kernel of this library is launched so that it may be
 * scheduled while its predecessor in the stream still runs; each kernel waits, before its first memory access, until that
 * predecessor has completed (griddepcontrol.wait), so results do not change - only launch latency overlaps.  Work that other
 * code puts into the same stream between two calls is ordered as usual. */
int dyb200_ctx_dependent_launch(dyb200_ctx* ctx, int enable);
/* K splits of a tensor-pipe product as one thread-block cluster per output tile, reduced through distributed shared memory
 * (on by default).  Off: the splits
 * go through a workspace and a second kernel.  Results are bitwise the same either way. */
int dyb200_ctx_cluster_splitk(dyb200_ctx* ctx, int enable);
int dyb200_ctx_params_changed(dyb200_ctx* ctx);
/* Library build string ("dyb200 <n> sm_100a"). */
const char* dyb200_version(void);

/* ---- attrs structs (the nodes' constructor arguments) ---- */
typedef struct { float alpha, lambda; } dyb200_elu_attrs;               /* dynet/nodes-activations.h:46-53 */
typedef struct { uint32_t dimension; } dyb200_dim_attrs;               /* dynet/nodes-softmaxes.h:26, nodes-logsumexp.h */
/* pval / pvals, dynet/nodes-pickneglogsoftmax.h:11-36.  ids_host == NULL means the caller has
 * already placed the n ids in the node's aux_mem on the device (no host check, no H2D copy);
 * a bad id is then clamped by the kernel and reported by dyb200_ctx_check_device_errors. */
typedef struct { const uint32_t* ids_host; uint32_t n; } dyb200_pick_attrs;
typedef struct {                                                        /* dynet/param-nodes.h:84-110 */
  const float* all_values; /* device, Dim({E}, V) == LookupParameterStorage::all_values */
  uint32_t vocab;          /* V */
  const uint32_t* ids_host; /* NULL: ids already in aux_mem on the device (see dyb200_pick_attrs) */
  uint32_t n;
  float weight_decay_scale; /* params.current_weight_decay() */
} dyb200_lookup_attrs;
typedef struct {                                                        /* dynet/nodes-lstm.h:9-26 */
  int32_t dropout;
  float weightnoise_std;
  float forget_gate_bias;
} dyb200_lstm_gates_attrs;
typedef struct {                                                        /* dynet/nodes-moments.h:35-69 */
  uint32_t dims[2];
  uint32_t ndims;
  uint32_t order;            /* MomentDimension only */
  int32_t include_batch_dim;
  uint32_t overwrite_n;
} dyb200_moment_attrs;

#define DYB200_FWD_ARGS const dyb200_tensor *xs, int nxs, dyb200_tensor *fx, const void *attrs, void *aux_mem, dyb200_ctx *ctx
#define DYB200_BWD_ARGS const dyb200_tensor *xs, int nxs, const dyb200_tensor *fx, const dyb200_tensor *dEdf, unsigned i, dyb200_tensor *dEdxi, const void *attrs, void *aux_mem, dyb200_ctx *ctx

/* ---- A12 unary activations ---- */
int dyb200_tanh_fwd(DYB200_FWD_ARGS);      /* Tanh::forward_dev_impl, dynet/nodes-trig.cc:312-315 */
int dyb200_tanh_bwd(DYB200_BWD_ARGS);      /* dynet/nodes-trig.cc:317-327 */
int dyb200_logistic_fwd(DYB200_FWD_ARGS);  /* LogisticSigmoid, dynet/nodes-activations.cc:64-68 */
int dyb200_logistic_bwd(DYB200_BWD_ARGS);  /* dynet/nodes-activations.cc:70-79 */
int dyb200_rectify_fwd(DYB200_FWD_ARGS);   /* Rectify, dynet/nodes-activations.cc:30-34 */
int dyb200_rectify_bwd(DYB200_BWD_ARGS);   /* dynet/nodes-activations.cc:36-45 */
int dyb200_elu_fwd(DYB200_FWD_ARGS);       /* ExponentialLinearUnit, attrs = dyb200_elu_attrs, dynet/nodes-activations.cc:166-170 */
int dyb200_elu_bwd(DYB200_BWD_ARGS);       /* dynet/nodes-activations.cc:172-181 */

/* ---- A13 cwise binary, with per-dim and batch broadcasting ---- */
int dyb200_cmult_fwd(DYB200_FWD_ARGS);     /* CwiseMultiply, dynet/nodes-arith-cwise.cc:196-251 */
int dyb200_cmult_bwd(DYB200_BWD_ARGS);     /* dynet/nodes-arith-cwise.cc:253-307 */
int dyb200_csum_fwd(DYB200_FWD_ARGS);      /* CwiseSum (layer_norm composite), dynet/nodes-arith-cwise.cc:49-97 */
int dyb200_csum_bwd(DYB200_BWD_ARGS);      /* dynet/nodes-arith-cwise.cc:99-157 */
int dyb200_cdiv_fwd(DYB200_FWD_ARGS);      /* CwiseQuotient (layer_norm composite), dynet/nodes-arith-cwise.cc:337-351 */
int dyb200_cdiv_bwd(DYB200_BWD_ARGS);      /* dynet/nodes-arith-cwise.cc:353-412 */

/* ---- A6-A9 softmax family ---- */
int dyb200_softmax_fwd(DYB200_FWD_ARGS);        /* Softmax, attrs = dyb200_dim_attrs, dynet/nodes-softmaxes.cc:40-87 */
int dyb200_softmax_bwd(DYB200_BWD_ARGS);        /* dynet/nodes-softmaxes.cc:89-131 */
int dyb200_log_softmax_fwd(DYB200_FWD_ARGS);    /* LogSoftmax, aux_mem = 2*cols*bd floats, dynet/nodes-softmaxes.cc:156-183 */
int dyb200_log_softmax_bwd(DYB200_BWD_ARGS);    /* dynet/nodes-softmaxes.cc:186-214 */
int dyb200_logsumexp_dim_fwd(DYB200_FWD_ARGS);  /* LogSumExpDimension, attrs = dyb200_dim_attrs, dynet/nodes-logsumexp.cc:125-131 + tensor.cc:468-507 */
int dyb200_logsumexp_dim_bwd(DYB200_BWD_ARGS);  /* dynet/nodes-logsumexp.cc:133-146 */
int dyb200_logsumexp_fwd(DYB200_FWD_ARGS);      /* n-ary LogSumExp, dynet/nodes-logsumexp.cc:37-73 */
int dyb200_logsumexp_bwd(DYB200_BWD_ARGS);      /* dynet/nodes-logsumexp.cc:75-98 */
/* PickNegLogSoftmax: attrs = dyb200_pick_attrs; aux_mem = 2*bd floats + bd uint32
 * (z, m, flat ids) exactly as aux_storage_size() sizes it, dynet/nodes-pickneglogsoftmax.cc:72-118 */
int dyb200_pickneglogsoftmax_fwd(DYB200_FWD_ARGS);
int dyb200_pickneglogsoftmax_bwd(DYB200_BWD_ARGS); /* dynet/nodes-pickneglogsoftmax.cc:120-146 */
/* Optional, beyond node granularity: the backward pass of loss_c = PickNegLogSoftmax(x_c), x = affine_transform({b, R, h})
 * (the output layer of examples/batching/rnnlm-batch.h:132-135) in one call.  Value-equivalent to
 * dyb200_pickneglogsoftmax_bwd into a zeroed d(x) followed by dyb200_affine_transform_bwd for i = 0, 1, 2
 * (dynet/nodes-pickneglogsoftmax.cc:120-146, dynet/nodes-affinetransform.cc:120-157), but d(x) is never stored as a
 * tensor: one pass over x writes it as the split operands of the two products (dR += d h^T, dh += R^T d) and as
 * per-tile column sums for db.  x: Dim({V}, n) logits; h: Dim({H}, n); R: Dim({V, H}); dEdf: n loss gradients; aux_mem:
 * the PickNegLogSoftmax node's aux_mem as left by its forward call; dR, db, dh are accumulated into.  dx_scratch
 * (Dim({V}, n), overwritten) is only used for shapes too small for the tensor-pipe products and may be NULL otherwise.
 * flags: DYB200_GEMM_A_IS_PARAM when R is a parameter and the parameter cache is on. */
int dyb200_softmax_output_bwd_fused(const dyb200_tensor* x, const dyb200_tensor* h, const dyb200_tensor* R,
                                    const dyb200_tensor* dEdf, const void* aux_mem, dyb200_tensor* dR, dyb200_tensor* db,
                                    dyb200_tensor* dh, dyb200_tensor* dx_scratch, uint32_t flags, dyb200_ctx* ctx);

/* ---- A10-A11 normalisation ---- */
int dyb200_weight_norm_fwd(DYB200_FWD_ARGS);   /* WeightNormalization, dynet/nodes-normalization.cc:28-41 (no host sync: g is read on the device) */
int dyb200_weight_norm_bwd(DYB200_BWD_ARGS);   /* dynet/nodes-normalization.cc:43-66 */
int dyb200_moment_dim_fwd(DYB200_FWD_ARGS);    /* MomentDimension, attrs = dyb200_moment_attrs, dynet/nodes-moments.cc:181-244 */
int dyb200_moment_dim_bwd(DYB200_BWD_ARGS);    /* dynet/nodes-moments.cc:246-310 */
int dyb200_std_dim_fwd(DYB200_FWD_ARGS);       /* StdDimension, attrs = dyb200_moment_attrs, dynet/nodes-moments.cc:434-496 */
int dyb200_std_dim_bwd(DYB200_BWD_ARGS);       /* dynet/nodes-moments.cc:498-556 */
/* The whole layer_norm composite (dynet/expr.cc:248-253: 8 nodes) as one kernel.
 * xs = {x Dim(...,B), g, b (bd 1)}; normalises over all non-batch dims.  Backward
 * index i: 0 = x, 1 = g, 2 = b.  The first backward call of a node computes all
 * three gradients' shared row statistics again; nothing is cached across calls. */
int dyb200_layer_norm_fwd(DYB200_FWD_ARGS);
int dyb200_layer_norm_bwd(DYB200_BWD_ARGS);

/* ---- A4-A5 embedding ---- */
/* LookupNode::forward_dev_impl, attrs = dyb200_lookup_attrs, nxs = 0, aux_mem = bd
 * uint32 (device copy of the ids), dynet/param-nodes.cc:304-329.  Ids are range-
 * checked on the host (the reference checks only in its CPU branch, :323). */
int dyb200_lookup_fwd(DYB200_FWD_ARGS);
/* LookupParameterStorage::accumulate_grads_dev<Device_GPU>, dynet/model.cc:728-747:
 * all_grads[:, ids[b]] += g[:, b] for b in order (deterministic: sort by id, then a
 * segmented row reduction that adds the rows of one id in ascending b). */
int dyb200_lookup_accumulate_grads(unsigned n, const unsigned* ids_host, const unsigned* ids_dev,
                                   const float* g, float* all_grads, unsigned dim_size,
                                   unsigned vocab, dyb200_ctx* ctx);

/* Allocation-free variant of dyb200_lookup_accumulate_grads (no counterpart in the reference).
 * For hosts that must not allocate device memory while training -- e.g. a DyNet-style process whose
 * device memory is a few pools reserved at start-up, or any caller inside a region where cudaMalloc
 * is forbidden.  Same arguments as dyb200_lookup_accumulate_grads, but the sort / segment tables live
 * in a fixed array inside the library image instead of the context's growable arena, and the call
 * performs no cudaMalloc / cudaFree and calls no allocating routine.
 *  - Result: every table row receives its gradient rows one after the other in ascending position,
 *    i.e. bit for bit what the sequential CPU loop of the reference gives.  dyb200_lookup_accumulate_grads
 *    adds an id's rows in chunks of 32 positions, so for an id that occurs more than 32 times the two
 *    entry points may differ by rounding.
 *  - Limit: n <= DYB200_NOALLOC_MAX_IDS ids per call; a larger n returns DYB200_EINVAL.
 *  - Cost: every GPU that loads the library keeps 49,408 bytes for that array until exit.
 *  - The context's device must be the current device of the calling thread (DYB200_EINVAL otherwise;
 *    the call never switches devices).
 *  - The first call on a device looks up the array's device address (a one-time set-up); make that
 *    first call before starting any stream capture: during a capture it returns DYB200_ERUNTIME.
 *  - All calls on a device share the array: two calls that can overlap on the GPU (different
 *    streams, contexts or host threads) race on it.  Calls on one stream are safe, and each call
 *    rewrites everything it reads, so nothing carries over between calls. */
#define DYB200_NOALLOC_MAX_IDS 4096
int dyb200_lookup_accumulate_grads_noalloc(unsigned n, const unsigned* ids_host, const unsigned* ids_dev,
                                           const float* g, float* all_grads, unsigned dim_size,
                                           unsigned vocab, dyb200_ctx* ctx);

/* ---- A1-A3 fused LSTM nodes ---- */
/* VanillaLSTMGates: xs = {x_1..x_k, h_tm1, Wx, Wh, b [, mask_x, mask_h]},
 * attrs = dyb200_lstm_gates_attrs, dynet/nodes-lstm.cc:101-235 / :237-527 */
int dyb200_vanilla_lstm_gates_fwd(DYB200_FWD_ARGS);
int dyb200_vanilla_lstm_gates_bwd(DYB200_BWD_ARGS);
int dyb200_vanilla_lstm_c_fwd(DYB200_FWD_ARGS);  /* xs = {c_tm1, gates}, dynet/nodes-lstm.cc:562-589 */
int dyb200_vanilla_lstm_c_bwd(DYB200_BWD_ARGS);  /* dynet/nodes-lstm.cc:591-615 */
int dyb200_vanilla_lstm_h_fwd(DYB200_FWD_ARGS);  /* xs = {c_t, gates}, dynet/nodes-lstm.cc:650-668 */
int dyb200_vanilla_lstm_h_bwd(DYB200_BWD_ARGS);  /* dynet/nodes-lstm.cc:670-703 */

/* Fused forms of the chain CompactVanillaLSTMBuilder emits per layer and time step
 * (vanilla_lstm_gates[_dropout] -> vanilla_lstm_c -> vanilla_lstm_h, dynet/lstm.cc:1067-1076), for executors
 * that recognise the pattern.  Values are those of the three nodes; only the launch count differs.
 *  fwd: gates = VanillaLSTMGates(x, h_tm1, Wx, Wh, b [, mask_x, mask_h]); c_t = VanillaLSTMC(c_tm1, gates);
 *       h_t = VanillaLSTMH(c_t, gates).  mask_x / mask_h are NULL exactly when attrs->dropout == 0.
 *  bwd: given dEdh (gradient w.r.t. h_t) and dEdc (w.r.t. c_t; NULL = zero), performs what the backward calls of
 *       the H node (i = 0, 1), the C node (i = 0, 1) and the gates node (i = 0..4) perform on a zeroed gates
 *       gradient: dx, dh_tm1, dc_tm1, dWx, dWh, db are ACCUMULATED into (dx / dh_tm1 / dc_tm1 may be NULL when
 *       that argument needs no gradient, e.g. the zero initial state).  The gate gradient is formed once and its
 *       packed form is shared by the four products.  With `deferred` non-NULL (a dyb200_wgrad created with
 *       M = 4H, N0 = I, N1 = H, see below) the two weight-gradient products are not run: their operands are
 *       appended to the accumulator and dWx / dWh (which may then be NULL) are produced by dyb200_wgrad_flush. */
int dyb200_vanilla_lstm_fwd_fused(const dyb200_tensor* x, const dyb200_tensor* h_tm1, const dyb200_tensor* c_tm1,
                                  const dyb200_tensor* Wx, const dyb200_tensor* Wh, const dyb200_tensor* b,
                                  const dyb200_tensor* mask_x, const dyb200_tensor* mask_h,
                                  const dyb200_lstm_gates_attrs* attrs, dyb200_tensor* gates, dyb200_tensor* c_t,
                                  dyb200_tensor* h_t, dyb200_ctx* ctx);
int dyb200_vanilla_lstm_bwd_fused(const dyb200_tensor* x, const dyb200_tensor* h_tm1, const dyb200_tensor* c_tm1,
                                  const dyb200_tensor* Wx, const dyb200_tensor* Wh, const dyb200_tensor* mask_x,
                                  const dyb200_tensor* mask_h, const dyb200_tensor* gates, const dyb200_tensor* c_t,
                                  const dyb200_tensor* dEdh, const dyb200_tensor* dEdc, dyb200_tensor* dx,
                                  dyb200_tensor* dh_tm1, dyb200_tensor* dc_tm1, dyb200_tensor* dWx, dyb200_tensor* dWh,
                                  dyb200_tensor* db, const dyb200_lstm_gates_attrs* attrs, struct dyb200_wgrad* deferred,
                                  dyb200_ctx* ctx);

/* The same two calls for a caller that knows the time step: with `deferred` non-NULL the forward call also places the
 * layer inputs (x .* mask_x, h_tm1 .* mask_h: the B operands of this step's weight-gradient products) at columns
 * [deferred_col, deferred_col + batch) of the accumulator, in the same launch that splits them for the gate product, and
 * the backward call writes only the gate gradient there - no operand-splitting launch remains in the backward step.
 * Use the same column for a step in both calls (e.g. t * batch).  deferred_col = DYB200_WGRAD_APPEND in the backward call
 * gives the behaviour of dyb200_vanilla_lstm_bwd_fused. */
#define DYB200_WGRAD_APPEND 0xffffffffu
int dyb200_vanilla_lstm_fwd_fused_at(const dyb200_tensor* x, const dyb200_tensor* h_tm1, const dyb200_tensor* c_tm1,
                                     const dyb200_tensor* Wx, const dyb200_tensor* Wh, const dyb200_tensor* b,
                                     const dyb200_tensor* mask_x, const dyb200_tensor* mask_h,
                                     const dyb200_lstm_gates_attrs* attrs, dyb200_tensor* gates, dyb200_tensor* c_t,
                                     dyb200_tensor* h_t, struct dyb200_wgrad* deferred, uint32_t deferred_col, dyb200_ctx* ctx);
int dyb200_vanilla_lstm_bwd_fused_at(const dyb200_tensor* x, const dyb200_tensor* h_tm1, const dyb200_tensor* c_tm1,
                                     const dyb200_tensor* Wx, const dyb200_tensor* Wh, const dyb200_tensor* mask_x,
                                     const dyb200_tensor* mask_h, const dyb200_tensor* gates, const dyb200_tensor* c_t,
                                     const dyb200_tensor* dEdh, const dyb200_tensor* dEdc, dyb200_tensor* dx,
                                     dyb200_tensor* dh_tm1, dyb200_tensor* dc_tm1, dyb200_tensor* dWx, dyb200_tensor* dWh,
                                     dyb200_tensor* db, const dyb200_lstm_gates_attrs* attrs, struct dyb200_wgrad* deferred,
                                     uint32_t deferred_col, dyb200_ctx* ctx);

/* Deferred parameter-gradient products.  A parameter shared by all time steps (Wx, Wh of an LSTM layer; the
 * output projection) receives dW += A_t * B_t^T from every step (dynet/nodes-lstm.cc:419-500: dgate * x^T summed over
 * the batch; dynet/nodes-matrixmultiply.cc:61-74).  An accumulator keeps the packed operands of every step side by
 * side and runs ONE product with K = sum of the steps' batch sizes at flush time: the same sum in a different
 * association (parity class 1e-4), a much better shape for the tensor pipe.  One A operand may feed two products
 * (N1 > 0): dWx and dWh of a layer share the gate gradient.  push: a is M x k, b0 / b1 are N0 x k / N1 x k, all
 * column-major; mask0 / mask1 multiply b0 / b1 elementwise (batch size 1 when *_full is 0). */
typedef struct dyb200_wgrad dyb200_wgrad;
int dyb200_wgrad_create(dyb200_ctx* ctx, uint32_t M, uint32_t N0, uint32_t N1, uint32_t Kcap, dyb200_wgrad** out);
int dyb200_wgrad_destroy(dyb200_wgrad* w);
int dyb200_wgrad_push(dyb200_wgrad* w, uint32_t k, const float* a, uint32_t lda, const float* b0, uint32_t ldb0,
                      const float* mask0, int mask0_full, const float* b1, uint32_t ldb1, const float* mask1,
                      int mask1_full, dyb200_ctx* ctx);
/* Optional, for a layer whose inputs of ALL time steps exist before its first step runs (any layer of a stack that is
 * run layer by layer): x_all = Dim({I}, n) holds the inputs of the n / step time steps side by side (`step` columns
 * each), mask_x = Dim({I}, step) or Dim({I}, 1) is the layer's input dropout mask (the same for every time step, as in
 * dynet/lstm.cc:1010-1030) or NULL.  One launch splits x_all .* mask_x into operand planes (one row per column; columns
 * [0, n) of the accumulator) that the gate products and the weight-gradient product both read.  Afterwards dyb200_vanilla_lstm_fwd_fused_at, called
 * with this accumulator for deferred_col = 0, step, 2 step, ... in order, launches no operand split of its own except
 * for h_tm1 of the first step: each step's epilogue also writes h_t .* mask_h as the next step's operand planes.  The pre-split
 * inputs are dropped by dyb200_wgrad_flush (one call per sequence).  The x
 * argument of those calls must be the matching columns of x_all.  Results are bitwise those of the calls without it.
 * step = 0 (mask_x must be NULL): the time steps have varying widths that never grow - the schedule of the batched executor
 * for sentences sorted by length (dynet/exec.cc:481-895), where step t uses the first B_t columns of the states of step
 * t - 1; the calls then pass deferred_col = the sum of the widths before their step. */
int dyb200_wgrad_pack_inputs(dyb200_wgrad* w, const dyb200_tensor* x_all, const dyb200_tensor* mask_x, uint32_t step, dyb200_ctx* ctx);
int dyb200_wgrad_flush(dyb200_wgrad* w, float* C0, uint32_t ldc0, float* C1, uint32_t ldc1, dyb200_ctx* ctx);

/* One LSTM layer over all time steps of a batch of equally long sequences: the calls RNNBuilder::add_input (dynet/rnn.h:120)
 * makes into CompactVanillaLSTMBuilder::add_input_impl (dynet/lstm.cc:1044-1080) for t = 0 .. steps - 1, in one call.
 * x_all = Dim({I}, steps * batch) holds the layer inputs of all steps side by side (batch columns each), gates_all / c_all /
 * h_all = Dim({4H} / {H} / {H}, steps * batch) receive every step's gates, c_t and h_t; h0 / c0 = Dim({H}, batch) are the state
 * before the first step; masks as in dyb200_vanilla_lstm_fwd_fused (the same mask for every step, dynet/lstm.cc:1010-1030).
 * Equivalent, bit for bit, to dyb200_wgrad_pack_inputs(deferred, x_all, mask_x, batch) followed by steps calls of
 * dyb200_vanilla_lstm_fwd_fused_at with deferred_col = t * batch, h_tm1 / c_tm1 = the previous step's outputs.  When the shape
 * allows (tensor-path sizes, whole tiles, every CTA resident at once) the steps run inside ONE kernel whose CTAs stay on the
 * GPU for the whole sequence and hand h_t over through device memory; otherwise the per-step calls are made.
 * dyb200_ctx_sequence_kernels(ctx, 0) forces the per-step form.  deferred may be NULL (per-step form, nothing recorded for
 * the weight gradients). */
int dyb200_vanilla_lstm_seq_fwd(const dyb200_tensor* x_all, const dyb200_tensor* h0, const dyb200_tensor* c0,
                                const dyb200_tensor* Wx, const dyb200_tensor* Wh, const dyb200_tensor* b,
                                const dyb200_tensor* mask_x, const dyb200_tensor* mask_h, const dyb200_lstm_gates_attrs* attrs,
                                dyb200_tensor* gates_all, dyb200_tensor* c_all, dyb200_tensor* h_all, struct dyb200_wgrad* deferred,
                                uint32_t steps, dyb200_ctx* ctx);
/* The backward pass of the same layer over all time steps, in sweep order (dynet/exec.cc:96-140 visits the nodes of step
 * steps - 1 first): equivalent, bit for bit, to calling dyb200_vanilla_lstm_bwd_fused_at for t = steps - 1 .. 0 with
 * gates / c_t / dEdh / dEdc = the columns of step t of gates_all / c_all / dh_all / dc_all, dx = the columns of step t of
 * dx_all, dh_tm1 / dc_tm1 = the columns of step t - 1 of dh_all / dc_all (NULL at t = 0; h_tm1 / c_tm1 are h0 / c0 there) and
 * deferred_col = t * batch.  dh_all / dc_all hold dE/dh_t and dE/dc_t of every
 * step as left by the layers above (the recurrent parts are accumulated into them on the way); dx_all accumulates.  With deferred the columns of the accumulator must hold the
 * layer inputs placed by dyb200_vanilla_lstm_seq_fwd / _fwd_fused_at, and dWx / dWh may be NULL; without it every step adds
 * its weight gradients to dWx / dWh at once.  When the shape allows (as for the forward call; deferred and dx_all given), the
 * steps run inside ONE kernel whose CTAs stay on the GPU: the cell pass and the [Wx; Wh]^T dgates product of a step hand
 * over through counters in device memory, and every CTA alternates between two independent blocks of batch columns so that
 * one block's hand-overs hide behind the other's products (the per-step call uses the same K splits for such shapes, which
 * keeps the two forms bit-identical).  dyb200_ctx_sequence_kernels(ctx, 0) forces the per-step form. */
int dyb200_vanilla_lstm_seq_bwd(const dyb200_tensor* x_all, const dyb200_tensor* h0, const dyb200_tensor* c0,
                                const dyb200_tensor* Wx, const dyb200_tensor* Wh, const dyb200_tensor* mask_x,
                                const dyb200_tensor* mask_h, const dyb200_lstm_gates_attrs* attrs, const dyb200_tensor* gates_all,
                                const dyb200_tensor* c_all, const dyb200_tensor* h_all, dyb200_tensor* dh_all, dyb200_tensor* dc_all,
                                dyb200_tensor* dx_all, dyb200_tensor* dWx, dyb200_tensor* dWh, dyb200_tensor* db,
                                struct dyb200_wgrad* deferred, uint32_t steps, dyb200_ctx* ctx);
/* Sequence-persistent kernels (1, the default): 0 makes dyb200_vanilla_lstm_seq_* issue one call per time step; 2 keeps the
 * kernels but launches them without the cooperative-launch attribute (profilers that cannot replay cooperative launches). */
int dyb200_ctx_sequence_kernels(dyb200_ctx* ctx, int enable);

/* ---- A14 autobatch ragged movers (same argument meaning as dynet/gpu-ops.h:14-15;
 * src/trg/len are DEVICE arrays of num_seqs entries, as dynet/exec.cc:346-356 uploads them) ---- */
int dyb200_parallel_memcpy(int num_seqs, int max_len, float** src, float** trg, size_t* len, dyb200_ctx* ctx);
/* trg[s][0..len[s]) += src[s][...]; sequences that share a target are added in
 * ascending s (deterministic; the reference uses atomicAdd, dynet/gpu-ops.cu:121-145). */
int dyb200_parallel_accumulate(int num_seqs, int max_len, float** src, float** trg, size_t* len, dyb200_ctx* ctx);

/* ---- glue around the hot path (not fused-layer nodes; they let a whole training step stay on the device) ---- */
int dyb200_fill(float* p, size_t n, float value, dyb200_ctx* ctx);            /* TensorTools::constant, dynet/tensor.cc:110-120 */
/* out[0] (+)= sum(x): the value of sum_batches(sum(errs)) over a contiguous block, dynet/nodes-arith-sum.cc (Sum, SumDimension) */
int dyb200_sum_all(const float* x, size_t n, float* out, int accumulate, dyb200_ctx* ctx);
/* out[0] (+)= sum(x^2): ParameterStorage::g_squared_l2norm, dynet/model.cc:547-553 */
int dyb200_squared_norm(const float* x, size_t n, float* out, int accumulate, dyb200_ctx* ctx);
/* SimpleSGDTrainer::update_rule with Trainer::clip_gradients folded in (dynet/training.cc:168-183, :619-622):
 * scale = clip / sqrt(*grad_sumsq) if that norm exceeds clip (clip <= 0 disables); params -= grads * lr * scale; grads = 0
 * (ParameterStorage::clear, dynet/model.cc:111-117).  grad_sumsq is a device scalar. */
int dyb200_sgd_update(float* params, float* grads, size_t n, float lr, float clip_threshold, const float* grad_sumsq,
                      dyb200_ctx* ctx);

/* Trainer update rules over a flat buffer (dynet/training.cc: SimpleSGD :619-622, MomentumSGD :669-673, Adagrad :735-739,
 * Adadelta :802-808, RMSProp :883-888, Adam :955-961, Amsgrad :1034-1041), with Trainer::clip_gradients (:168-183) folded in:
 * gscale = clip_threshold / sqrt(*grad_sumsq) when that norm exceeds clip_threshold (grad_sumsq NULL or clip_threshold <= 0:
 * no clipping).  state0..2 are the rule's shadow buffers (momentum; Adagrad / RMSProp: squared-gradient accumulator;
 * Adadelta: hg, hd; Adam: m, v; Amsgrad: m, v, vhat), NULL where the rule has none.  weight_decay is
 * model->get_weight_decay().current_weight_decay() (1 when unused); updates = Trainer::updates before this update.
 * zero_grads != 0 clears the gradient in the same pass (ParameterStorage::clear, dynet/model.cc:111-117); otherwise the
 * rules that rewrite the gradient in the reference (all but SGD and momentum) leave the same values in it. */
enum { DYB200_RULE_SGD = 0, DYB200_RULE_MOMENTUM = 1, DYB200_RULE_ADAGRAD = 2, DYB200_RULE_ADADELTA = 3, DYB200_RULE_RMSPROP = 4,
       DYB200_RULE_ADAM = 5, DYB200_RULE_AMSGRAD = 6 };
typedef struct {
  float learning_rate, clip_threshold, weight_decay;
  float momentum;          /* MomentumSGD */
  float epsilon;           /* Adagrad, Adadelta, RMSProp, Adam, Amsgrad */
  float rho;               /* Adadelta, RMSProp */
  float beta_1, beta_2;    /* Adam, Amsgrad */
  uint64_t updates;        /* Adam, Amsgrad: number of updates done so far */
} dyb200_trainer_hyper;
int dyb200_trainer_update(int rule, float* params, float* grads, float* state0, float* state1, float* state2, size_t n,
                          const dyb200_trainer_hyper* hyper, const float* grad_sumsq, int zero_grads, dyb200_ctx* ctx);

/* ---- GEMM used by the LSTM gates (dynet/matrix-multiply.h:16-37, :97-117, :162-180) ----
 * C[M x N] (+)= op(A) * op(B), column-major, fp32 in/out, 3xTF32 on the tensor pipe
 * when the shape allows (else an fp32 CUDA-core kernel).  transA/transB as in BLAS. */
#define DYB200_GEMM_A_IS_PARAM 1u /* flags: A is a parameter matrix (see dyb200_ctx_param_cache) */
int dyb200_gemm(int transA, int transB, uint32_t M, uint32_t N, uint32_t K, const float* A,
                uint32_t lda, const float* B, uint32_t ldb, float* C, uint32_t ldc, int accumulate,
                unsigned flags, dyb200_ctx* ctx);

/* ---- MatrixMultiply and AffineTransform nodes (the callers of the products above) ----
 * xs of MatrixMultiply = {A, B}; xs of AffineTransform = {bias, A1, B1, A2, B2, ...}: fx = bias + sum_k A_k * B_k,
 * the bias block tiled over the columns / batch elements of fx when it is smaller (its batch size must then be 1,
 * as on the reference's CPU path).  A left operand with one batch element multiplies all batch columns of the right
 * operand in one product; otherwise the batch elements are multiplied one by one.  Backward: bias gradient summed
 * over the tiles, dA += dEdf * B^T, dB += A^T * dEdf.  attrs may be NULL. */
typedef struct {
  unsigned flags; /* DYB200_GEMM_A_IS_PARAM: the left operands are parameter matrices (see dyb200_ctx_param_cache) */
} dyb200_affine_attrs;
int dyb200_matmul_fwd(DYB200_FWD_ARGS);            /* MatrixMultiply::forward_dev_impl, dynet/nodes-matrixmultiply.cc:50-56 */
int dyb200_matmul_bwd(DYB200_BWD_ARGS);            /* dynet/nodes-matrixmultiply.cc:58-74 */
int dyb200_affine_transform_fwd(DYB200_FWD_ARGS);  /* AffineTransform::forward_dev_impl, dynet/nodes-affinetransform.cc:77-110 */
int dyb200_affine_transform_bwd(DYB200_BWD_ARGS);  /* dynet/nodes-affinetransform.cc:112-157 */

/* ---- glue nodes around the fused layers ----------------------------------------------------------- */
typedef struct { unsigned start, end, dim; } dyb200_pick_range_attrs;                    /* PickRange(start, end, dim) */
typedef struct { unsigned dims[2]; unsigned ndims; int include_batch_dim; } dyb200_sum_dim_attrs;   /* SumDimension(dims, b) */
typedef struct { float c; } dyb200_const_attrs;                                          /* ConstantPlusX / ConstantMinusX */
/* RandomBernoulli(p, scale): element e = (u_e < p) ? scale : 0 with u_e from Philox-4x32-10 keyed by `seed` at counter
 * offset + e / 4.  The reference draws from std::mt19937 (CPU) or cuRAND's default generator (GPU); only the distribution
 * is the same, so parity runs feed masks in instead of drawing them. */
typedef struct { float p, scale; uint64_t seed, offset; } dyb200_bernoulli_attrs;
int dyb200_pick_range_fwd(DYB200_FWD_ARGS);        /* dynet/nodes-select.cc:229-240 */
int dyb200_pick_range_bwd(DYB200_BWD_ARGS);        /* dynet/nodes-select.cc:243-259 */
int dyb200_concatenate_fwd(DYB200_FWD_ARGS);       /* attrs = dyb200_dim_attrs; dynet/nodes-concat.cc:51-68 */
int dyb200_concatenate_bwd(DYB200_BWD_ARGS);       /* dynet/nodes-concat.cc:70-90 */
int dyb200_sum_fwd(DYB200_FWD_ARGS);               /* n-ary Sum, dynet/nodes-arith-sum.cc:66-114 */
int dyb200_sum_bwd(DYB200_BWD_ARGS);               /* dynet/nodes-arith-sum.cc:116-137 */
int dyb200_sum_dim_fwd(DYB200_FWD_ARGS);           /* SumDimension (sum_dim, sum_batches), dynet/nodes-arith-sum.cc:198-217 */
int dyb200_sum_dim_bwd(DYB200_BWD_ARGS);           /* dynet/nodes-arith-sum.cc:219-248 */
int dyb200_squared_norm_fwd(DYB200_FWD_ARGS);      /* dynet/nodes-norms.cc:30-34 */
int dyb200_squared_norm_bwd(DYB200_BWD_ARGS);      /* dynet/nodes-norms.cc:36-46 */
int dyb200_negate_fwd(DYB200_FWD_ARGS);            /* dynet/nodes-arith-unary.cc:195-198 */
int dyb200_negate_bwd(DYB200_BWD_ARGS);            /* dynet/nodes-arith-unary.cc:200-209 */
int dyb200_constant_plus_x_fwd(DYB200_FWD_ARGS);   /* attrs = dyb200_const_attrs; dynet/nodes-arith-const.cc:62-65 */
int dyb200_constant_plus_x_bwd(DYB200_BWD_ARGS);   /* dynet/nodes-arith-const.cc:67-75 */
int dyb200_constant_minus_x_fwd(DYB200_FWD_ARGS);  /* dynet/nodes-arith-const.cc:29-32 */
int dyb200_constant_minus_x_bwd(DYB200_BWD_ARGS);  /* dynet/nodes-arith-const.cc:34-42 */
int dyb200_random_bernoulli_fwd(DYB200_FWD_ARGS);  /* dynet/nodes-random.cc:100-104 (no backward: arity 0) */

#ifdef __cplusplus
}
#endif
#endif /* DYB200_H_ */
