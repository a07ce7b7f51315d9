// Shared host/device helpers for the dyb200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/dyb200.h"

#ifndef __CUDA_ARCH__
#define DYB200_HOST_ONLY 1
#endif

struct dyb200_ctx {
  int device;
  cudaStream_t stream;
  int sm_count;
  char err[512];
  // Arena for node-local temporaries: a bump allocator that every public entry point resets
  // (dyb200_scratch_begin) and nested helpers carve from (dyb200_scratch).  Requests that do not
  // fit are served from overflow blocks that live until the next reset, when the main block is
  // re-sized to the high-water mark.
  void* scratch;
  size_t scratch_bytes, scratch_off, scratch_peak;
  void* overflow[64];
  int n_overflow;
  uint32_t* dev_flags;   // device words: [0] error bits (set by kernels, never traps); [DYB200_DEV_COUNTER0 ..) arrival counters
                         // of kernels whose last CTA finishes a reduction (zero between launches: the last CTA resets them)
  uint64_t launches;     // kernels launched through this context
  // 3xTF32 GEMM state (tensor maps are encoded per call; driver entry point cached)
  void* encode_tiled;    // cuTensorMapEncodeTiled
  // Optional cache of packed (hi/lo, K-major) parameter matrices, so that a weight used by every
  // time step is split once per optimizer step instead of once per GEMM.  Off by default: when on,
  // the caller must report every in-place parameter change (dyb200_ctx_params_changed).
  int pdl;               // launch kernels with programmatic stream serialization (see dyb_launch)
  int cluster_splitk;    // K splits of a tensor-pipe product as one thread-block cluster per tile (see dyb200_ctx_cluster_splitk)
  int param_cache_on;
  // per-device facts this context has established on its device: kernels whose dynamic shared-memory limit is raised
  // (bit per kernel family) and how many thread-block clusters of each size fit on the GPU at once
  uint32_t func_attr_done;
  int max_clusters[2][9];
  // sequence-persistent LSTM kernels (one launch per layer instead of one per time step): on by default
  int seq_kernels;
  int seq_max_clusters[2][9];   // thread-block clusters of each size that fit at once, per tile width (0 = not asked yet)
  int seq_coop;                 // 0 = not tried, 1 = launched with the cooperative attribute, -1 = the driver refused it
  uint64_t param_version, param_tick;
  struct ParamPack {
    const float* src; const float* src2; uint32_t ld, rows, rows2, K, pitch; int k_is_fast;   // src2 / rows2: a second matrix stacked below the first
    uint64_t version, last_use;
    float *hi, *lo; size_t floats;
  } param_pack[24];
  // optional per-launch timing of the GEMM kernels (CUDA events on the launch stream)
  cudaEvent_t* prof_ev;  // 2 * prof_cap events: start/stop pairs
  double* prof_flops;    // useful FLOPs of each recorded launch
  int* prof_path;        // 1 = tensor-pipe kernel, 0 = CUDA-core kernel
  uint32_t* prof_shape;  // 4 words per launch: M, N, sum of K, epilogue mode
  int prof_cap, prof_n;
};

// Brackets a GEMM launch with events when profiling is on (see dyb200_ctx_profile_begin).
struct GemmProfScope {
  dyb200_ctx* ctx; int slot;
  GemmProfScope(dyb200_ctx* c, double flops, int path, uint32_t M = 0, uint32_t N = 0, uint32_t K = 0, uint32_t mode = 0)
      : ctx(c), slot(-1) {
    if (c->prof_ev && c->prof_n < c->prof_cap) {
      slot = c->prof_n++;
      c->prof_flops[slot] = flops;
      c->prof_path[slot] = path;
      c->prof_shape[4 * slot] = M; c->prof_shape[4 * slot + 1] = N; c->prof_shape[4 * slot + 2] = K; c->prof_shape[4 * slot + 3] = mode;
      cudaEventRecord(c->prof_ev[2 * slot], c->stream);
    }
  }
  ~GemmProfScope() { if (slot >= 0) cudaEventRecord(ctx->prof_ev[2 * slot + 1], ctx->stream); }
};

#define DYB200_DEV_WORDS 2048
#define DYB200_DEV_SEQ0 16      // 32 words: hand-over counters of the sequence kernels (zeroed before each launch)
#define DYB200_DEV_COUNTER0 64
#define DYB200_DEV_COUNTERS (DYB200_DEV_WORDS - DYB200_DEV_COUNTER0)
// Device error bits written into ctx->dev_flags.
#define DYB200_FLAG_BAD_INDEX 1u     // an id >= vocab/rows reached a kernel (clamped, not dereferenced)
#define DYB200_FLAG_WAIT_TIMEOUT 2u  // a bounded mbarrier wait ran out

int dyb200_fail(dyb200_ctx* ctx, int code, const char* fmt, ...);
int dyb200_scratch_begin(dyb200_ctx* ctx);                      // start of a public entry point: release everything
int dyb200_scratch(dyb200_ctx* ctx, size_t bytes, void** out);  // 256-byte aligned block, valid until the next begin

#define DYB_CHECK_ARG(ctx, cond, ...)                                    \
  do {                                                                   \
    if (!(cond)) return dyb200_fail((ctx), DYB200_EINVAL, __VA_ARGS__);  \
  } while (0)

#define DYB_CUDA(ctx, expr)                                                            \
  do {                                                                                 \
    cudaError_t e__ = (expr);                                                          \
    if (e__ != cudaSuccess)                                                            \
      return dyb200_fail((ctx), DYB200_ECUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

// Counts the launch and reports a launch-configuration error as a status.
#define DYB_LAUNCHED(ctx)                                                              \
  do {                                                                                 \
    (ctx)->launches++;                                                                 \
    cudaError_t e__ = cudaGetLastError();                                              \
    if (e__ != cudaSuccess)                                                            \
      return dyb200_fail((ctx), DYB200_ECUDA, "kernel launch failed at %s:%d: %s", __FILE__, __LINE__, \
                         cudaGetErrorString(e__));                                     \
  } while (0)

static inline size_t t_batch_size(const dyb200_tensor* t) {
  size_t n = 1;
  for (uint32_t k = 0; k < t->nd; ++k) n *= t->d[k];
  return n;
}
static inline size_t t_size(const dyb200_tensor* t) { return t_batch_size(t) * t->bd; }
static inline uint32_t t_dim(const dyb200_tensor* t, uint32_t k) { return k < t->nd ? t->d[k] : 1u; }
static inline uint32_t t_rows(const dyb200_tensor* t) { return t_dim(t, 0); }
static inline uint32_t t_cols(const dyb200_tensor* t) { return t_dim(t, 1); }
__host__ __device__ static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Grid for a streaming kernel: enough CTAs to cover the work, capped at a
// multiple of the SM count (148 on B200) so every SM holds the same number.
static inline unsigned stream_grid(const dyb200_ctx* ctx, size_t work_items, unsigned per_cta,
                                   unsigned ctas_per_sm = 8) {
  size_t need = (work_items + per_cta - 1) / per_cta;
  size_t cap = (size_t)ctx->sm_count * ctas_per_sm;
  if (need < 1) need = 1;
  return (unsigned)(need < cap ? need : cap);
}

#ifdef __CUDACC__
// Every kernel goes out through this helper.  With programmatic dependent launch on (dyb200_ctx::pdl), a kernel may be
// scheduled while its predecessor in the stream is still running: its launch latency and whatever it does before
// dyb_grid_dep_sync() overlap the predecessor's tail; nothing after that call runs before the predecessor has completed
// and its writes are visible.  With it off the launch is an ordinary stream-ordered one and the device call is a no-op.
template <class... KArgs, class... Args>
inline void dyb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, dyb200_ctx* ctx, Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // a failure is picked up by DYB_LAUNCHED (cudaGetLastError)
}
__device__ __forceinline__ void dyb_grid_dep_sync() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide reductions through shared memory (red must hold 32 floats).
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4_stream(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4_stream(float* p, float4 v) { __stcs(reinterpret_cast<float4*>(p), v); }

__device__ __forceinline__ float sigmoidf_dev(float x) { return 1.0f / (1.0f + expf(-x)); }
// Gate non-linearities of the LSTM products.  They run in GEMM epilogues, 64 per thread with 8 warps per SM, where the
// IEEE division and the accurate expf / tanhf made the epilogue take 11 us of a 56 us tile; ex2.approx and rcp.approx cut
// that.  Errors: sigmoid <= ~1.5e-6 relative for |x| <= 20; tanh <= 2.4e-7 absolute (1 - 2/(1 + e^2x) cancels near 0),
// both far inside the 1e-4 class of LSTM states; the stand-alone Tanh / LogisticSigmoid nodes keep the accurate forms.
// (rcp.approx: 1 ulp; the correctly rounded __frcp_rn is a ~20-instruction sequence that cost 2 - 3 us per time step in the
// epilogues of the LSTM products, where 16 of these run per thread and column on the step's critical path)
__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float gate_sigmoid(float x) { return rcp_approx(1.0f + __expf(-x)); }
__device__ __forceinline__ float gate_tanh(float x) { return 1.0f - 2.0f * rcp_approx(1.0f + __expf(2.0f * x)); }
// x = hi + lo with hi = tf32(x) and lo = tf32(x - hi): the two operand planes of the 3xTF32 products
__device__ __forceinline__ void split_tf32(float v, float& hi, float& lo) {
  uint32_t h, l;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
  hi = __uint_as_float(h);
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(v - hi));
  lo = __uint_as_float(l);
}
// c = i g + f c_tm1 and h = o tanh(c) with one fixed rounding sequence, shared by every kernel that forms them
__device__ __forceinline__ float lstm_cell_c(float i, float g, float f, float c_tm1) { return __fmaf_rn(i, g, __fmul_rn(f, c_tm1)); }
__device__ __forceinline__ float lstm_cell_h(float o, float c) { return __fmul_rn(o, tanhf(c)); }
#endif
