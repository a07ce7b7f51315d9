// Small kernels around the hot path that a training step needs and the in-scope nodes do
// not cover: filling a tensor, summing a tensor to a scalar (the Sum / SumDimension nodes at
// the root of the loss), and the SimpleSGD update with DyNet's global-norm gradient clipping.
// All reductions use a fixed grid + ordered second stage, so they are run-to-run reproducible.
#include "common.cuh"

namespace {

constexpr int kBlock = 256;

__global__ void __launch_bounds__(kBlock) k_fill(float* __restrict__ p, size_t n, float v) {
  dyb_grid_dep_sync();
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (size_t)gridDim.x * kBlock) p[i] = v;
}

// partial[blk] = sum over this CTA's grid-stride slice of x (SQUARE: of x^2)
template <bool SQUARE>
__global__ void __launch_bounds__(kBlock) k_sum_partial(const float* __restrict__ x, size_t n, float* __restrict__ partial) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  float acc = 0.f;
  if (aligned16(x)) {
    size_t n4 = n / 4;
    for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n4; i += (size_t)gridDim.x * kBlock) {
      float4 v = ld4(x + 4 * i);
      acc += SQUARE ? (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w) : (v.x + v.y) + (v.z + v.w);
    }
    if (blockIdx.x == 0) {
      size_t i = 4 * n4 + threadIdx.x;
      if (i < n) acc += SQUARE ? x[i] * x[i] : x[i];
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (size_t)gridDim.x * kBlock)
      acc += SQUARE ? x[i] * x[i] : x[i];
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}
__global__ void __launch_bounds__(kBlock) k_sum_final(const float* __restrict__ partial, int np, float* __restrict__ out,
                                                     int accumulate) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  float acc = 0.f;
  for (int k = threadIdx.x; k < np; k += kBlock) acc += partial[k];
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + acc : acc;
}

// p -= g * (lr * gscale), g = 0; gscale = clip / ||g|| when ||g|| > clip (dynet/training.cc:168-183, :619-622).
// sumsq[0] holds the squared global gradient norm (already reduced over ranks when data-parallel).
__global__ void __launch_bounds__(kBlock) k_sgd_update(float* __restrict__ p, float* __restrict__ g, size_t n, float lr,
                                                      float clip, const float* __restrict__ sumsq) {
  dyb_grid_dep_sync();
  float gg = sqrtf(sumsq[0]);
  float gscale = (clip > 0.f && gg > clip) ? clip / gg : 1.f;
  float step = lr * gscale;
  size_t n4 = (aligned16(p) && aligned16(g)) ? n / 4 : 0;
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n4; i += (size_t)gridDim.x * kBlock) {
    float4 pv = ld4(p + 4 * i), gv = ld4(g + 4 * i);
    st4(p + 4 * i, make_float4(pv.x - gv.x * step, pv.y - gv.y * step, pv.z - gv.z * step, pv.w - gv.w * step));
    st4(g + 4 * i, make_float4(0.f, 0.f, 0.f, 0.f));
  }
  for (size_t i = 4 * n4 + (size_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (size_t)gridDim.x * kBlock) {
    p[i] -= g[i] * step;
    g[i] = 0.f;
  }
}

}  // namespace

extern "C" {

int dyb200_fill(float* p, size_t n, float value, dyb200_ctx* ctx) {
  if (n == 0) return DYB200_OK;
  DYB_CHECK_ARG(ctx, p != nullptr, "fill: null pointer");
  dyb_launch(k_fill, stream_grid(ctx, n, kBlock * 4), kBlock, 0, ctx, p, n, value);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

static int sum_impl(const float* x, size_t n, float* out, int square, int accumulate, dyb200_ctx* ctx) {
  DYB_CHECK_ARG(ctx, x != nullptr && out != nullptr, "sum: null pointer");
  int np = ctx->sm_count * 4;
  void* partial;
  int rc = dyb200_scratch(ctx, np * sizeof(float), &partial);
  if (rc) return rc;
  if (square) dyb_launch(k_sum_partial<true>, np, kBlock, 0, ctx, x, n, (float*)partial);
  else dyb_launch(k_sum_partial<false>, np, kBlock, 0, ctx, x, n, (float*)partial);
  DYB_LAUNCHED(ctx);
  dyb_launch(k_sum_final, 1, kBlock, 0, ctx, (const float*)partial, np, out, accumulate);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_sum_all(const float* x, size_t n, float* out, int accumulate, dyb200_ctx* ctx) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  return sum_impl(x, n, out, 0, accumulate, ctx);
}
int dyb200_squared_norm(const float* x, size_t n, float* out, int accumulate, dyb200_ctx* ctx) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  return sum_impl(x, n, out, 1, accumulate, ctx);
}

int dyb200_sgd_update(float* params, float* grads, size_t n, float lr, float clip_threshold, const float* grad_sumsq,
                      dyb200_ctx* ctx) {
  if (n == 0) return DYB200_OK;
  DYB_CHECK_ARG(ctx, params && grads && grad_sumsq, "sgd_update: null pointer");
  dyb_launch(k_sgd_update, stream_grid(ctx, n / 4 + 1, kBlock * 2), kBlock, 0, ctx, params, grads, n, lr, clip_threshold, grad_sumsq);
  DYB_LAUNCHED(ctx);
  ctx->param_version++;   // packed copies of the parameters in the cache are stale now
  return DYB200_OK;
}

}  // extern "C"
