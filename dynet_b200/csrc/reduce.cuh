// Deterministic reduction over the batch axis: out[r] += sum_b f(r, b) for r < n.
// Two fixed stages (ascending b inside a chunk, ascending chunk order after), so
// the result depends only on (n, B, SM count), never on scheduling.
#pragma once
#include "common.cuh"

template <class F>
__global__ void __launch_bounds__(128) k_batch_reduce_partial(F f, size_t n, uint32_t B, uint32_t chunk,
                                                             float* __restrict__ partial,
                                                             float* __restrict__ out, int direct) {
  dyb_grid_dep_sync();
  size_t r = (size_t)blockIdx.x * 128 + threadIdx.x;
  if (r >= n) return;
  uint32_t b0 = blockIdx.y * chunk, b1 = min(B, b0 + chunk);
  float acc = 0.f;
  uint32_t b = b0;
  for (; b + 8 <= b1; b += 8) {   // eight loads in flight, summed in ascending order
    float v[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] = f(r, b + q);
#pragma unroll
    for (int q = 0; q < 8; ++q) acc += v[q];
  }
  for (; b < b1; ++b) acc += f(r, b);
  if (direct) out[r] += acc;
  else partial[(size_t)blockIdx.y * n + r] = acc;
}

static __global__ void __launch_bounds__(128) k_batch_reduce_final(const float* __restrict__ partial, uint32_t S,
                                                                   size_t n, float* __restrict__ out) {
  dyb_grid_dep_sync();
  size_t r = (size_t)blockIdx.x * 128 + threadIdx.x;
  if (r >= n) return;
  float acc = 0.f;
  for (uint32_t s = 0; s < S; ++s) acc += partial[(size_t)s * n + r];
  out[r] += acc;
}
// The same for few outputs and many partial sums (a bias gradient over 100 000 columns: n = 45, S = 2368): a warp per
// output, lane l adds the partials l, l + 32, ... in ascending order (four loads in flight), then the lanes are added by a
// butterfly - a fixed order, so the result is reproducible.
static __global__ void __launch_bounds__(128) k_batch_reduce_final_warp(const float* __restrict__ partial, uint32_t S,
                                                                        size_t n, float* __restrict__ out) {
  dyb_grid_dep_sync();
  const size_t r = (size_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= n) return;
  const uint32_t lane = threadIdx.x & 31;
  float acc = 0.f;
  uint32_t s = lane;
  for (; s + 96 < S; s += 128) {
    const float v0 = partial[(size_t)s * n + r], v1 = partial[(size_t)(s + 32) * n + r], v2 = partial[(size_t)(s + 64) * n + r],
                v3 = partial[(size_t)(s + 96) * n + r];
    acc += v0; acc += v1; acc += v2; acc += v3;
  }
  for (; s < S; s += 32) acc += partial[(size_t)s * n + r];
  acc = warp_sum(acc);
  if (lane == 0) out[r] += acc;
}

template <class F>
static int batch_reduce_add(dyb200_ctx* ctx, F f, size_t n, uint32_t B, float* out) {
  if (n == 0 || B == 0) return DYB200_OK;
  unsigned gx = (unsigned)((n + 127) / 128);
  unsigned want = (16u * ctx->sm_count + gx - 1) / gx;   // about 16 CTAs of 128 threads per SM
  unsigned S = want < 1 ? 1 : want;
  if (S > (B + 15) / 16) S = (B + 15) / 16;
  if (S < 1) S = 1;
  uint32_t chunk = (B + S - 1) / S;
  S = (B + chunk - 1) / chunk;
  if (S == 1) {
    dyb_launch(k_batch_reduce_partial<F>, dim3(gx, 1), 128, 0, ctx, f, n, B, chunk, nullptr, out, 1);
    DYB_LAUNCHED(ctx);
    return DYB200_OK;
  }
  void* scratch = nullptr;
  int rc = dyb200_scratch(ctx, (size_t)S * n * sizeof(float), &scratch);
  if (rc) return rc;
  dyb_launch(k_batch_reduce_partial<F>, dim3(gx, S), 128, 0, ctx, f, n, B, chunk, (float*)scratch, out, 0);
  DYB_LAUNCHED(ctx);
  if (n <= 512 && S >= 64) dyb_launch(k_batch_reduce_final_warp, (unsigned)((n + 3) / 4), 128, 0, ctx, (const float*)scratch, S, n, out);
  else dyb_launch(k_batch_reduce_final, gx, 128, 0, ctx, (const float*)scratch, S, n, out);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}
