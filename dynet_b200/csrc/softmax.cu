// Softmax (d = 0, 1), LogSoftmax, LogSumExpDimension, n-ary LogSumExp and
// PickNegLogSoftmax.  Reductions along dim 0 work on contiguous columns:
//   rows <= 256          one warp per column, values held in registers
//   rows <= 4096         one 256-thread CTA per column, 128-bit loads, registers
//   larger               one CTA per column, streaming online (max, sum) pass; ops
//                        that must write a full output re-read the column (L2-hot)
// so every forward reads its input from HBM once.  Reductions along dim 1 use
// 8-row x 128-lane tiles so each warp still touches whole 32-byte sectors.
#include <stdlib.h>

#include "common.cuh"
#include "gemm.cuh"
#include "reduce.cuh"

namespace {

constexpr int kBlock = 256;
constexpr int kWarpRowsMax = 256;   // warp-per-column limit (8 values per lane)
constexpr int kWarpVals = kWarpRowsMax / 32;
constexpr int kBlockVec = 4;        // float4 per thread in the CTA-per-column path
constexpr int kBlockRowsMax = kBlock * 4 * kBlockVec;

// One ex2.approx per element (relative error ~2^-22 plus |x - m| * 2^-24 from the scaled argument),
// one rescale test per 16 elements; four 128-bit loads are in flight per thread.
constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

enum Mode { M_SOFTMAX, M_LOGSOFTMAX, M_LSE, M_PNLS };

struct ColArgs {
  const float* x;
  float* y;          // softmax / logsoftmax output
  float* z;          // logsumexp per column (LSE output, PNLS/LogSoftmax aux)
  float* m;          // max per column (aux), may be null
  const uint32_t* ids;  // PNLS: row picked in each column
  float* loss;       // PNLS output
  uint32_t rows;
  size_t ncols;
  uint32_t* flags;
};

template <int MODE>
__device__ __forceinline__ void finish_column(const ColArgs& a, size_t c, float mx, float s, bool leader) {
  if (!leader) return;
  float z = logf(s) + mx;
  if (MODE != M_SOFTMAX) a.z[c] = z;
  if (a.m && MODE != M_SOFTMAX) a.m[c] = mx;
  if (MODE == M_PNLS) {
    uint32_t id = a.ids[c];
    if (id >= a.rows) { atomicOr(a.flags, DYB200_FLAG_BAD_INDEX); id = a.rows - 1; }
    a.loss[c] = z - a.x[c * a.rows + id];
  }
}

// ---- warp per column, rows <= 256 ------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(kBlock) k_col_warp(ColArgs a) {
  dyb_grid_dep_sync();
  const int lane = threadIdx.x & 31;
  const size_t warps = (size_t)gridDim.x * (kBlock / 32);
  for (size_t c = (size_t)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); c < a.ncols; c += warps) {
    const float* xc = a.x + c * a.rows;
    float v[kWarpVals];
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < kWarpVals; ++k) {
      uint32_t r = lane + 32 * k;
      v[k] = r < a.rows ? xc[r] : -INFINITY;
      mx = fmaxf(mx, v[k]);
    }
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kWarpVals; ++k) {
      uint32_t r = lane + 32 * k;
      float e = r < a.rows ? expf(v[k] - mx) : 0.f;
      if (MODE == M_SOFTMAX) v[k] = e;
      s += e;
    }
    s = warp_sum(s);
    finish_column<MODE>(a, c, mx, s, lane == 0);
    if (MODE == M_SOFTMAX || MODE == M_LOGSOFTMAX) {
      float z = logf(s) + mx;
      float* yc = a.y + c * a.rows;
#pragma unroll
      for (int k = 0; k < kWarpVals; ++k) {
        uint32_t r = lane + 32 * k;
        if (r < a.rows) yc[r] = MODE == M_SOFTMAX ? v[k] / s : v[k] - z;
      }
    }
  }
}

// ---- CTA per column, rows <= 4096, 16-byte aligned columns --------------------
template <int MODE>
__global__ void __launch_bounds__(kBlock) k_col_block_vec(ColArgs a) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  const uint32_t rows4 = a.rows / 4;
  for (size_t c = blockIdx.x; c < a.ncols; c += gridDim.x) {
    const float* xc = a.x + c * a.rows;
    float4 v[kBlockVec];
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < kBlockVec; ++k) {
      uint32_t i = threadIdx.x + kBlock * k;
      if (i < rows4) {
        v[k] = ld4_stream(xc + 4 * i);
        mx = fmaxf(mx, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
      }
    }
    mx = block_max(mx, red);
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kBlockVec; ++k) {
      uint32_t i = threadIdx.x + kBlock * k;
      if (i < rows4) {
        const float ml = mx * kLog2e;
        float4 e = make_float4(ex2_approx(fmaf(v[k].x, kLog2e, -ml)), ex2_approx(fmaf(v[k].y, kLog2e, -ml)),
                               ex2_approx(fmaf(v[k].z, kLog2e, -ml)), ex2_approx(fmaf(v[k].w, kLog2e, -ml)));
        s += (e.x + e.y) + (e.z + e.w);
        if (MODE == M_SOFTMAX) v[k] = e;
      }
    }
    s = block_sum(s, red);
    finish_column<MODE>(a, c, mx, s, threadIdx.x == 0);
    if (MODE == M_SOFTMAX || MODE == M_LOGSOFTMAX) {
      float z = logf(s) + mx;
      const float inv = 1.f / s;   // one division per column
      float* yc = a.y + c * a.rows;
#pragma unroll
      for (int k = 0; k < kBlockVec; ++k) {
        uint32_t i = threadIdx.x + kBlock * k;
        if (i < rows4) {
          float4 r = MODE == M_SOFTMAX ? make_float4(v[k].x * inv, v[k].y * inv, v[k].z * inv, v[k].w * inv)
                                       : make_float4(v[k].x - z, v[k].y - z, v[k].z - z, v[k].w - z);
          st4_stream(yc + 4 * i, r);
        }
      }
    }
    __syncthreads();
  }
}

// ---- CTA per column, any length: streaming online (max, sum) -------------------
// The running sum is kept in base 2 relative to the running max: s = sum 2^((x - m) * log2(e)).
// A -inf entry contributes nothing (the reference subtracts the column maximum first, so it sees exp(-inf) = 0); while the
// running maximum itself is still -inf the exponent would be inf - inf, so such entries are skipped / the shift is 0.
__device__ __forceinline__ void online_add(float& m, float& s, float v) {
  if (v > m) { s = s * ex2_approx((m - v) * kLog2e) + 1.f; m = v; }
  else if (v != -INFINITY) s += ex2_approx((v - m) * kLog2e);
}
__device__ __forceinline__ float shift_log2(float m) { return m == -INFINITY ? 0.f : m * kLog2e; }
__device__ __forceinline__ float max4(float4 v) { return fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)); }
__device__ __forceinline__ float sumexp4(float4 v, float ml) {
  return (ex2_approx(fmaf(v.x, kLog2e, -ml)) + ex2_approx(fmaf(v.y, kLog2e, -ml))) +
         (ex2_approx(fmaf(v.z, kLog2e, -ml)) + ex2_approx(fmaf(v.w, kLog2e, -ml)));
}
template <int MODE>
__global__ void __launch_bounds__(kBlock) k_col_stream(ColArgs a) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  for (size_t c = blockIdx.x; c < a.ncols; c += gridDim.x) {
    const float* xc = a.x + c * a.rows;
    float m = -INFINITY, s = 0.f;
    // peel to a 16-byte boundary, then 128-bit loads, then the tail
    uint32_t head = (uint32_t)(((16 - (reinterpret_cast<uintptr_t>(xc) & 15)) & 15) / 4);
    if (head > a.rows) head = a.rows;
    uint32_t body4 = (a.rows - head) / 4;
    if (threadIdx.x < head) online_add(m, s, xc[threadIdx.x]);
    const float* xb = xc + head;
    uint32_t i = threadIdx.x;
    for (; i + 3 * kBlock < body4; i += 4 * kBlock) {
      float4 v0 = ld4_stream(xb + 4 * i), v1 = ld4_stream(xb + 4 * (i + kBlock));
      float4 v2 = ld4_stream(xb + 4 * (i + 2 * kBlock)), v3 = ld4_stream(xb + 4 * (i + 3 * kBlock));
      float vm = fmaxf(fmaxf(max4(v0), max4(v1)), fmaxf(max4(v2), max4(v3)));
      if (vm > m) { s *= ex2_approx((m - vm) * kLog2e); m = vm; }
      const float ml = shift_log2(m);
      s += (sumexp4(v0, ml) + sumexp4(v1, ml)) + (sumexp4(v2, ml) + sumexp4(v3, ml));
    }
    for (; i < body4; i += kBlock) {
      float4 v = ld4_stream(xb + 4 * i);
      float vm = max4(v);
      if (vm > m) { s *= ex2_approx((m - vm) * kLog2e); m = vm; }
      s += sumexp4(v, shift_log2(m));
    }
    uint32_t t = head + 4 * body4 + threadIdx.x;
    if (t < a.rows) online_add(m, s, xc[t]);
    float mx = block_max(m, red);
    float sc = (m == -INFINITY) ? 0.f : s * ex2_approx((m - mx) * kLog2e);
    float tot = block_sum(sc, red);
    finish_column<MODE>(a, c, mx, tot, threadIdx.x == 0);
    if (MODE == M_SOFTMAX || MODE == M_LOGSOFTMAX) {
      float z = logf(tot) + mx;
      float* yc = a.y + c * a.rows;
      for (uint32_t r = threadIdx.x; r < a.rows; r += kBlock)
        yc[r] = MODE == M_SOFTMAX ? expf(xc[r] - mx) / tot : xc[r] - z;
    }
    __syncthreads();
  }
}

template <int MODE>
int run_columns(dyb200_ctx* ctx, ColArgs a) {
  if (a.ncols == 0 || a.rows == 0) return DYB200_OK;
  a.flags = ctx->dev_flags;
  if (a.rows <= kWarpRowsMax) {
    dyb_launch(k_col_warp<MODE>, stream_grid(ctx, a.ncols, kBlock / 32), kBlock, 0, ctx, a);
  } else if (a.rows <= kBlockRowsMax && a.rows % 4 == 0 && aligned16(a.x) && (a.y == nullptr || aligned16(a.y))) {
    dyb_launch(k_col_block_vec<MODE>, stream_grid(ctx, a.ncols, 1), kBlock, 0, ctx, a);
  } else {
    dyb_launch(k_col_stream<MODE>, stream_grid(ctx, a.ncols, 1), kBlock, 0, ctx, a);
  }
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

// ---- backward along dim 0: needs one dot product per column, then a RMW pass ---
// SOFTMAX: z = sum(y*dy); dx += (dy - z) * y      LOGSOFTMAX: z = sum(dy); dx += exp(y) * -z + dy
template <bool LOGSM>
__global__ void __launch_bounds__(kBlock) k_col_bwd(const float* __restrict__ y, const float* __restrict__ dy,
                                                   float* __restrict__ dx, uint32_t rows, size_t ncols) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  for (size_t c = blockIdx.x; c < ncols; c += gridDim.x) {
    const float *yc = y + c * rows, *dc = dy + c * rows;
    float* xc = dx + c * rows;
    float acc = 0.f;
    for (uint32_t r = threadIdx.x; r < rows; r += kBlock) acc += LOGSM ? dc[r] : yc[r] * dc[r];
    float z = block_sum(acc, red);
    for (uint32_t r = threadIdx.x; r < rows; r += kBlock)
      xc[r] += LOGSM ? (expf(yc[r]) * -z + dc[r]) : (dc[r] - z) * yc[r];
    __syncthreads();
  }
}
template <bool LOGSM>
__global__ void __launch_bounds__(kBlock) k_col_bwd_warp(const float* __restrict__ y, const float* __restrict__ dy,
                                                        float* __restrict__ dx, uint32_t rows, size_t ncols) {
  dyb_grid_dep_sync();
  const int lane = threadIdx.x & 31;
  const size_t warps = (size_t)gridDim.x * (kBlock / 32);
  for (size_t c = (size_t)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); c < ncols; c += warps) {
    const float *yc = y + c * rows, *dc = dy + c * rows;
    float* xc = dx + c * rows;
    float acc = 0.f;
    for (uint32_t r = lane; r < rows; r += 32) acc += LOGSM ? dc[r] : yc[r] * dc[r];
    float z = warp_sum(acc);
    for (uint32_t r = lane; r < rows; r += 32)
      xc[r] += LOGSM ? (expf(yc[r]) * -z + dc[r]) : (dc[r] - z) * yc[r];
  }
}
// 128-bit variant for 16-byte aligned columns held in registers (rows <= 4096).
template <bool LOGSM>
__global__ void __launch_bounds__(kBlock) k_col_bwd_vec(const float* __restrict__ y, const float* __restrict__ dy,
                                                       float* __restrict__ dx, uint32_t rows, size_t ncols) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  const uint32_t rows4 = rows / 4;
  for (size_t c = blockIdx.x; c < ncols; c += gridDim.x) {
    const float *yc = y + c * rows, *dc = dy + c * rows;
    float* xc = dx + c * rows;
    float4 vy[kBlockVec], vd[kBlockVec], vx[kBlockVec];
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < kBlockVec; ++k) {
      uint32_t i = threadIdx.x + kBlock * k;
      if (i < rows4) {
        vy[k] = ld4_stream(yc + 4 * i); vd[k] = ld4_stream(dc + 4 * i); vx[k] = ld4_stream(xc + 4 * i);
        acc += LOGSM ? (vd[k].x + vd[k].y) + (vd[k].z + vd[k].w)
                     : (vy[k].x * vd[k].x + vy[k].y * vd[k].y) + (vy[k].z * vd[k].z + vy[k].w * vd[k].w);
      }
    }
    float z = block_sum(acc, red);
#pragma unroll
    for (int k = 0; k < kBlockVec; ++k) {
      uint32_t i = threadIdx.x + kBlock * k;
      if (i < rows4) {
        float4 r;
        if (LOGSM) r = make_float4(vx[k].x + (expf(vy[k].x) * -z + vd[k].x), vx[k].y + (expf(vy[k].y) * -z + vd[k].y),
                                   vx[k].z + (expf(vy[k].z) * -z + vd[k].z), vx[k].w + (expf(vy[k].w) * -z + vd[k].w));
        else r = make_float4(vx[k].x + (vd[k].x - z) * vy[k].x, vx[k].y + (vd[k].y - z) * vy[k].y,
                             vx[k].z + (vd[k].z - z) * vy[k].z, vx[k].w + (vd[k].w - z) * vy[k].w);
        st4_stream(xc + 4 * i, r);
      }
    }
    __syncthreads();
  }
}
template <bool LOGSM>
int run_col_bwd(dyb200_ctx* ctx, const float* y, const float* dy, float* dx, uint32_t rows, size_t ncols) {
  if (rows == 0 || ncols == 0) return DYB200_OK;
  if (rows <= 128) dyb_launch(k_col_bwd_warp<LOGSM>, stream_grid(ctx, ncols, kBlock / 32), kBlock, 0, ctx, y, dy, dx, rows, ncols);
  else if (rows <= kBlockRowsMax && rows % 4 == 0 && aligned16(y) && aligned16(dy) && aligned16(dx))
    dyb_launch(k_col_bwd_vec<LOGSM>, stream_grid(ctx, ncols, 1), kBlock, 0, ctx, y, dy, dx, rows, ncols);
  else dyb_launch(k_col_bwd<LOGSM>, stream_grid(ctx, ncols, 1), kBlock, 0, ctx, y, dy, dx, rows, ncols);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

// ---- dx[:, c] += exp(x[:, c] - z[c]) * dz[c]   (- dz[c] at the picked row) -------
// LogSumExpDimension(axis 0) and PickNegLogSoftmax backward: one RMW pass.
__global__ void __launch_bounds__(kBlock) k_expsub_bwd(const float* __restrict__ x, const float* __restrict__ z,
                                                      const float* __restrict__ dz, const uint32_t* __restrict__ ids,
                                                      float* __restrict__ dx, uint32_t rows, size_t ncols,
                                                      uint32_t chunks_per_col, uint32_t chunk, int vec) {
  dyb_grid_dep_sync();
  size_t work = (size_t)ncols * chunks_per_col;
  for (size_t w = blockIdx.x; w < work; w += gridDim.x) {
    size_t c = w / chunks_per_col;
    uint32_t r0 = (uint32_t)(w % chunks_per_col) * chunk, r1 = min(rows, r0 + chunk);
    const float zc = z[c], dc = dz[c];
    const float* xc = x + c * rows;
    float* oc = dx + c * rows;
    uint32_t pick = ids ? ids[c] : 0xffffffffu;
    if (vec) {
      for (uint32_t r = r0 + 4 * threadIdx.x; r < r1; r += 4 * kBlock) {
        float4 v = ld4_stream(xc + r), o = ld4_stream(oc + r);
        const float zl = zc * kLog2e;
        float4 res = make_float4(o.x + ex2_approx(fmaf(v.x, kLog2e, -zl)) * dc, o.y + ex2_approx(fmaf(v.y, kLog2e, -zl)) * dc,
                                 o.z + ex2_approx(fmaf(v.z, kLog2e, -zl)) * dc, o.w + ex2_approx(fmaf(v.w, kLog2e, -zl)) * dc);
        if (pick - r < 4u) {
          uint32_t k = pick - r;
          if (k == 0) res.x -= dc; else if (k == 1) res.y -= dc; else if (k == 2) res.z -= dc; else res.w -= dc;
        }
        st4_stream(oc + r, res);
      }
    } else {
      for (uint32_t r = r0 + threadIdx.x; r < r1; r += kBlock) {
        float res = oc[r] + expf(xc[r] - zc) * dc;
        if (r == pick) res -= dc;
        oc[r] = res;
      }
    }
  }
}
int run_expsub_bwd(dyb200_ctx* ctx, const float* x, const float* z, const float* dz, const uint32_t* ids, float* dx,
                   uint32_t rows, size_t ncols) {
  if (rows == 0 || ncols == 0) return DYB200_OK;
  int vec = rows % 4 == 0 && aligned16(x) && aligned16(dx);
  uint32_t chunk = 4 * kBlock * 4;  // 4096 rows per CTA pass
  uint32_t cpc = (rows + chunk - 1) / chunk;
  dyb_launch(k_expsub_bwd, stream_grid(ctx, ncols * cpc, 1), kBlock, 0, ctx, x, z, dz, ids, dx, rows, ncols, cpc, chunk, vec);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

// ---- PickNegLogSoftmax backward written directly as GEMM operands ------------------------------------------------------
// d[r, c] = exp(x[r, c] - z[c]) dz[c]  (- dz[c] at the picked row): the same value k_expsub_bwd adds into a zeroed tensor,
// but stored only as the hi / lo TF32 planes of the two products that consume it in the backward pass of
// x = b + R h:  planes bh / bl [c][r] - K-major right operand of dh += R^T d (reduction index = r) and, as they are, the
// MN-major left operand of dR += d h^T (reduction index = c) - plus the sums over the 64 columns of the tile for the bias
// gradient (transposed through shared memory).  One 64 x 64 tile per CTA, 16-byte accesses along r.  x is read once;
// nothing else of d reaches HBM (the fp32 tensor, its zero fill, two packing passes and a transposed copy of the planes go).
struct ChunkOfPart {   // f(r, b) = v[r + n * b]
  const float* v; size_t n;
  __device__ float operator()(size_t r, uint32_t b) const { return v[r + n * (size_t)b]; }
};

__global__ void __launch_bounds__(256) k_softmax_bwd_split(const float* __restrict__ x, const float* __restrict__ z,
                                                           const float* __restrict__ dz, const uint32_t* __restrict__ ids,
                                                           uint32_t rows, uint32_t ncols, float* __restrict__ bh,
                                                           float* __restrict__ bl, uint32_t pitch_b,
                                                           float* __restrict__ colsum_part, int vec_in) {
  dyb_grid_dep_sync();
  __shared__ float tile[64][65];   // [column][row]
  const uint32_t r0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
  {
    const uint32_t rq = threadIdx.x & 15, cl = threadIdx.x >> 4;
    const uint32_t r = r0 + 4 * rq;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const uint32_t c = c0 + cl + 16 * p;
      float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < ncols && r < rows) {
        const float zc = z[c], dc = dz[c];
        const uint32_t pick = ids ? ids[c] : 0xffffffffu;
        const float* xc = x + (size_t)c * rows;
        if (vec_in) {   // rows % 4 == 0: the four rows exist; same arithmetic as the vector path of k_expsub_bwd
          const float4 v = ld4_stream(xc + r);
          const float zl = zc * kLog2e;
          d = make_float4(ex2_approx(fmaf(v.x, kLog2e, -zl)) * dc, ex2_approx(fmaf(v.y, kLog2e, -zl)) * dc,
                          ex2_approx(fmaf(v.z, kLog2e, -zl)) * dc, ex2_approx(fmaf(v.w, kLog2e, -zl)) * dc);
          if (pick - r < 4u) {
            const uint32_t k = pick - r;
            if (k == 0) d.x -= dc; else if (k == 1) d.y -= dc; else if (k == 2) d.z -= dc; else d.w -= dc;
          }
          float4 h, l;
          split_tf32(d.x, h.x, l.x); split_tf32(d.y, h.y, l.y); split_tf32(d.z, h.z, l.z); split_tf32(d.w, h.w, l.w);
          st4(bh + (size_t)c * pitch_b + r, h);
          st4(bl + (size_t)c * pitch_b + r, l);
        } else {        // same arithmetic as its scalar path
          float e[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (r + k < rows) {
              e[k] = expf(xc[r + k] - zc) * dc;
              if (r + k == pick) e[k] -= dc;
              float h, l;
              split_tf32(e[k], h, l);
              bh[(size_t)c * pitch_b + r + k] = h;
              bl[(size_t)c * pitch_b + r + k] = l;
            }
          }
          d = make_float4(e[0], e[1], e[2], e[3]);
        }
      }
      float* t = &tile[cl + 16 * p][4 * rq];
      t[0] = d.x; t[1] = d.y; t[2] = d.z; t[3] = d.w;
    }
  }
  __syncthreads();
  {
    const uint32_t cq = threadIdx.x & 15, rl = threadIdx.x >> 4;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const uint32_t rr = rl + 16 * p, r = r0 + rr;
      const float4 d = make_float4(tile[4 * cq][rr], tile[4 * cq + 1][rr], tile[4 * cq + 2][rr], tile[4 * cq + 3][rr]);
      float s = (d.x + d.y) + (d.z + d.w);   // (columns past ncols hold zeros)
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      if (r >= rows) continue;
      if (cq == 0) colsum_part[(size_t)blockIdx.y * rows + r] = s;
    }
  }
}

// ---- reductions along dim 1 (strided): 8 rows x 128 lanes per CTA -------------
constexpr int kRT = 8, kCL = 128, kRowVals = 32;  // registers hold cols <= 4096
enum RowMode { R_SOFTMAX, R_LSE, R_SOFTMAX_BWD, R_LSE_BWD };

__device__ __forceinline__ float tile_reduce(float v, float (*sm)[kCL], int ri, int cj, bool is_max) {
  __syncthreads();
  sm[ri][cj] = v;
  __syncthreads();
  for (int o = kCL / 2; o > 0; o >>= 1) {
    if (cj < o) sm[ri][cj] = is_max ? fmaxf(sm[ri][cj], sm[ri][cj + o]) : sm[ri][cj] + sm[ri][cj + o];
    __syncthreads();
  }
  return sm[ri][0];
}

// x, y, dy, dx: rows x cols per batch element (grid.y = batch); z/m: rows per batch.
template <int MODE>
__global__ void __launch_bounds__(kRT * kCL) k_row(const float* __restrict__ x, const float* __restrict__ aux_in,
                                                  float* __restrict__ out, float* __restrict__ z_out,
                                                  uint32_t rows, uint32_t cols) {
  dyb_grid_dep_sync();
  __shared__ float sm[kRT][kCL];
  const int ri = threadIdx.x % kRT, cj = threadIdx.x / kRT;
  const uint32_t r = blockIdx.x * kRT + ri;
  const size_t boff = (size_t)blockIdx.y * rows * cols;
  const bool live = r < rows;
  const bool cached = cols <= (uint32_t)kCL * kRowVals;
  const float* xb = x + boff + r;
  float v[kRowVals];
  if (MODE == R_SOFTMAX || MODE == R_LSE) {
    float mx = -INFINITY;
    if (cached) {
#pragma unroll
      for (int k = 0; k < kRowVals; ++k) {
        uint32_t c = cj + kCL * k;
        v[k] = (live && c < cols) ? xb[(size_t)c * rows] : -INFINITY;
        mx = fmaxf(mx, v[k]);
      }
    } else if (live) {
      for (uint32_t c = cj; c < cols; c += kCL) mx = fmaxf(mx, xb[(size_t)c * rows]);
    }
    mx = tile_reduce(mx, sm, ri, cj, true);
    // one ex2.approx per element and one reciprocal per row, as in the kernels along dim 0 (expf and a division per element
    // made this kernel bound by instruction issue: 32 values per thread, 1024 threads per CTA)
    const float ml = shift_log2(mx);
    float s = 0.f;
    if (cached) {
#pragma unroll
      for (int k = 0; k < kRowVals; ++k) {
        uint32_t c = cj + kCL * k;
        float e = (live && c < cols) ? ex2_approx(fmaf(v[k], kLog2e, -ml)) : 0.f;
        v[k] = e;
        s += e;
      }
    } else if (live) {
      for (uint32_t c = cj; c < cols; c += kCL) s += ex2_approx(fmaf(xb[(size_t)c * rows], kLog2e, -ml));
    }
    s = tile_reduce(s, sm, ri, cj, false);
    if (MODE == R_LSE) {
      if (live && cj == 0) {
        z_out[(size_t)blockIdx.y * rows + r] = logf(s) + mx;
        if (out) out[(size_t)blockIdx.y * rows + r] = mx;
      }
    } else if (live) {
      float* yb = out + boff + r;
      const float inv = 1.f / s;
      if (cached) {
#pragma unroll
        for (int k = 0; k < kRowVals; ++k) {
          uint32_t c = cj + kCL * k;
          if (c < cols) yb[(size_t)c * rows] = v[k] * inv;
        }
      } else {
        for (uint32_t c = cj; c < cols; c += kCL) yb[(size_t)c * rows] = ex2_approx(fmaf(xb[(size_t)c * rows], kLog2e, -ml)) * inv;
      }
    }
  } else if (MODE == R_SOFTMAX_BWD) {  // x = y, aux_in = dy, out = dx
    const float* db = aux_in + boff + r;
    float acc = 0.f;
    if (live) for (uint32_t c = cj; c < cols; c += kCL) acc += xb[(size_t)c * rows] * db[(size_t)c * rows];
    float z = tile_reduce(acc, sm, ri, cj, false);
    if (live) {
      float* ob = out + boff + r;
      for (uint32_t c = cj; c < cols; c += kCL) ob[(size_t)c * rows] += (db[(size_t)c * rows] - z) * xb[(size_t)c * rows];
    }
  } else {  // R_LSE_BWD: aux_in = z (rows per batch), z_out reused as dz input; out = dx
    if (live) {
      float zc = aux_in[(size_t)blockIdx.y * rows + r], dc = z_out[(size_t)blockIdx.y * rows + r];
      float* ob = out + boff + r;
      for (uint32_t c = cj; c < cols; c += kCL) ob[(size_t)c * rows] += expf(xb[(size_t)c * rows] - zc) * dc;
    }
  }
}

// ---- n-ary LogSumExp ---------------------------------------------------------------
constexpr int kMaxNary = 16;
struct NaryArgs {
  const float* x[kMaxNary];
  uint32_t bd[kMaxNary];
  int k;
};
__global__ void __launch_bounds__(kBlock) k_lse_nary_fwd(NaryArgs a, float* __restrict__ y, size_t n, uint32_t bd) {
  dyb_grid_dep_sync();
  size_t total = n * bd;
  for (size_t e = (size_t)blockIdx.x * kBlock + threadIdx.x; e < total; e += (size_t)gridDim.x * kBlock) {
    size_t r = e % n;
    float mx = -INFINITY;
    for (int j = 0; j < a.k; ++j) mx = fmaxf(mx, a.x[j][a.bd[j] == bd ? e : r]);
    float s = 0.f;
    for (int j = 0; j < a.k; ++j) s += expf(a.x[j][a.bd[j] == bd ? e : r] - mx);
    y[e] = logf(s) + mx;
  }
}
__global__ void __launch_bounds__(kBlock) k_lse_nary_bwd(const float* __restrict__ xi, const float* __restrict__ y,
                                                        const float* __restrict__ dy, float* __restrict__ dxi,
                                                        size_t total, int identity) {
  dyb_grid_dep_sync();
  for (size_t e = (size_t)blockIdx.x * kBlock + threadIdx.x; e < total; e += (size_t)gridDim.x * kBlock)
    dxi[e] += identity ? dy[e] : expf(xi[e] - y[e]) * dy[e];
}
struct NaryBcastBwd {
  const float *xi, *y, *dy;
  size_t n;
  __device__ float operator()(size_t r, uint32_t b) const { return expf(xi[r] - y[(size_t)b * n + r]) * dy[(size_t)b * n + r]; }
};

int check_2d(dyb200_ctx* ctx, const dyb200_tensor* t, const char* name) {
  DYB_CHECK_ARG(ctx, t->nd <= 2, "Bad input dimensions in %s, must be 2 or fewer", name);
  return DYB200_OK;
}

}  // namespace

extern "C" {

int dyb200_softmax_fwd(DYB200_FWD_ARGS) {
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 1, "Failed input count check in Softmax");
  int rc = check_2d(ctx, &xs[0], "Softmax");
  if (rc) return rc;
  uint32_t dimension = attrs ? ((const dyb200_dim_attrs*)attrs)->dimension : 0;
  DYB_CHECK_ARG(ctx, dimension < (xs[0].nd ? xs[0].nd : 1), "reduction dimension must be < number of dimensions, was %u", dimension);
  DYB_CHECK_ARG(ctx, t_size(fx) == t_size(&xs[0]), "Softmax: output size mismatch");
  uint32_t rows = t_rows(&xs[0]), cols = t_cols(&xs[0]), bd = xs[0].bd;
  if (t_size(fx) == 0) return DYB200_OK;
  if (dimension == 0) {
    ColArgs a{xs[0].v, fx->v, nullptr, nullptr, nullptr, nullptr, rows, (size_t)cols * bd, nullptr};
    return run_columns<M_SOFTMAX>(ctx, a);
  }
  dyb_launch(k_row<R_SOFTMAX>, dim3((rows + kRT - 1) / kRT, bd), kRT * kCL, 0, ctx, xs[0].v, nullptr, fx->v, nullptr, rows, cols);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_softmax_bwd(DYB200_BWD_ARGS) {
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 1 && i == 0, "Failed dimension check in Softmax::backward");
  uint32_t dimension = attrs ? ((const dyb200_dim_attrs*)attrs)->dimension : 0;
  DYB_CHECK_ARG(ctx, t_size(fx) == t_size(dEdf) && t_size(fx) == t_size(dEdxi), "Softmax::backward: size mismatch");
  uint32_t rows = t_rows(fx), cols = t_cols(fx), bd = fx->bd;
  if (t_size(fx) == 0) return DYB200_OK;
  if (dimension == 0) return run_col_bwd<false>(ctx, fx->v, dEdf->v, dEdxi->v, rows, (size_t)cols * bd);
  dyb_launch(k_row<R_SOFTMAX_BWD>, dim3((rows + kRT - 1) / kRT, bd), kRT * kCL, 0, ctx, fx->v, dEdf->v, dEdxi->v, nullptr, rows, cols);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_log_softmax_fwd(DYB200_FWD_ARGS) {
  (void)attrs;
  DYB_CHECK_ARG(ctx, nxs == 1, "Failed input count check in LogSoftmax");
  int rc = check_2d(ctx, &xs[0], "LogSoftmax");
  if (rc) return rc;
  DYB_CHECK_ARG(ctx, aux_mem != nullptr, "LogSoftmax: aux_mem (2 * cols * bd floats) required");
  uint32_t rows = t_rows(&xs[0]);
  size_t ncols = (size_t)t_cols(&xs[0]) * xs[0].bd;
  ColArgs a{xs[0].v, fx->v, (float*)aux_mem, (float*)aux_mem + ncols, nullptr, nullptr, rows, ncols, nullptr};
  return run_columns<M_LOGSOFTMAX>(ctx, a);
}

int dyb200_log_softmax_bwd(DYB200_BWD_ARGS) {
  (void)xs; (void)attrs; (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 1 && i == 0, "Failed dimension check in LogSoftmax::backward");
  return run_col_bwd<true>(ctx, fx->v, dEdf->v, dEdxi->v, t_rows(fx), (size_t)t_cols(fx) * fx->bd);
}

int dyb200_logsumexp_dim_fwd(DYB200_FWD_ARGS) {
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 1, "LogSumExpDimension takes only one argument");
  int rc = check_2d(ctx, &xs[0], "LogSumExpDimension");
  if (rc) return rc;
  uint32_t dimension = attrs ? ((const dyb200_dim_attrs*)attrs)->dimension : 0;
  DYB_CHECK_ARG(ctx, dimension < (xs[0].nd ? xs[0].nd : 1), "LogSumExpDimension: dimension %u out of range", dimension);
  uint32_t rows = t_rows(&xs[0]), cols = t_cols(&xs[0]), bd = xs[0].bd;
  DYB_CHECK_ARG(ctx, t_size(fx) == (size_t)(dimension == 0 ? cols : rows) * bd, "LogSumExpDimension: output size mismatch");
  if (t_size(&xs[0]) == 0) return DYB200_OK;
  if (dimension == 0) {
    ColArgs a{xs[0].v, nullptr, fx->v, nullptr, nullptr, nullptr, rows, (size_t)cols * bd, nullptr};
    return run_columns<M_LSE>(ctx, a);
  }
  dyb_launch(k_row<R_LSE>, dim3((rows + kRT - 1) / kRT, bd), kRT * kCL, 0, ctx, xs[0].v, nullptr, nullptr, fx->v, rows, cols);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_logsumexp_dim_bwd(DYB200_BWD_ARGS) {
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 1 && i == 0, "Failed dimension check in LogSumExpDimension::backward");
  uint32_t dimension = attrs ? ((const dyb200_dim_attrs*)attrs)->dimension : 0;
  uint32_t rows = t_rows(&xs[0]), cols = t_cols(&xs[0]), bd = xs[0].bd;
  DYB_CHECK_ARG(ctx, t_size(dEdxi) == t_size(&xs[0]) && t_size(dEdf) == t_size(fx), "LogSumExpDimension::backward: size mismatch");
  if (t_size(&xs[0]) == 0) return DYB200_OK;
  if (dimension == 0) return run_expsub_bwd(ctx, xs[0].v, fx->v, dEdf->v, nullptr, dEdxi->v, rows, (size_t)cols * bd);
  dyb_launch(k_row<R_LSE_BWD>, dim3((rows + kRT - 1) / kRT, bd), kRT * kCL, 0, ctx, xs[0].v, fx->v, dEdxi->v, dEdf->v, rows, cols);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_logsumexp_fwd(DYB200_FWD_ARGS) {
  (void)attrs; (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs >= 1 && nxs <= kMaxNary, "LogSumExp: between 1 and %d arguments supported, got %d", kMaxNary, nxs);
  size_t n = t_batch_size(fx);
  NaryArgs a;
  a.k = nxs;
  for (int j = 0; j < nxs; ++j) {
    DYB_CHECK_ARG(ctx, t_batch_size(&xs[j]) == n && (xs[j].bd == fx->bd || xs[j].bd == 1), "Mismatched input dimensions in LogSumExp");
    a.x[j] = xs[j].v;
    a.bd[j] = xs[j].bd;
  }
  size_t total = n * fx->bd;
  if (total == 0) return DYB200_OK;
  dyb_launch(k_lse_nary_fwd, stream_grid(ctx, total, kBlock), kBlock, 0, ctx, a, fx->v, n, fx->bd);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_logsumexp_bwd(DYB200_BWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)attrs; (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs >= 1 && i < (unsigned)nxs, "Failed dimension check in LogSumExp::backward");
  size_t n = t_batch_size(fx), total = n * fx->bd;
  if (total == 0) return DYB200_OK;
  if (nxs == 1 || xs[i].bd == fx->bd) {
    dyb_launch(k_lse_nary_bwd, stream_grid(ctx, total, kBlock), kBlock, 0, ctx, xs[i].v, fx->v, dEdf->v, dEdxi->v, total, nxs == 1);
    DYB_LAUNCHED(ctx);
    return DYB200_OK;
  }
  NaryBcastBwd f{xs[i].v, fx->v, dEdf->v, n};
  return batch_reduce_add(ctx, f, n, fx->bd, dEdxi->v);
}

int dyb200_pickneglogsoftmax_fwd(DYB200_FWD_ARGS) {
  DYB_CHECK_ARG(ctx, nxs == 1, "Failed input count check in PickNegLogSoftmax");
  DYB_CHECK_ARG(ctx, attrs != nullptr && aux_mem != nullptr, "PickNegLogSoftmax: attrs (ids) and aux_mem required");
  if (t_cols(&xs[0]) != 1) return dyb200_fail(ctx, DYB200_ERUNTIME, "PickNegLogSoftmax::forward not yet implemented for multiple columns");
  const dyb200_pick_attrs* p = (const dyb200_pick_attrs*)attrs;
  uint32_t rows = t_rows(&xs[0]), bd = xs[0].bd;
  DYB_CHECK_ARG(ctx, p->n == bd && fx->bd == bd, "In PickNegLogSoftmax::forward, number of elements in the passed-in index vector (%u) did not match number of elements in mini-batch elements in expression (%u)", p->n, bd);
  float* z = (float*)aux_mem;
  float* m = z + bd;
  uint32_t* ids_dev = (uint32_t*)(m + bd);
  // the reference stores flat indices (b * rows + id); the column kernels index per column
  if (p->ids_host) {
    for (uint32_t b = 0; b < bd; ++b)
      DYB_CHECK_ARG(ctx, p->ids_host[b] < rows, "Index error in PickNegLogSoftmax: Index %u out of bounds for input tensor of %u rows", p->ids_host[b], rows);
    DYB_CUDA(ctx, cudaMemcpyAsync(ids_dev, p->ids_host, bd * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream));
  }  // else: the ids are already in aux_mem on the device; the kernel clamps and flags a bad id
  ColArgs a{xs[0].v, nullptr, z, m, ids_dev, fx->v, rows, bd, nullptr};
  return run_columns<M_PNLS>(ctx, a);
}

int dyb200_pickneglogsoftmax_bwd(DYB200_BWD_ARGS) {
  (void)attrs;
  DYB_CHECK_ARG(ctx, nxs == 1 && i == 0, "Failed dimension check in PickNegLogSoftmax::backward");
  if (t_cols(&xs[0]) != 1) return dyb200_fail(ctx, DYB200_ERUNTIME, "PickNegLogSoftmax::backward not yet implemented for multiple columns");
  uint32_t rows = t_rows(&xs[0]), bd = xs[0].bd;
  DYB_CHECK_ARG(ctx, aux_mem != nullptr && t_size(dEdxi) == t_size(&xs[0]) && t_size(dEdf) == bd && fx->bd == bd, "PickNegLogSoftmax::backward: size mismatch");
  const float* z = (const float*)aux_mem;
  const uint32_t* ids_dev = (const uint32_t*)(z + 2 * (size_t)bd);
  return run_expsub_bwd(ctx, xs[0].v, z, dEdf->v, ids_dev, dEdxi->v, rows, bd);
}

int dyb200_softmax_output_bwd_fused(const dyb200_tensor* x, const dyb200_tensor* h, const dyb200_tensor* R,
                                    const dyb200_tensor* dEdf, const void* aux_mem, dyb200_tensor* dR, dyb200_tensor* db,
                                    dyb200_tensor* dh, dyb200_tensor* dx_scratch, uint32_t flags, dyb200_ctx* ctx) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  DYB_CHECK_ARG(ctx, x && h && R && dEdf && aux_mem && dR && db && dh && x->v && h->v && R->v && dEdf->v && dR->v && db->v && dh->v,
                "softmax_output_bwd_fused: null argument");
  const uint32_t V = t_rows(x), H = t_rows(h), n = x->bd;
  DYB_CHECK_ARG(ctx, t_cols(x) == 1 && t_cols(h) == 1 && h->bd == n && R->nd == 2 && R->bd == 1 && R->d[0] == V && R->d[1] == H &&
                     t_size(dEdf) == n && t_size(dR) == (size_t)V * H && t_size(db) == V && t_size(dh) == (size_t)H * n,
                "softmax_output_bwd_fused: shape mismatch (x %u x %u, h %u x %u)", V, n, H, h->bd);
  if (V == 0 || n == 0 || H == 0) return DYB200_OK;
  const float* z = (const float*)aux_mem;
  const uint32_t* ids_dev = (const uint32_t*)(z + 2 * (size_t)n);
  const double flops = 2.0 * V * (double)H * n;
  if (!(dyb200_tc_eligible(V, H, flops) && dyb200_tc_eligible(H, n, flops))) {
    // small shapes: the node-by-node sequence through the caller's tensor
    DYB_CHECK_ARG(ctx, dx_scratch && dx_scratch->v && t_size(dx_scratch) == (size_t)V * n,
                  "softmax_output_bwd_fused: shapes this small need the V x n scratch tensor");
    DYB_CUDA(ctx, cudaMemsetAsync(dx_scratch->v, 0, (size_t)V * n * sizeof(float), ctx->stream));
    int rc = run_expsub_bwd(ctx, x->v, z, dEdf->v, ids_dev, dx_scratch->v, V, n);
    if (rc) return rc;
    dyb200_tensor dv = *x;   // the gradient of x, with x's shape
    dv.v = dx_scratch->v;
    dyb200_tensor xs[3] = {*db, *R, *h};
    dyb200_affine_attrs at = {flags};
    for (unsigned i = 0; i < 3 && !rc; ++i)
      rc = dyb200_affine_transform_bwd(xs, 3, x, &dv, i, i == 0 ? db : i == 1 ? dR : dh, &at, nullptr, ctx);
    return rc;
  }
  int rc;
  PackedOp dA, dB, hT, RT;
  if ((rc = dyb200_tc_planes(ctx, n, V, &dB))) return rc;   // rows = columns, reduction over the vocabulary
  dA = dB; dA.rows = V; dA.K = n; dA.mn_major = 1;           // the same planes read with the vocabulary as rows
  const dim3 grid((V + 63) / 64, (n + 63) / 64);
  void* part;
  if ((rc = dyb200_scratch(ctx, (size_t)grid.y * V * sizeof(float), &part))) return rc;
  const int vec_in = V % 4 == 0 && aligned16(x->v);
  DYB_CHECK_ARG(ctx, grid.y <= 65535u, "softmax_output_bwd_fused: too many columns (%u)", n);
  dyb_launch(k_softmax_bwd_split, grid, 256, 0, ctx, x->v, z, dEdf->v, ids_dev, V, n, dB.hi, dB.lo, dB.pitch,
             (float*)part, vec_in);
  DYB_LAUNCHED(ctx);
  if ((rc = batch_reduce_add(ctx, ChunkOfPart{(const float*)part, V}, V, grid.y, db->v))) return rc;   // db += sum over column tiles
  // dR += d h^T : M = V, N = H, K = n; both operands MN-major (h split as it lies: row = column, H values)
  if ((rc = dyb200_tc_pack(ctx, h->v, H, true, n, H, nullptr, 0, 0, &hT, nullptr))) return rc;
  hT.rows = H; hT.K = n; hT.mn_major = 1;
  {
    GemmEpilogue e{EPI_ACCUM, dR->v, V, nullptr, 0, 0.f, nullptr, 0, 0};
    if ((rc = dyb200_tc_gemm_packed(ctx, V, H, 1, &dA, &hT, e))) return rc;
  }
  // dh += R^T d : M = H, N = n, K = V
  if (flags & DYB200_GEMM_A_IS_PARAM) rc = dyb200_tc_param(ctx, R->v, V, true, H, V, &RT);
  else rc = dyb200_tc_pack(ctx, R->v, V, true, H, V, nullptr, 0, 0, &RT, nullptr);
  if (rc) return rc;
  GemmEpilogue e{EPI_ACCUM, dh->v, H, nullptr, 0, 0.f, nullptr, 0, 0};
  return dyb200_tc_gemm_packed(ctx, H, n, 1, &RT, &dB, e);
}

}  // extern "C"
