// WeightNormalization, MomentDimension, StdDimension and the fused layer_norm
// composite.  Whole-tensor reductions use a fixed grid of per-CTA partials that
// every CTA of the follow-up kernel re-reduces in the same order, so results are
// reproducible run to run; the gain scalar is read on the device (no host sync).
#include "common.cuh"
#include "reduce.cuh"

namespace {

constexpr int kBlock = 256;
constexpr int kVec = 4;  // float4 per thread cached in the CTA-per-column kernels
constexpr int kColMax = kBlock * 4 * kVec;

// ---------------------------------------------------------------- whole-tensor partial sums
// partial[2*blk] = sum w^2 ; partial[2*blk+1] = sum w*d (d may be null)
__global__ void __launch_bounds__(kBlock) k_sumsq_dot_partial(const float* __restrict__ w, const float* __restrict__ d,
                                                             size_t n, float* __restrict__ partial) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  float ss = 0.f, dot = 0.f;
  const bool vec = aligned16(w) && (d == nullptr || aligned16(d));
  if (vec) {
    size_t n4 = n / 4;
    for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n4; i += (size_t)gridDim.x * kBlock) {
      float4 a = ld4(w + 4 * i);
      ss += (a.x * a.x + a.y * a.y) + (a.z * a.z + a.w * a.w);
      if (d) { float4 b = ld4_stream(d + 4 * i); dot += (a.x * b.x + a.y * b.y) + (a.z * b.z + a.w * b.w); }
    }
    if (blockIdx.x == 0) {
      size_t i = 4 * n4 + threadIdx.x;
      if (i < n) { ss += w[i] * w[i]; if (d) dot += w[i] * d[i]; }
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (size_t)gridDim.x * kBlock) {
      ss += w[i] * w[i];
      if (d) dot += w[i] * d[i];
    }
  }
  ss = block_sum(ss, red);
  dot = block_sum(dot, red);
  if (threadIdx.x == 0) { partial[2 * blockIdx.x] = ss; partial[2 * blockIdx.x + 1] = dot; }
}
// Every CTA reduces the same partial list in the same order.
__device__ __forceinline__ void reduce_partials(const float* partial, int np, float* red, float& ss, float& dot) {
  float a = 0.f, b = 0.f;
  for (int k = threadIdx.x; k < np; k += kBlock) { a += partial[2 * k]; b += partial[2 * k + 1]; }
  ss = block_sum(a, red);
  dot = block_sum(b, red);
}
// MODE 0: y = (w / nrm) * g          MODE 1: dw += (dy / nrm) * g - y * (dot / ss)
template <int MODE>
__global__ void __launch_bounds__(kBlock) k_weight_norm_apply(const float* __restrict__ w, const float* __restrict__ gptr,
                                                             const float* __restrict__ y, const float* __restrict__ dy,
                                                             float* __restrict__ out, size_t n,
                                                             const float* __restrict__ partial, int np) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  float ss, dot;
  reduce_partials(partial, np, red, ss, dot);
  const float nrm = sqrtf(ss), g = gptr[0], t2 = dot / ss, sc = g / nrm;
  const bool vec = aligned16(w) && aligned16(out) && (MODE == 0 || (aligned16(y) && aligned16(dy)));
  const size_t n4 = vec ? n / 4 : 0;
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n4; i += (size_t)gridDim.x * kBlock) {
    if (MODE == 0) {
      float4 a = ld4(w + 4 * i);
      st4_stream(out + 4 * i, make_float4(a.x * sc, a.y * sc, a.z * sc, a.w * sc));
    } else {
      float4 d = ld4_stream(dy + 4 * i), yy = ld4_stream(y + 4 * i), o = ld4_stream(out + 4 * i);
      st4_stream(out + 4 * i, make_float4(o.x + (d.x * sc - yy.x * t2), o.y + (d.y * sc - yy.y * t2),
                                          o.z + (d.z * sc - yy.z * t2), o.w + (d.w * sc - yy.w * t2)));
    }
  }
  for (size_t i = 4 * n4 + (size_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (size_t)gridDim.x * kBlock) {
    if (MODE == 0) out[i] = w[i] * sc;
    else out[i] += dy[i] * sc - y[i] * t2;
  }
}
__global__ void __launch_bounds__(kBlock) k_weight_norm_dg(const float* __restrict__ partial, int np, float* __restrict__ dg) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  float ss, dot;
  reduce_partials(partial, np, red, ss, dot);
  if (threadIdx.x == 0) dg[0] += dot / sqrtf(ss);
}

// ---------------------------------------------------------------- moments
// View of the input as (d0, d1, d2, bd) with a reduce mask per axis.
struct Axes {
  uint32_t s[4];
  uint32_t red[4];  // 1 if the axis is reduced
};
__device__ __forceinline__ float mpow(float v, uint32_t order) {
  return order == 1 ? v : (order == 2 ? v * v : powf(v, (float)order));
}
// One CTA per output element; threads stride over the reduced sub-space.
// MODE 0: moment of `order`; MODE 1: population std (mean first, then squares).
template <int MODE>
__global__ void __launch_bounds__(kBlock) k_moment_generic(const float* __restrict__ x, Axes ax, uint32_t order, float n,
                                                          float* __restrict__ out, size_t nout) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  for (size_t o = blockIdx.x; o < nout; o += gridDim.x) {
    // base offset of this output element
    size_t t = o, base = 0, stride = 1, nred = 1;
    for (int k = 0; k < 4; ++k) {
      if (!ax.red[k]) { base += (t % ax.s[k]) * stride; t /= ax.s[k]; }
      else nred *= ax.s[k];
      stride *= ax.s[k];
    }
    auto offset = [&](size_t r) {
      size_t off = base, st = 1;
      for (int k = 0; k < 4; ++k) {
        if (ax.red[k]) { off += (r % ax.s[k]) * st; r /= ax.s[k]; }
        st *= ax.s[k];
      }
      return off;
    };
    float acc = 0.f;
    if (MODE == 0) {
      for (size_t r = threadIdx.x; r < nred; r += kBlock) acc += mpow(x[offset(r)], order);
      acc = block_sum(acc, red);
      if (threadIdx.x == 0) out[o] = acc / n;
    } else {
      for (size_t r = threadIdx.x; r < nred; r += kBlock) acc += x[offset(r)];
      float mean = block_sum(acc, red) / n;
      float q = 0.f;
      for (size_t r = threadIdx.x; r < nred; r += kBlock) { float d = x[offset(r)] - mean; q += d * d; }
      q = block_sum(q, red);
      if (threadIdx.x == 0) out[o] = sqrtf(q / n);
    }
    __syncthreads();
  }
}
// Backward: one thread per input element.
// MODE 0: dx += dE * order * x^(order-1) / n ; MODE 1: dx += (2/n)(x - mean) * dE / (2 fx), mean recomputed per output.
template <int MODE>
__global__ void __launch_bounds__(kBlock) k_moment_bwd_generic(const float* __restrict__ x, Axes ax, uint32_t order, float n,
                                                              const float* __restrict__ fx, const float* __restrict__ dE,
                                                              const float* __restrict__ mean, float* __restrict__ dx,
                                                              size_t total) {
  dyb_grid_dep_sync();
  for (size_t e = (size_t)blockIdx.x * kBlock + threadIdx.x; e < total; e += (size_t)gridDim.x * kBlock) {
    size_t t = e, o = 0, ostride = 1;
    for (int k = 0; k < 4; ++k) {
      uint32_t ik = (uint32_t)(t % ax.s[k]);
      t /= ax.s[k];
      if (!ax.red[k]) { o += ik * ostride; ostride *= ax.s[k]; }
    }
    float v = x[e];
    if (MODE == 0) {
      if (order == 1) dx[e] += dE[o] / n;
      else if (order == 2) dx[e] += (dE[o] * v) * (2.f / n);
      else if (order == 3) dx[e] += (dE[o] * (v * v)) * (3.f / n);
      else dx[e] += (dE[o] * powf(v, (float)order - 1.f)) * ((float)order / n);
    } else {
      dx[e] += (2.f / n) * (v - mean[o]) * (dE[o] / (2.f * fx[o]));
    }
  }
}

// ---------------------------------------------------------------- fused layer_norm
// Column statistics held in registers (n <= 4096, 16-byte aligned columns) or
// re-read (any n).  stats[2c] = mean, stats[2c+1] = sigma.
struct LnLoad {
  const float* xc;
  uint32_t n;
  bool cached;
  float4 v[kVec];
};
__device__ __forceinline__ void ln_stats(LnLoad& L, float* red, float& mean, float& sigma) {
  const float fn = (float)L.n;
  float s = 0.f;
  if (L.cached) {
    const uint32_t n4 = L.n / 4;
#pragma unroll
    for (int k = 0; k < kVec; ++k) {
      uint32_t i = threadIdx.x + kBlock * k;
      if (i < n4) { L.v[k] = ld4_stream(L.xc + 4 * i); s += (L.v[k].x + L.v[k].y) + (L.v[k].z + L.v[k].w); }
    }
  } else {
    for (uint32_t i = threadIdx.x; i < L.n; i += kBlock) s += L.xc[i];
  }
  mean = block_sum(s, red) / fn;
  float q = 0.f;
  if (L.cached) {
    const uint32_t n4 = L.n / 4;
#pragma unroll
    for (int k = 0; k < kVec; ++k) {
      uint32_t i = threadIdx.x + kBlock * k;
      if (i < n4) {
        float a = L.v[k].x - mean, b = L.v[k].y - mean, c = L.v[k].z - mean, d = L.v[k].w - mean;
        q += (a * a + b * b) + (c * c + d * d);
      }
    }
  } else {
    for (uint32_t i = threadIdx.x; i < L.n; i += kBlock) { float d = L.xc[i] - mean; q += d * d; }
  }
  sigma = sqrtf(block_sum(q, red) / fn);
}

__global__ void __launch_bounds__(kBlock) k_layer_norm_fwd(const float* __restrict__ x, const float* __restrict__ g,
                                                          const float* __restrict__ b, float* __restrict__ y,
                                                          uint32_t n, size_t ncols, int cached) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  for (size_t c = blockIdx.x; c < ncols; c += gridDim.x) {
    LnLoad L;
    L.xc = x + c * n; L.n = n; L.cached = cached;
    float mean, sigma;
    ln_stats(L, red, mean, sigma);
    const float neg = -mean, inv = 1.f / (sigma + 1e-8f);   // one reciprocal per column instead of n divisions
    float* yc = y + c * n;
    if (cached) {
      const uint32_t n4 = n / 4;
#pragma unroll
      for (int k = 0; k < kVec; ++k) {
        uint32_t i = threadIdx.x + kBlock * k;
        if (i < n4) {
          float4 gg = ld4(g + 4 * i), bb = ld4(b + 4 * i), v = L.v[k];
          float4 r = make_float4(gg.x * ((v.x + neg) * inv) + bb.x, gg.y * ((v.y + neg) * inv) + bb.y,
                                 gg.z * ((v.z + neg) * inv) + bb.z, gg.w * ((v.w + neg) * inv) + bb.w);
          st4_stream(yc + 4 * i, r);
        }
      }
    } else {
      for (uint32_t i = threadIdx.x; i < n; i += kBlock) yc[i] = g[i] * ((L.xc[i] + neg) * inv) + b[i];
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kBlock) k_layer_norm_bwd_x(const float* __restrict__ x, const float* __restrict__ g,
                                                            const float* __restrict__ dy, float* __restrict__ dx,
                                                            uint32_t n, size_t ncols, int cached) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  const float fn = (float)n;
  for (size_t c = blockIdx.x; c < ncols; c += gridDim.x) {
    LnLoad L;
    L.xc = x + c * n; L.n = n; L.cached = cached;
    float mean, sigma;
    ln_stats(L, red, mean, sigma);
    const float neg = -mean, s2 = sigma + 1e-8f, inv = 1.f / s2;
    const float* dc = dy + c * n;
    float* oc = dx + c * n;
    float4 dq[kVec];
    float A = 0.f, Bs = 0.f;  // A = sum dq*xc (divided by s2^2 once) ; Bs = sum dq (divided by s2 once)
    if (cached) {
      const uint32_t n4 = n / 4;
#pragma unroll
      for (int k = 0; k < kVec; ++k) {
        uint32_t i = threadIdx.x + kBlock * k;
        if (i < n4) {
          float4 d = ld4_stream(dc + 4 * i), gg = ld4(g + 4 * i), v = L.v[k];
          dq[k] = make_float4(d.x * gg.x, d.y * gg.y, d.z * gg.z, d.w * gg.w);
          A += (dq[k].x * (v.x + neg) + dq[k].y * (v.y + neg)) + (dq[k].z * (v.z + neg) + dq[k].w * (v.w + neg));
          Bs += (dq[k].x + dq[k].y) + (dq[k].z + dq[k].w);
        }
      }
    } else {
      for (uint32_t i = threadIdx.x; i < n; i += kBlock) {
        float q = dc[i] * g[i];
        A += q * (L.xc[i] + neg);
        Bs += q;
      }
    }
    A = block_sum(A, red) * inv * inv;
    Bs = block_sum(Bs, red) * inv;
    const float sb = (-A) / (2.f * sigma), dmu_n = (-Bs) / fn, two_n = 2.f / fn;
    if (cached) {
      const uint32_t n4 = n / 4;
#pragma unroll
      for (int k = 0; k < kVec; ++k) {
        uint32_t i = threadIdx.x + kBlock * k;
        if (i < n4) {
          float4 o = ld4_stream(oc + 4 * i), v = L.v[k];
          o.x = ((o.x + two_n * (v.x - mean) * sb) + dq[k].x * inv) + dmu_n;
          o.y = ((o.y + two_n * (v.y - mean) * sb) + dq[k].y * inv) + dmu_n;
          o.z = ((o.z + two_n * (v.z - mean) * sb) + dq[k].z * inv) + dmu_n;
          o.w = ((o.w + two_n * (v.w - mean) * sb) + dq[k].w * inv) + dmu_n;
          st4_stream(oc + 4 * i, o);
        }
      }
    } else {
      for (uint32_t i = threadIdx.x; i < n; i += kBlock)
        oc[i] = ((oc[i] + two_n * (L.xc[i] - mean) * sb) + (dc[i] * g[i]) * inv) + dmu_n;
    }
    __syncthreads();
  }
}

// Columns of at most 1024 elements (n % 128 == 0): one WARP per column, the column in the lanes' registers (NV float4 each),
// both statistics by warp shuffles only - no CTA barrier, eight columns in flight per CTA.  With a CTA per column a
// 4 KB column paid two block reductions (four barriers) for one 16-byte load per thread.
template <int NV>
__global__ void __launch_bounds__(kBlock) k_layer_norm_fwd_warp(const float* __restrict__ x, const float* __restrict__ g,
                                                                const float* __restrict__ b, float* __restrict__ y,
                                                                uint32_t n, size_t ncols) {
  dyb_grid_dep_sync();
  const uint32_t lane = threadIdx.x & 31, n4 = n / 4;
  const float fn = (float)n;
  for (size_t c = (size_t)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); c < ncols; c += (size_t)gridDim.x * (kBlock / 32)) {
    const float* xc = x + c * n;
    float4 v[NV];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const uint32_t i = lane + 32 * k;
      v[k] = i < n4 ? ld4_stream(xc + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
      s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    }
    const float mean = warp_sum(s) / fn;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
      if (lane + 32 * k < n4) {
        const float a = v[k].x - mean, bq = v[k].y - mean, cq = v[k].z - mean, d = v[k].w - mean;
        q += (a * a + bq * bq) + (cq * cq + d * d);
      }
    const float sigma = sqrtf(warp_sum(q) / fn);
    const float neg = -mean, inv = 1.f / (sigma + 1e-8f);
    float* yc = y + c * n;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const uint32_t i = lane + 32 * k;
      if (i < n4) {
        const float4 gg = ld4(g + 4 * i), bb = ld4(b + 4 * i);
        st4_stream(yc + 4 * i, make_float4(gg.x * ((v[k].x + neg) * inv) + bb.x, gg.y * ((v[k].y + neg) * inv) + bb.y,
                                           gg.z * ((v[k].z + neg) * inv) + bb.z, gg.w * ((v[k].w + neg) * inv) + bb.w));
      }
    }
  }
}
template <int NV>
__global__ void __launch_bounds__(kBlock) k_layer_norm_bwd_x_warp(const float* __restrict__ x, const float* __restrict__ g,
                                                                  const float* __restrict__ dy, float* __restrict__ dx,
                                                                  uint32_t n, size_t ncols) {
  dyb_grid_dep_sync();
  const uint32_t lane = threadIdx.x & 31, n4 = n / 4;
  const float fn = (float)n;
  for (size_t c = (size_t)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); c < ncols; c += (size_t)gridDim.x * (kBlock / 32)) {
    const float* xc = x + c * n;
    const float* dc = dy + c * n;
    float* oc = dx + c * n;
    float4 v[NV], dq[NV];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {   // x and dy of the column are requested together
      const uint32_t i = lane + 32 * k;
      v[k] = i < n4 ? ld4_stream(xc + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
      dq[k] = i < n4 ? ld4_stream(dc + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
      s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    }
    const float mean = warp_sum(s) / fn;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
      if (lane + 32 * k < n4) {
        const float a = v[k].x - mean, bq = v[k].y - mean, cq = v[k].z - mean, d = v[k].w - mean;
        q += (a * a + bq * bq) + (cq * cq + d * d);
      }
    const float sigma = sqrtf(warp_sum(q) / fn);
    const float neg = -mean, s2 = sigma + 1e-8f, inv = 1.f / s2;
    float A = 0.f, Bs = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const uint32_t i = lane + 32 * k;
      if (i < n4) {
        const float4 gg = ld4(g + 4 * i);
        dq[k] = make_float4(dq[k].x * gg.x, dq[k].y * gg.y, dq[k].z * gg.z, dq[k].w * gg.w);
        A += (dq[k].x * (v[k].x + neg) + dq[k].y * (v[k].y + neg)) + (dq[k].z * (v[k].z + neg) + dq[k].w * (v[k].w + neg));
        Bs += (dq[k].x + dq[k].y) + (dq[k].z + dq[k].w);
      }
    }
    A = warp_sum(A) * inv * inv;
    Bs = warp_sum(Bs) * inv;
    const float sb = (-A) / (2.f * sigma), dmu_n = (-Bs) / fn, two_n = 2.f / fn;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const uint32_t i = lane + 32 * k;
      if (i < n4) {
        float4 o = ld4_stream(oc + 4 * i);
        o.x = ((o.x + two_n * (v[k].x - mean) * sb) + dq[k].x * inv) + dmu_n;
        o.y = ((o.y + two_n * (v[k].y - mean) * sb) + dq[k].y * inv) + dmu_n;
        o.z = ((o.z + two_n * (v[k].z - mean) * sb) + dq[k].z * inv) + dmu_n;
        o.w = ((o.w + two_n * (v[k].w - mean) * sb) + dq[k].w * inv) + dmu_n;
        st4_stream(oc + 4 * i, o);
      }
    }
  }
}

__global__ void __launch_bounds__(kBlock) k_layer_norm_stats(const float* __restrict__ x, float* __restrict__ stats,
                                                            uint32_t n, size_t ncols, int cached) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  for (size_t c = blockIdx.x; c < ncols; c += gridDim.x) {
    LnLoad L;
    L.xc = x + c * n; L.n = n; L.cached = cached;
    float mean, sigma;
    ln_stats(L, red, mean, sigma);
    if (threadIdx.x == 0) { stats[2 * c] = mean; stats[2 * c + 1] = sigma; }
    __syncthreads();
  }
}
struct LnDg {
  const float *x, *dy, *stats;
  size_t n;
  __device__ float operator()(size_t r, uint32_t b) const {
    float mean = stats[2 * (size_t)b], s2 = stats[2 * (size_t)b + 1] + 1e-8f;
    return dy[(size_t)b * n + r] * ((x[(size_t)b * n + r] + (-mean)) / s2);
  }
};
struct LnDb {
  const float* dy;
  size_t n;
  __device__ float operator()(size_t r, uint32_t b) const { return dy[(size_t)b * n + r]; }
};

int moment_setup(dyb200_ctx* ctx, const dyb200_tensor* x, const dyb200_moment_attrs* a, const char* name, Axes* ax,
                 float* n_out, size_t* nout) {
  DYB_CHECK_ARG(ctx, a != nullptr, "%s: attrs required", name);
  DYB_CHECK_ARG(ctx, x->nd <= 3, "%s implemented up to tensors of order 3 (with minibatch) for now", name);
  DYB_CHECK_ARG(ctx, a->ndims <= 2, "Number of dimensions to reduce (excluding batch dimension) implemented up to 2 in %s (received %u)", name, a->ndims);
  if (a->ndims == 0) DYB_CHECK_ARG(ctx, a->include_batch_dim, "At least one dimension has to be reduced (including batch dimension) in %s", name);
  for (int k = 0; k < 3; ++k) { ax->s[k] = t_dim(x, k); ax->red[k] = 0; }
  ax->s[3] = x->bd;
  ax->red[3] = a->include_batch_dim ? 1 : 0;
  float n = 1.f;
  for (uint32_t k = 0; k < a->ndims; ++k) {
    DYB_CHECK_ARG(ctx, a->dims[k] < 3 && a->dims[k] <= x->nd, "dimension %u is out of bounds of tensor of order %u in %s", a->dims[k], x->nd, name);
    ax->red[a->dims[k]] = 1;
    n *= (float)t_dim(x, a->dims[k]);
  }
  if (a->include_batch_dim) n *= (float)x->bd;
  if (a->overwrite_n) n = (float)a->overwrite_n;
  size_t no = 1;
  for (int k = 0; k < 4; ++k) if (!ax->red[k]) no *= ax->s[k];
  *n_out = n;
  *nout = no;
  return DYB200_OK;
}

int ln_check(dyb200_ctx* ctx, const dyb200_tensor* xs, int nxs, size_t* n, size_t* ncols, int* cached) {
  DYB_CHECK_ARG(ctx, nxs == 3, "layer_norm expects (x, g, b)");
  *n = t_batch_size(&xs[0]);
  *ncols = xs[0].bd;
  DYB_CHECK_ARG(ctx, t_size(&xs[1]) == *n && t_size(&xs[2]) == *n, "layer_norm: gain and bias must have the size of one batch element of x and batch size 1");
  DYB_CHECK_ARG(ctx, *n <= 0xffffffffu, "layer_norm: batch element too large");
  *cached = (*n <= (size_t)kColMax && *n % 4 == 0 && aligned16(xs[0].v) && aligned16(xs[1].v) && aligned16(xs[2].v)) ? 1 : 0;
  return DYB200_OK;
}

}  // namespace

extern "C" {

int dyb200_weight_norm_fwd(DYB200_FWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)attrs; (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 2, "Failed input count check in WeightNormalization");
  DYB_CHECK_ARG(ctx, t_size(&xs[1]) == 1, "Size of gain parameter in WeightNormalization should be 1, received %zu", t_size(&xs[1]));
  size_t n = t_size(&xs[0]);
  DYB_CHECK_ARG(ctx, t_size(fx) == n, "WeightNormalization: output size mismatch");
  if (n == 0) return DYB200_OK;
  int np = ctx->sm_count * 4;
  void* partial;
  int rc = dyb200_scratch(ctx, 2 * np * sizeof(float), &partial);
  if (rc) return rc;
  dyb_launch(k_sumsq_dot_partial, np, kBlock, 0, ctx, xs[0].v, nullptr, n, (float*)partial);
  DYB_LAUNCHED(ctx);
  dyb_launch(k_weight_norm_apply<0>, stream_grid(ctx, n, kBlock * 4), kBlock, 0, ctx, xs[0].v, xs[1].v, nullptr, nullptr, fx->v, n, (const float*)partial, np);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_weight_norm_bwd(DYB200_BWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)attrs; (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 2 && i < 2, "Failed dimension check in WeightNormalization::backward");
  size_t n = t_size(&xs[0]);
  DYB_CHECK_ARG(ctx, t_size(dEdf) == n && t_size(fx) == n && t_size(dEdxi) == (i == 0 ? n : 1), "WeightNormalization::backward: size mismatch");
  if (n == 0) return DYB200_OK;
  int np = ctx->sm_count * 4;
  void* partial;
  int rc = dyb200_scratch(ctx, 2 * np * sizeof(float), &partial);
  if (rc) return rc;
  dyb_launch(k_sumsq_dot_partial, np, kBlock, 0, ctx, xs[0].v, dEdf->v, n, (float*)partial);
  DYB_LAUNCHED(ctx);
  if (i == 0) dyb_launch(k_weight_norm_apply<1>, stream_grid(ctx, n, kBlock * 4), kBlock, 0, ctx, xs[0].v, xs[1].v, fx->v, dEdf->v, dEdxi->v, n, (const float*)partial, np);
  else dyb_launch(k_weight_norm_dg, 1, kBlock, 0, ctx, (const float*)partial, np, dEdxi->v);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_moment_dim_fwd(DYB200_FWD_ARGS) {
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 1, "Failed input count check in MomentDimension");
  const dyb200_moment_attrs* a = (const dyb200_moment_attrs*)attrs;
  Axes ax; float n; size_t nout;
  int rc = moment_setup(ctx, &xs[0], a, "MomentDimension", &ax, &n, &nout);
  if (rc) return rc;
  DYB_CHECK_ARG(ctx, a->order >= 1, "Order of moment should be >=1 in MomentDimension (received %u)", a->order);
  DYB_CHECK_ARG(ctx, t_size(fx) == nout, "MomentDimension: output size mismatch");
  if (nout == 0) return DYB200_OK;
  dyb_launch(k_moment_generic<0>, stream_grid(ctx, nout, 1), kBlock, 0, ctx, xs[0].v, ax, a->order, n, fx->v, nout);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_moment_dim_bwd(DYB200_BWD_ARGS) {
  (void)aux_mem; (void)fx;
  DYB_CHECK_ARG(ctx, nxs == 1 && i == 0, "Failed dimension check in MomentDimension::backward");
  const dyb200_moment_attrs* a = (const dyb200_moment_attrs*)attrs;
  Axes ax; float n; size_t nout;
  int rc = moment_setup(ctx, &xs[0], a, "MomentDimension", &ax, &n, &nout);
  if (rc) return rc;
  size_t total = t_size(&xs[0]);
  DYB_CHECK_ARG(ctx, t_size(dEdf) == nout && t_size(dEdxi) == total, "MomentDimension::backward: size mismatch");
  if (total == 0) return DYB200_OK;
  dyb_launch(k_moment_bwd_generic<0>, stream_grid(ctx, total, kBlock), kBlock, 0, ctx, xs[0].v, ax, a->order, n, nullptr, dEdf->v, nullptr, dEdxi->v, total);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_std_dim_fwd(DYB200_FWD_ARGS) {
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 1, "Failed input count check in StdDimension");
  Axes ax; float n; size_t nout;
  int rc = moment_setup(ctx, &xs[0], (const dyb200_moment_attrs*)attrs, "StdDimension", &ax, &n, &nout);
  if (rc) return rc;
  DYB_CHECK_ARG(ctx, t_size(fx) == nout, "StdDimension: output size mismatch");
  if (nout == 0) return DYB200_OK;
  dyb_launch(k_moment_generic<1>, stream_grid(ctx, nout, 1), kBlock, 0, ctx, xs[0].v, ax, 2, n, fx->v, nout);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_std_dim_bwd(DYB200_BWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 1 && i == 0, "Failed dimension check in StdDimension::backward");
  Axes ax; float n; size_t nout;
  int rc = moment_setup(ctx, &xs[0], (const dyb200_moment_attrs*)attrs, "StdDimension", &ax, &n, &nout);
  if (rc) return rc;
  size_t total = t_size(&xs[0]);
  DYB_CHECK_ARG(ctx, t_size(dEdf) == nout && t_size(fx) == nout && t_size(dEdxi) == total, "StdDimension::backward: size mismatch");
  if (total == 0) return DYB200_OK;
  // the mean of every reduced group, recomputed as the reference does (nodes-moments.cc:521-523)
  void* mean;
  rc = dyb200_scratch(ctx, nout * sizeof(float), &mean);
  if (rc) return rc;
  dyb_launch(k_moment_generic<0>, stream_grid(ctx, nout, 1), kBlock, 0, ctx, xs[0].v, ax, 1, n, (float*)mean, nout);
  DYB_LAUNCHED(ctx);
  dyb_launch(k_moment_bwd_generic<1>, stream_grid(ctx, total, kBlock), kBlock, 0, ctx, xs[0].v, ax, 2, n, fx->v, dEdf->v, (const float*)mean, dEdxi->v, total);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_layer_norm_fwd(DYB200_FWD_ARGS) {
  (void)attrs; (void)aux_mem;
  size_t n, ncols; int cached;
  int rc = ln_check(ctx, xs, nxs, &n, &ncols, &cached);
  if (rc) return rc;
  DYB_CHECK_ARG(ctx, t_size(fx) == n * ncols, "layer_norm: output size mismatch");
  if (n * ncols == 0) return DYB200_OK;
  cached = cached && aligned16(fx->v);
  if (cached && n % 128 == 0 && n <= 1024 && aligned16(xs[1].v) && aligned16(xs[2].v)) {   // a warp per column
    const unsigned grid = stream_grid(ctx, (ncols + 7) / 8, 1);
    if (n <= 256) dyb_launch(k_layer_norm_fwd_warp<2>, grid, kBlock, 0, ctx, xs[0].v, xs[1].v, xs[2].v, fx->v, (uint32_t)n, ncols);
    else dyb_launch(k_layer_norm_fwd_warp<8>, grid, kBlock, 0, ctx, xs[0].v, xs[1].v, xs[2].v, fx->v, (uint32_t)n, ncols);
    DYB_LAUNCHED(ctx);
    return DYB200_OK;
  }
  dyb_launch(k_layer_norm_fwd, stream_grid(ctx, ncols, 1), kBlock, 0, ctx, xs[0].v, xs[1].v, xs[2].v, fx->v, (uint32_t)n, ncols, cached);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_layer_norm_bwd(DYB200_BWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)attrs; (void)aux_mem; (void)fx;
  size_t n, ncols; int cached;
  int rc = ln_check(ctx, xs, nxs, &n, &ncols, &cached);
  if (rc) return rc;
  DYB_CHECK_ARG(ctx, i < 3, "layer_norm::backward: argument index %u out of range", i);
  DYB_CHECK_ARG(ctx, t_size(dEdf) == n * ncols && t_size(dEdxi) == (i == 0 ? n * ncols : n), "layer_norm::backward: size mismatch");
  if (n * ncols == 0) return DYB200_OK;
  if (i == 0) {
    cached = cached && aligned16(dEdf->v) && aligned16(dEdxi->v);
    if (cached && n % 128 == 0 && n <= 1024 && aligned16(xs[1].v)) {   // a warp per column (1024: 20.5 us against 25.8 us for a CTA per column, 4096 columns)
      const unsigned grid = stream_grid(ctx, (ncols + 7) / 8, 1);
      if (n <= 256) dyb_launch(k_layer_norm_bwd_x_warp<2>, grid, kBlock, 0, ctx, xs[0].v, xs[1].v, dEdf->v, dEdxi->v, (uint32_t)n, ncols);
      else dyb_launch(k_layer_norm_bwd_x_warp<8>, grid, kBlock, 0, ctx, xs[0].v, xs[1].v, dEdf->v, dEdxi->v, (uint32_t)n, ncols);
      DYB_LAUNCHED(ctx);
      return DYB200_OK;
    }
    dyb_launch(k_layer_norm_bwd_x, stream_grid(ctx, ncols, 1), kBlock, 0, ctx, xs[0].v, xs[1].v, dEdf->v, dEdxi->v, (uint32_t)n, ncols, cached);
    DYB_LAUNCHED(ctx);
    return DYB200_OK;
  }
  if (i == 2) {
    LnDb f{dEdf->v, n};
    return batch_reduce_add(ctx, f, n, (uint32_t)ncols, dEdxi->v);
  }
  // i == 1: per-column statistics first
  void* arena;
  rc = dyb200_scratch(ctx, 2 * ncols * sizeof(float), &arena);
  if (rc) return rc;
  float* stats = (float*)arena;
  dyb_launch(k_layer_norm_stats, stream_grid(ctx, ncols, 1), kBlock, 0, ctx, xs[0].v, stats, (uint32_t)n, ncols, cached);
  DYB_LAUNCHED(ctx);
  LnDg f{xs[0].v, dEdf->v, stats, n};
  return batch_reduce_add(ctx, f, n, (uint32_t)ncols, dEdxi->v);
}

}  // extern "C"
