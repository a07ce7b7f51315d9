// Unary activations (Tanh, LogisticSigmoid, Rectify, ExponentialLinearUnit) and the
// broadcasting cwise binaries (CwiseMultiply, CwiseSum, CwiseQuotient).
// One HBM pass per call: 128-bit streaming loads/stores, four vectors in flight per
// thread, grid sized to a multiple of the SM count.  Backward kernels read-modify-
// write dEdxi because the reference's contract is "dEdxi += ...".
#include "common.cuh"
#include "reduce.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

// ------------------------------------------------------------ functors
struct FTanh { __device__ float operator()(float x) const { return tanhf(x); } };
// 1 / (1 + e^-x) with ex2.approx and a correctly rounded reciprocal.  Relative error of __expf(-x): 2 ulp of ex2.approx plus
// |x| log2(e) 2^-24 from the scaled argument, i.e. <= 8e-6 at |x| = 87 and <= 2e-6 for |x| <= 20; no branch.
struct FLogistic { __device__ float operator()(float x) const { return __frcp_rn(1.0f + __expf(-x)); } };
// e^x - 1 for x <= 0 without expm1f, branch-free: the Taylor polynomial of degree 6 for x > -0.25 (error x^6 / 5040 <= 5e-8
// relative), __expf(x) - 1 below (|e^x - 1| >= 0.22 there, so the error of ex2.approx stays below 1e-6 relative).
__device__ __forceinline__ float expm1_neg(float x) {
  float p = fmaf(x, 1.f / 720.f, 1.f / 120.f);
  p = fmaf(x, p, 1.f / 24.f); p = fmaf(x, p, 1.f / 6.f); p = fmaf(x, p, 0.5f); p = fmaf(x, p, 1.f);
  const float e = __expf(x) - 1.f;
  return x > -0.25f ? x * p : e;
}
struct FRectify { __device__ float operator()(float x) const { return fmaxf(x, 0.f); } };
struct FElu {
  float alpha, lambda;
  __device__ float operator()(float x) const { return lambda * (x > 0.f ? x : alpha * expm1_neg(x)); }
};
struct FNegate { __device__ float operator()(float x) const { return -x; } };
struct FConstPlus { float c; __device__ float operator()(float x) const { return x + c; } };
struct FConstMinus { float c; __device__ float operator()(float x) const { return c - x; } };
struct BPass { __device__ float operator()(float, float d) const { return d; } };
struct BNeg { __device__ float operator()(float, float d) const { return -d; } };
// backward: g(a, d) where a is fx (tanh/logistic/rectify) or x (elu)
struct BTanh { __device__ float operator()(float t, float d) const { return (1.f - t * t) * d; } };
struct BLogistic { __device__ float operator()(float t, float d) const { return (1.f - t) * t * d; } };
struct BRectify { __device__ float operator()(float t, float d) const { return (t != 0.f ? 1.f : 0.f) * d; } };
struct BElu {
  float alpha, lambda;
  __device__ float operator()(float x, float d) const { return d * (x > 0.f ? lambda : lambda * alpha * __expf(x)); }   // (error of __expf: see FLogistic)
};

template <class F>
__global__ void __launch_bounds__(kThreads) k_unary_fwd(const float* __restrict__ x, float* __restrict__ y,
                                                       size_t n4, size_t n, F f) {
  dyb_grid_dep_sync();
  const size_t stride = (size_t)gridDim.x * kThreads * kUnroll;
  for (size_t base = (size_t)blockIdx.x * kThreads * kUnroll + threadIdx.x; base < n4; base += stride) {
    float4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      size_t i = base + (size_t)u * kThreads;
      if (i < n4) v[u] = ld4_stream(x + 4 * i);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      size_t i = base + (size_t)u * kThreads;
      if (i < n4) {
        float4 r = make_float4(f(v[u].x), f(v[u].y), f(v[u].z), f(v[u].w));
        st4_stream(y + 4 * i, r);
      }
    }
  }
  if (blockIdx.x == 0) {
    size_t i = 4 * n4 + threadIdx.x;
    if (i < n) y[i] = f(x[i]);
  }
}
template <class F>
__global__ void __launch_bounds__(kThreads) k_unary_fwd_scalar(const float* __restrict__ x, float* __restrict__ y,
                                                              size_t n, F f) {
  dyb_grid_dep_sync();
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (size_t)gridDim.x * kThreads)
    y[i] = f(x[i]);
}

template <class G>
__global__ void __launch_bounds__(kThreads) k_unary_bwd(const float* __restrict__ a, const float* __restrict__ dy,
                                                       float* __restrict__ dx, size_t n4, size_t n, G g) {
  dyb_grid_dep_sync();
  const size_t stride = (size_t)gridDim.x * kThreads * kUnroll;
  for (size_t base = (size_t)blockIdx.x * kThreads * kUnroll + threadIdx.x; base < n4; base += stride) {
    float4 va[kUnroll], vd[kUnroll], vx[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      size_t i = base + (size_t)u * kThreads;
      if (i < n4) { va[u] = ld4_stream(a + 4 * i); vd[u] = ld4_stream(dy + 4 * i); vx[u] = ld4_stream(dx + 4 * i); }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      size_t i = base + (size_t)u * kThreads;
      if (i < n4) {
        float4 r = make_float4(vx[u].x + g(va[u].x, vd[u].x), vx[u].y + g(va[u].y, vd[u].y),
                               vx[u].z + g(va[u].z, vd[u].z), vx[u].w + g(va[u].w, vd[u].w));
        st4_stream(dx + 4 * i, r);
      }
    }
  }
  if (blockIdx.x == 0) {
    size_t i = 4 * n4 + threadIdx.x;
    if (i < n) dx[i] += g(a[i], dy[i]);
  }
}
template <class G>
__global__ void __launch_bounds__(kThreads) k_unary_bwd_scalar(const float* __restrict__ a, const float* __restrict__ dy,
                                                              float* __restrict__ dx, size_t n, G g) {
  dyb_grid_dep_sync();
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (size_t)gridDim.x * kThreads)
    dx[i] += g(a[i], dy[i]);
}

template <class F>
int unary_fwd(dyb200_ctx* ctx, const dyb200_tensor* xs, int nxs, dyb200_tensor* fx, F f, const char* name) {
  DYB_CHECK_ARG(ctx, nxs == 1, "Failed input count check in %s", name);
  size_t n = t_size(fx);
  DYB_CHECK_ARG(ctx, t_size(&xs[0]) == n, "%s: input and output sizes differ", name);
  if (n == 0) return DYB200_OK;
  if (aligned16(xs[0].v) && aligned16(fx->v)) {
    size_t n4 = n / 4;
    dyb_launch(k_unary_fwd<F>, stream_grid(ctx, n4 ? n4 : 1, kThreads * kUnroll), kThreads, 0, ctx, xs[0].v, fx->v, n4, n, f);
  } else {
    dyb_launch(k_unary_fwd_scalar<F>, stream_grid(ctx, n, kThreads), kThreads, 0, ctx, xs[0].v, fx->v, n, f);
  }
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}
template <class G>
int unary_bwd(dyb200_ctx* ctx, const float* a, const dyb200_tensor* dEdf, unsigned i, dyb200_tensor* dEdxi, G g,
              const char* name) {
  DYB_CHECK_ARG(ctx, i == 0, "%s::backward: argument index %u out of range", name, i);
  size_t n = t_size(dEdxi);
  DYB_CHECK_ARG(ctx, t_size(dEdf) == n, "%s::backward: gradient sizes differ", name);
  if (n == 0) return DYB200_OK;
  if (aligned16(a) && aligned16(dEdf->v) && aligned16(dEdxi->v)) {
    size_t n4 = n / 4;
    dyb_launch(k_unary_bwd<G>, stream_grid(ctx, n4 ? n4 : 1, kThreads * kUnroll), kThreads, 0, ctx, a, dEdf->v, dEdxi->v, n4, n, g);
  } else {
    dyb_launch(k_unary_bwd_scalar<G>, stream_grid(ctx, n, kThreads), kThreads, 0, ctx, a, dEdf->v, dEdxi->v, n, g);
  }
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

// ------------------------------------------------------------ cwise binary
enum { OP_MUL = 0, OP_SUM = 1, OP_DIV = 2 };
template <int OP> __device__ __forceinline__ float bin_fwd(float a, float b) {
  return OP == OP_MUL ? a * b : (OP == OP_SUM ? a + b : a / b);
}
// gradient contribution to argument i given (a, b, d)
template <int OP> __device__ __forceinline__ float bin_bwd(float a, float b, float d, unsigned i) {
  if (OP == OP_MUL) return d * (i == 0 ? b : a);
  if (OP == OP_SUM) return d;
  return i == 0 ? d / b : -(d / (b * b) * a);
}

struct Shape5 {
  uint32_t s[5];
};
__host__ __device__ inline size_t shape5_size(const Shape5& s) {
  return (size_t)s.s[0] * s.s[1] * s.s[2] * s.s[3] * s.s[4];
}

// Fast path: both arguments have the same non-batch dims; `a` has the full batch,
// `b` has nb elements and is either full (period == total) or batch-1 (period == n).
template <int OP, bool SWAP>
__global__ void __launch_bounds__(kThreads) k_bin_fwd_vec(const float* __restrict__ a, const float* __restrict__ b,
                                                         float* __restrict__ y, size_t n4, size_t period4) {
  dyb_grid_dep_sync();
  const size_t stride = (size_t)gridDim.x * kThreads * kUnroll;
  for (size_t base = (size_t)blockIdx.x * kThreads * kUnroll + threadIdx.x; base < n4; base += stride) {
    float4 va[kUnroll], vb[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      size_t i = base + (size_t)u * kThreads;
      if (i < n4) { va[u] = ld4_stream(a + 4 * i); vb[u] = ld4(b + 4 * (i % period4)); }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      size_t i = base + (size_t)u * kThreads;
      if (i < n4) {
        float4 r;
        if (SWAP) r = make_float4(bin_fwd<OP>(vb[u].x, va[u].x), bin_fwd<OP>(vb[u].y, va[u].y), bin_fwd<OP>(vb[u].z, va[u].z), bin_fwd<OP>(vb[u].w, va[u].w));
        else r = make_float4(bin_fwd<OP>(va[u].x, vb[u].x), bin_fwd<OP>(va[u].y, vb[u].y), bin_fwd<OP>(va[u].z, vb[u].z), bin_fwd<OP>(va[u].w, vb[u].w));
        st4_stream(y + 4 * i, r);
      }
    }
  }
}

__device__ __forceinline__ size_t bidx(size_t lin, const Shape5& o, const Shape5& s) {
  size_t off = 0, stride = 1;
#pragma unroll
  for (int k = 0; k < 5; ++k) {
    uint32_t ik = (uint32_t)(lin % o.s[k]);
    lin /= o.s[k];
    off += (s.s[k] == 1 ? 0 : ik) * stride;
    stride *= s.s[k];
  }
  return off;
}

// Generic broadcast forward: one thread per output element.
template <int OP>
__global__ void __launch_bounds__(kThreads) k_bin_fwd_generic(const float* __restrict__ a, Shape5 sa,
                                                             const float* __restrict__ b, Shape5 sb,
                                                             float* __restrict__ y, Shape5 so, size_t total) {
  dyb_grid_dep_sync();
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < total; e += (size_t)gridDim.x * kThreads)
    y[e] = bin_fwd<OP>(a[bidx(e, so, sa)], b[bidx(e, so, sb)]);
}

// Backward, no reduction needed (argument i has the output's shape); the other
// argument may still be broadcast.
template <int OP>
__global__ void __launch_bounds__(kThreads) k_bin_bwd_noreduce(const float* __restrict__ a, Shape5 sa,
                                                              const float* __restrict__ b, Shape5 sb,
                                                              const float* __restrict__ dy, Shape5 so, size_t total,
                                                              unsigned i, float* __restrict__ dxi) {
  dyb_grid_dep_sync();
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < total; e += (size_t)gridDim.x * kThreads)
    dxi[e] += bin_bwd<OP>(a[bidx(e, so, sa)], b[bidx(e, so, sb)], dy[e], i);
}

// Backward fast path: equal non-batch dims, argument i has the full batch; a and
// b are read with their own periods (full tensor or one batch element).
template <int OP>
__global__ void __launch_bounds__(kThreads) k_bin_bwd_vec(const float* __restrict__ a, size_t pa4,
                                                         const float* __restrict__ b, size_t pb4,
                                                         const float* __restrict__ dy, size_t n4, unsigned i,
                                                         float* __restrict__ dxi) {
  dyb_grid_dep_sync();
  const size_t stride = (size_t)gridDim.x * kThreads * kUnroll;
  for (size_t base = (size_t)blockIdx.x * kThreads * kUnroll + threadIdx.x; base < n4; base += stride) {
    float4 va[kUnroll], vb[kUnroll], vd[kUnroll], vx[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      size_t e = base + (size_t)u * kThreads;
      if (e < n4) {
        if (OP != OP_SUM) { va[u] = ld4(a + 4 * (e % pa4)); vb[u] = ld4(b + 4 * (e % pb4)); }
        else { va[u] = make_float4(0, 0, 0, 0); vb[u] = va[u]; }
        vd[u] = ld4_stream(dy + 4 * e);
        vx[u] = ld4_stream(dxi + 4 * e);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      size_t e = base + (size_t)u * kThreads;
      if (e < n4) {
        float4 r = make_float4(vx[u].x + bin_bwd<OP>(va[u].x, vb[u].x, vd[u].x, i), vx[u].y + bin_bwd<OP>(va[u].y, vb[u].y, vd[u].y, i),
                               vx[u].z + bin_bwd<OP>(va[u].z, vb[u].z, vd[u].z, i), vx[u].w + bin_bwd<OP>(va[u].w, vb[u].w, vd[u].w, i));
        st4_stream(dxi + 4 * e, r);
      }
    }
  }
}

// Backward with reduction over the broadcast axes of argument i: one thread per
// element of dxi, summing the output elements that map to it in ascending linear
// order (what a sequential Eigen reduction does).
template <int OP>
__global__ void __launch_bounds__(kThreads) k_bin_bwd_reduce(const float* __restrict__ a, Shape5 sa,
                                                            const float* __restrict__ b, Shape5 sb,
                                                            const float* __restrict__ dy, Shape5 so, unsigned i,
                                                            float* __restrict__ dxi, size_t ni) {
  dyb_grid_dep_sync();
  const Shape5& si = i == 0 ? sa : sb;
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < ni; e += (size_t)gridDim.x * kThreads) {
    // unravel e in the shape of argument i
    uint32_t idx[5], red[5];
    size_t t = e, nred = 1;
#pragma unroll
    for (int k = 0; k < 5; ++k) {
      idx[k] = (uint32_t)(t % si.s[k]);
      t /= si.s[k];
      red[k] = (si.s[k] == 1 && so.s[k] > 1) ? so.s[k] : 1;
      nred *= red[k];
    }
    float acc = 0.f;
    for (size_t r = 0; r < nred; ++r) {
      size_t rr = r, lin = 0, stride = 1, offa = 0, offb = 0, stra = 1, strb = 1;
#pragma unroll
      for (int k = 0; k < 5; ++k) {
        uint32_t ik = idx[k];
        if (red[k] > 1) { ik = (uint32_t)(rr % red[k]); rr /= red[k]; }
        lin += ik * stride; stride *= so.s[k];
        offa += (sa.s[k] == 1 ? 0 : ik) * stra; stra *= sa.s[k];
        offb += (sb.s[k] == 1 ? 0 : ik) * strb; strb *= sb.s[k];
      }
      acc += bin_bwd<OP>(a[offa], b[offb], dy[lin], i);
    }
    dxi[e] += acc;
  }
}

// f(r, b) for the batch-reduction fast path (same dims, argument i has batch 1).
template <int OP>
struct BatchBwd {
  const float *a, *b, *dy;
  size_t n;
  unsigned i;
  uint32_t bda, bdb;
  __device__ float operator()(size_t r, uint32_t bt) const {
    float av = a[(bda == 1 ? 0 : (size_t)bt * n) + r], bv = b[(bdb == 1 ? 0 : (size_t)bt * n) + r];
    return bin_bwd<OP>(av, bv, dy[(size_t)bt * n + r], i);
  }
};

void to_shape5(const dyb200_tensor* t, Shape5* s) {
  for (int k = 0; k < 4; ++k) s->s[k] = t_dim(t, k);
  s->s[4] = t->bd;
}

template <int OP>
int binary_check(dyb200_ctx* ctx, const dyb200_tensor* xs, int nxs, const char* name, Shape5* sa, Shape5* sb,
                 Shape5* so) {
  DYB_CHECK_ARG(ctx, nxs == 2, "Failed input count check in %s", name);
  DYB_CHECK_ARG(ctx, xs[0].nd <= 4 && xs[1].nd <= 4, "%s: more than 4 dimensions are not supported", name);
  to_shape5(&xs[0], sa);
  to_shape5(&xs[1], sb);
  for (int k = 0; k < 5; ++k) {
    uint32_t x = sa->s[k], y = sb->s[k];
    bool ok = OP == OP_DIV ? (x == y || y == 1) : (x == y || x == 1 || y == 1);
    DYB_CHECK_ARG(ctx, ok, "%s: For each dimension, the dim size needs to match or equal 1 (dim %d: %u vs %u)", name, k, x, y);
    so->s[k] = x > y ? x : y;
  }
  return DYB200_OK;
}

template <int OP>
int binary_fwd(dyb200_ctx* ctx, const dyb200_tensor* xs, int nxs, dyb200_tensor* fx, const char* name) {
  Shape5 sa, sb, so;
  int rc = binary_check<OP>(ctx, xs, nxs, name, &sa, &sb, &so);
  if (rc) return rc;
  size_t total = shape5_size(so);
  DYB_CHECK_ARG(ctx, t_size(fx) == total, "%s: output size %zu does not match broadcast size %zu", name, t_size(fx), total);
  if (total == 0) return DYB200_OK;
  bool same_dims = true;
  for (int k = 0; k < 4; ++k) same_dims = same_dims && sa.s[k] == sb.s[k];
  size_t n = (size_t)so.s[0] * so.s[1] * so.s[2] * so.s[3];
  bool vec_ok = same_dims && (n % 4 == 0) && aligned16(xs[0].v) && aligned16(xs[1].v) && aligned16(fx->v);
  if (vec_ok) {
    size_t n4 = total / 4;
    unsigned grid = stream_grid(ctx, n4, kThreads * kUnroll);
    if (sa.s[4] >= sb.s[4]) {
      size_t period4 = (sb.s[4] == so.s[4] ? total : n) / 4;
      dyb_launch(k_bin_fwd_vec<OP, false>, grid, kThreads, 0, ctx, xs[0].v, xs[1].v, fx->v, n4, period4);
    } else {
      dyb_launch(k_bin_fwd_vec<OP, true>, grid, kThreads, 0, ctx, xs[1].v, xs[0].v, fx->v, n4, n / 4);
    }
  } else {
    dyb_launch(k_bin_fwd_generic<OP>, stream_grid(ctx, total, kThreads), kThreads, 0, ctx, xs[0].v, sa, xs[1].v, sb, fx->v, so, total);
  }
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

template <int OP>
int binary_bwd(dyb200_ctx* ctx, const dyb200_tensor* xs, int nxs, const dyb200_tensor* dEdf, unsigned i,
               dyb200_tensor* dEdxi, const char* name) {
  Shape5 sa, sb, so;
  int rc = binary_check<OP>(ctx, xs, nxs, name, &sa, &sb, &so);
  if (rc) return rc;
  DYB_CHECK_ARG(ctx, i < 2, "Failed dimension check in %s::backward", name);
  const Shape5& si = i == 0 ? sa : sb;
  size_t total = shape5_size(so), ni = shape5_size(si);
  DYB_CHECK_ARG(ctx, t_size(dEdf) == total && t_size(dEdxi) == ni, "%s::backward: gradient sizes do not match", name);
  if (total == 0) return DYB200_OK;
  bool same_dims = true, need_reduce = false;
  for (int k = 0; k < 4; ++k) same_dims = same_dims && sa.s[k] == sb.s[k];
  for (int k = 0; k < 5; ++k) need_reduce = need_reduce || si.s[k] != so.s[k];
  size_t n = (size_t)so.s[0] * so.s[1] * so.s[2] * so.s[3];
  if (!need_reduce && same_dims && n % 4 == 0 && aligned16(xs[0].v) && aligned16(xs[1].v) && aligned16(dEdf->v) &&
      aligned16(dEdxi->v)) {
    size_t n4 = total / 4;
    size_t pa4 = (sa.s[4] == so.s[4] ? total : n) / 4, pb4 = (sb.s[4] == so.s[4] ? total : n) / 4;
    dyb_launch(k_bin_bwd_vec<OP>, stream_grid(ctx, n4, kThreads * kUnroll), kThreads, 0, ctx, xs[0].v, pa4, xs[1].v, pb4, dEdf->v, n4, i, dEdxi->v);
    DYB_LAUNCHED(ctx);
    return DYB200_OK;
  }
  if (!need_reduce) {
    dyb_launch(k_bin_bwd_noreduce<OP>, stream_grid(ctx, total, kThreads), kThreads, 0, ctx, xs[0].v, sa, xs[1].v, sb, dEdf->v, so, total, i, dEdxi->v);
    DYB_LAUNCHED(ctx);
    return DYB200_OK;
  }
  if (same_dims) {  // only the batch is reduced
    BatchBwd<OP> f{xs[0].v, xs[1].v, dEdf->v, n, i, sa.s[4], sb.s[4]};
    return batch_reduce_add(ctx, f, n, so.s[4], dEdxi->v);
  }
  dyb_launch(k_bin_bwd_reduce<OP>, stream_grid(ctx, ni, kThreads), kThreads, 0, ctx, xs[0].v, sa, xs[1].v, sb, dEdf->v, so, i, dEdxi->v, ni);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

}  // namespace

extern "C" {

int dyb200_tanh_fwd(DYB200_FWD_ARGS) { (void)attrs; (void)aux_mem; return unary_fwd(ctx, xs, nxs, fx, FTanh{}, "Tanh"); }
int dyb200_tanh_bwd(DYB200_BWD_ARGS) { (void)xs; (void)nxs; (void)attrs; (void)aux_mem; return unary_bwd(ctx, fx->v, dEdf, i, dEdxi, BTanh{}, "Tanh"); }
int dyb200_logistic_fwd(DYB200_FWD_ARGS) { (void)attrs; (void)aux_mem; return unary_fwd(ctx, xs, nxs, fx, FLogistic{}, "LogisticSigmoid"); }
int dyb200_logistic_bwd(DYB200_BWD_ARGS) { (void)xs; (void)nxs; (void)attrs; (void)aux_mem; return unary_bwd(ctx, fx->v, dEdf, i, dEdxi, BLogistic{}, "LogisticSigmoid"); }
int dyb200_rectify_fwd(DYB200_FWD_ARGS) { (void)attrs; (void)aux_mem; return unary_fwd(ctx, xs, nxs, fx, FRectify{}, "Rectify"); }
int dyb200_rectify_bwd(DYB200_BWD_ARGS) { (void)xs; (void)nxs; (void)attrs; (void)aux_mem; return unary_bwd(ctx, fx->v, dEdf, i, dEdxi, BRectify{}, "Rectify"); }
// Negate, ConstantPlusX, ConstantMinusX: the backward pass needs no saved value (dEdf stands in for it)
int dyb200_negate_fwd(DYB200_FWD_ARGS) { (void)attrs; (void)aux_mem; return unary_fwd(ctx, xs, nxs, fx, FNegate{}, "Negate"); }
int dyb200_negate_bwd(DYB200_BWD_ARGS) { (void)xs; (void)nxs; (void)fx; (void)attrs; (void)aux_mem; return unary_bwd(ctx, dEdf->v, dEdf, i, dEdxi, BNeg{}, "Negate"); }
int dyb200_constant_plus_x_fwd(DYB200_FWD_ARGS) {
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, attrs != nullptr, "ConstantPlusX: attrs (c) required");
  return unary_fwd(ctx, xs, nxs, fx, FConstPlus{((const dyb200_const_attrs*)attrs)->c}, "ConstantPlusX");
}
int dyb200_constant_plus_x_bwd(DYB200_BWD_ARGS) { (void)xs; (void)nxs; (void)fx; (void)attrs; (void)aux_mem; return unary_bwd(ctx, dEdf->v, dEdf, i, dEdxi, BPass{}, "ConstantPlusX"); }
int dyb200_constant_minus_x_fwd(DYB200_FWD_ARGS) {
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, attrs != nullptr, "ConstantMinusX: attrs (c) required");
  return unary_fwd(ctx, xs, nxs, fx, FConstMinus{((const dyb200_const_attrs*)attrs)->c}, "ConstantMinusX");
}
int dyb200_constant_minus_x_bwd(DYB200_BWD_ARGS) { (void)xs; (void)nxs; (void)fx; (void)attrs; (void)aux_mem; return unary_bwd(ctx, dEdf->v, dEdf, i, dEdxi, BNeg{}, "ConstantMinusX"); }
int dyb200_elu_fwd(DYB200_FWD_ARGS) {
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, attrs != nullptr, "ExponentialLinearUnit: attrs (alpha, lambda) required");
  const dyb200_elu_attrs* a = (const dyb200_elu_attrs*)attrs;
  return unary_fwd(ctx, xs, nxs, fx, FElu{a->alpha, a->lambda}, "ExponentialLinearUnit");
}
int dyb200_elu_bwd(DYB200_BWD_ARGS) {
  (void)fx; (void)aux_mem;
  DYB_CHECK_ARG(ctx, attrs != nullptr && nxs == 1, "ExponentialLinearUnit: attrs (alpha, lambda) and one input required");
  const dyb200_elu_attrs* a = (const dyb200_elu_attrs*)attrs;
  return unary_bwd(ctx, xs[0].v, dEdf, i, dEdxi, BElu{a->alpha, a->lambda}, "ExponentialLinearUnit");
}

int dyb200_cmult_fwd(DYB200_FWD_ARGS) { (void)attrs; (void)aux_mem; return binary_fwd<OP_MUL>(ctx, xs, nxs, fx, "CwiseMultiply"); }
int dyb200_cmult_bwd(DYB200_BWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; } (void)fx; (void)attrs; (void)aux_mem; return binary_bwd<OP_MUL>(ctx, xs, nxs, dEdf, i, dEdxi, "CwiseMultiply"); }
int dyb200_csum_fwd(DYB200_FWD_ARGS) { (void)attrs; (void)aux_mem; return binary_fwd<OP_SUM>(ctx, xs, nxs, fx, "CwiseSum"); }
int dyb200_csum_bwd(DYB200_BWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; } (void)fx; (void)attrs; (void)aux_mem; return binary_bwd<OP_SUM>(ctx, xs, nxs, dEdf, i, dEdxi, "CwiseSum"); }
int dyb200_cdiv_fwd(DYB200_FWD_ARGS) { (void)attrs; (void)aux_mem; return binary_fwd<OP_DIV>(ctx, xs, nxs, fx, "CwiseQuotient"); }
int dyb200_cdiv_bwd(DYB200_BWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; } (void)fx; (void)attrs; (void)aux_mem; return binary_bwd<OP_DIV>(ctx, xs, nxs, dEdf, i, dEdxi, "CwiseQuotient"); }

}  // extern "C"
