// Glue nodes the LSTM graphs execute between the fused kernels:
//   PickRange        dynet/nodes-select.cc:229-259
//   Concatenate      dynet/nodes-concat.cc:51-90
//   Sum (n-ary)      dynet/nodes-arith-sum.cc:66-137
//   SumDimension     dynet/nodes-arith-sum.cc:198-248   (sum_dim, sum_batches)
//   SquaredNorm      dynet/nodes-norms.cc:30-46
//   RandomBernoulli  dynet/nodes-random.cc:100-104, dynet/tensor.cc:261-275
// A slice along dimension k of a column-major tensor is `outer` runs of `inner * len` contiguous floats
// (inner = product of the dimensions below k, outer = product of those above it times the batch size), so
// PickRange and Concatenate are one strided 2-D copy / accumulate each.
#include "common.cuh"
#include "reduce.cuh"

namespace {

constexpr int kThreads = 256;

// dst[r * dst_pitch + c] (+)= src[(r % src_rows) * src_pitch + c] for r < rows, c < row_len
template <int ADD>
__global__ void __launch_bounds__(kThreads) k_copy2d(const float* __restrict__ src, size_t src_pitch, size_t src_rows,
                                                     float* __restrict__ dst, size_t dst_pitch, size_t row_len, size_t rows, int vec) {
  dyb_grid_dep_sync();
  if (vec) {
    const size_t len4 = row_len / 4, total = len4 * rows;
    for (size_t q = (size_t)blockIdx.x * kThreads + threadIdx.x; q < total; q += (size_t)gridDim.x * kThreads) {
      const size_t r = q / len4, c = 4 * (q % len4);
      float4 v = ld4(src + (r % src_rows) * src_pitch + c);
      float* d = dst + r * dst_pitch + c;
      if (ADD) { float4 o = ld4(d); v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
      st4(d, v);
    }
    return;
  }
  const size_t total = row_len * rows;
  for (size_t q = (size_t)blockIdx.x * kThreads + threadIdx.x; q < total; q += (size_t)gridDim.x * kThreads) {
    const size_t r = q / row_len, c = q % row_len;
    const float v = src[(r % src_rows) * src_pitch + c];
    float* d = dst + r * dst_pitch + c;
    if (ADD) *d += v; else *d = v;
  }
}

int copy2d(dyb200_ctx* ctx, const float* src, size_t src_pitch, size_t src_rows, float* dst, size_t dst_pitch, size_t row_len,
           size_t rows, bool add) {
  if (row_len == 0 || rows == 0) return DYB200_OK;
  const int vec = row_len % 4 == 0 && src_pitch % 4 == 0 && dst_pitch % 4 == 0 && aligned16(src) && aligned16(dst);
  const unsigned grid = stream_grid(ctx, row_len * rows / (vec ? 4 : 1) + 1, kThreads);
  if (add) dyb_launch(k_copy2d<1>, grid, kThreads, 0, ctx, src, src_pitch, src_rows, dst, dst_pitch, row_len, rows, vec);
  else dyb_launch(k_copy2d<0>, grid, kThreads, 0, ctx, src, src_pitch, src_rows, dst, dst_pitch, row_len, rows, vec);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

// (inner, len, outer-without-batch) of dimension k of a tensor
struct Split { size_t inner, len, higher; };
Split split_at(const dyb200_tensor* t, unsigned k) {
  Split s{1, t_dim(t, k), 1};
  for (unsigned q = 0; q < k; ++q) s.inner *= t_dim(t, q);
  for (unsigned q = k + 1; q < t->nd; ++q) s.higher *= t->d[q];
  return s;
}

// f(r, b) = element r of the slice of batch element b (slice rows of `row_len` floats, `higher` rows per batch element)
struct SliceOf {
  const float* v; size_t pitch, row_len, higher;
  __device__ float operator()(size_t r, uint32_t b) const { return v[((size_t)b * higher + r / row_len) * pitch + r % row_len]; }
};
struct BatchOf {   // f(r, b) = v[r + n * b]
  const float* v; size_t n;
  __device__ float operator()(size_t r, uint32_t b) const { return v[r + n * (size_t)b]; }
};

// fx = x0 + x1 + x2 + x3 (left to right), or fx += (x0 + x1 + x2 + x3); absent operands are null.
// An operand with one batch element under a batched result is read modulo its size.
struct SumArgs { const float* x[4]; size_t size[4]; int n; };
template <int ACC>
__global__ void __launch_bounds__(kThreads) k_sum_group(const SumArgs a, float* __restrict__ fx, size_t n) {
  dyb_grid_dep_sync();
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < n; e += (size_t)gridDim.x * kThreads) {
    float s = a.x[0][e % a.size[0]];
    for (int k = 1; k < a.n; ++k) s += a.x[k][e % a.size[k]];
    fx[e] = ACC ? fx[e] + s : s;
  }
}

// Generic SumDimension: x as [d0, d1, d2, bd]; one thread per output element, reduced dimensions in ascending order
// (lower dimension innermost), batch outermost.
struct Dims4 { uint32_t d[4]; uint32_t red[4]; };
__global__ void __launch_bounds__(kThreads) k_sum_dims(const float* __restrict__ x, float* __restrict__ y, const Dims4 s, size_t n_out) {
  dyb_grid_dep_sync();
  for (size_t o = (size_t)blockIdx.x * kThreads + threadIdx.x; o < n_out; o += (size_t)gridDim.x * kThreads) {
    uint32_t idx[4]; size_t rem = o;
    for (int k = 0; k < 4; ++k) {
      if (s.red[k]) idx[k] = 0;
      else { idx[k] = (uint32_t)(rem % s.d[k]); rem /= s.d[k]; }
    }
    const uint32_t n0 = s.red[0] ? s.d[0] : 1, n1 = s.red[1] ? s.d[1] : 1, n2 = s.red[2] ? s.d[2] : 1, n3 = s.red[3] ? s.d[3] : 1;
    float acc = 0.f;
    for (uint32_t i3 = 0; i3 < n3; ++i3)
      for (uint32_t i2 = 0; i2 < n2; ++i2)
        for (uint32_t i1 = 0; i1 < n1; ++i1)
          for (uint32_t i0 = 0; i0 < n0; ++i0) {
            const size_t e = (idx[0] + i0) + (size_t)s.d[0] * ((idx[1] + i1) + (size_t)s.d[1] * ((idx[2] + i2) + (size_t)s.d[2] * (idx[3] + i3)));
            acc += x[e];
          }
    y[o] = acc;
  }
}
// dEdxi[e] += dEdf[index of e with the reduced coordinates dropped]
__global__ void __launch_bounds__(kThreads) k_sum_dims_bwd(const float* __restrict__ dy, float* __restrict__ dx, const Dims4 s, size_t n_in) {
  dyb_grid_dep_sync();
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < n_in; e += (size_t)gridDim.x * kThreads) {
    size_t rem = e, o = 0, mul = 1;
    for (int k = 0; k < 4; ++k) {
      const uint32_t c = (uint32_t)(rem % s.d[k]); rem /= s.d[k];
      if (!s.red[k]) { o += mul * c; mul *= s.d[k]; }
    }
    dx[e] += dy[o];
  }
}
// Sum over dimension 0 (contiguous): one warp per output element.
__global__ void __launch_bounds__(kThreads) k_sum_dim0(const float* __restrict__ x, float* __restrict__ y, uint32_t d0, size_t n_out) {
  dyb_grid_dep_sync();
  const size_t warp = ((size_t)blockIdx.x * kThreads + threadIdx.x) >> 5, nw = ((size_t)gridDim.x * kThreads) >> 5;
  const int lane = threadIdx.x & 31;
  for (size_t o = warp; o < n_out; o += nw) {
    const float* c = x + o * d0;
    float acc = 0.f;
    for (uint32_t i = lane; i < d0; i += 32) acc += c[i];
    acc = warp_sum(acc);
    if (lane == 0) y[o] = acc;
  }
}

// y[b] = sum_i x[i, b]^2 : one CTA per batch element
__global__ void __launch_bounds__(kThreads) k_squared_norm(const float* __restrict__ x, float* __restrict__ y, size_t n) {
  dyb_grid_dep_sync();
  __shared__ float red[32];
  const float* c = x + (size_t)blockIdx.x * n;
  float acc = 0.f;
  if (n % 4 == 0 && aligned16(c)) {
    for (size_t i = threadIdx.x; i < n / 4; i += kThreads) { float4 v = ld4(c + 4 * i); acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
  } else {
    for (size_t i = threadIdx.x; i < n; i += kThreads) acc += c[i] * c[i];
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) y[blockIdx.x] = acc;
}
__global__ void __launch_bounds__(kThreads) k_squared_norm_bwd(const float* __restrict__ x, const float* __restrict__ dy,
                                                               float* __restrict__ dx, size_t n, size_t total) {
  dyb_grid_dep_sync();
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < total; e += (size_t)gridDim.x * kThreads)
    dx[e] += x[e] * dy[e / n] * 2.0f;
}

// Philox-4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"): counter = element index / 4,
// key = seed; four 32-bit words per counter.
__device__ __forceinline__ void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t lo0 = 0xD2511F53u * c[0], hi0 = __umulhi(0xD2511F53u, c[0]);
    const uint32_t lo1 = 0xCD9E8D57u * c[2], hi1 = __umulhi(0xCD9E8D57u, c[2]);
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
}
// y[e] = (u_e < p) ? scale : 0, u_e uniform in [0, 1) from 24 random bits
__global__ void __launch_bounds__(kThreads) k_bernoulli(float* __restrict__ y, size_t n, float p, float scale, uint64_t seed, uint64_t offset) {
  dyb_grid_dep_sync();
  const size_t n4 = (n + 3) / 4;
  const bool vec = aligned16(y);
  for (size_t q = (size_t)blockIdx.x * kThreads + threadIdx.x; q < n4; q += (size_t)gridDim.x * kThreads) {
    const uint64_t ctr = offset + q;
    uint32_t c[4] = {(uint32_t)ctr, (uint32_t)(ctr >> 32), 0u, 0u};
    philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = ((float)(c[k] >> 8) * (1.0f / 16777216.0f) < p) ? scale : 0.f;
    if (vec && 4 * q + 3 < n) st4_stream(y + 4 * q, make_float4(v[0], v[1], v[2], v[3]));
    else {
#pragma unroll
      for (int k = 0; k < 4; ++k) if (4 * q + k < n) y[4 * q + k] = v[k];
    }
  }
}

}  // namespace

extern "C" {

int dyb200_pick_range_fwd(DYB200_FWD_ARGS) {
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 1 && attrs && fx && fx->v && xs[0].v, "PickRange: one input and attrs (start, end, dim) required");
  const dyb200_pick_range_attrs* a = (const dyb200_pick_range_attrs*)attrs;
  DYB_CHECK_ARG(ctx, a->dim < 4 && a->start < a->end && a->end <= t_dim(&xs[0], a->dim),
                "PickRange: bad range [%u, %u) on dimension %u of size %u", a->start, a->end, a->dim, t_dim(&xs[0], a->dim));
  const Split s = split_at(&xs[0], a->dim);
  const size_t len = a->end - a->start, rows = s.higher * xs[0].bd;
  DYB_CHECK_ARG(ctx, t_size(fx) == s.inner * len * rows, "PickRange: output size mismatch");
  return copy2d(ctx, xs[0].v + a->start * s.inner, s.inner * s.len, rows, fx->v, s.inner * len, s.inner * len, rows, false);
}

int dyb200_pick_range_bwd(DYB200_BWD_ARGS) {
  (void)aux_mem; (void)fx;
  DYB_CHECK_ARG(ctx, nxs == 1 && i == 0 && attrs && dEdf && dEdf->v && dEdxi && dEdxi->v, "PickRange: bad backward arguments");
  const dyb200_pick_range_attrs* a = (const dyb200_pick_range_attrs*)attrs;
  DYB_CHECK_ARG(ctx, a->dim < 4 && a->start < a->end && a->end <= t_dim(dEdxi, a->dim), "PickRange: bad range");
  const Split s = split_at(dEdxi, a->dim);
  const size_t len = a->end - a->start, rows = s.higher * dEdxi->bd;
  DYB_CHECK_ARG(ctx, t_size(dEdf) == s.inner * len * rows, "PickRange: gradient size mismatch");
  return copy2d(ctx, dEdf->v, s.inner * len, rows, dEdxi->v + a->start * s.inner, s.inner * s.len, s.inner * len, rows, true);
}

int dyb200_concatenate_fwd(DYB200_FWD_ARGS) {
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs >= 1 && attrs && fx && fx->v, "Concatenate: inputs and attrs (dimension) required");
  const unsigned k = ((const dyb200_dim_attrs*)attrs)->dimension;
  DYB_CHECK_ARG(ctx, k < 4, "Concatenate: dimension %u out of range", k);
  const Split sf = split_at(fx, k);
  size_t curr = 0;
  for (int q = 0; q < nxs; ++q) {
    const Split sx = split_at(&xs[q], k);
    DYB_CHECK_ARG(ctx, xs[q].v && sx.inner == sf.inner && sx.higher == sf.higher && (xs[q].bd == fx->bd || xs[q].bd == 1),
                  "Concatenate: bad input dimensions (argument %d)", q);
    int rc = copy2d(ctx, xs[q].v, sx.inner * sx.len, sx.higher * xs[q].bd, fx->v + curr * sf.inner, sf.inner * sf.len, sx.inner * sx.len,
                    sf.higher * fx->bd, false);
    if (rc) return rc;
    curr += sx.len;
  }
  DYB_CHECK_ARG(ctx, curr == sf.len, "Concatenate: inputs cover %zu of %zu rows", curr, sf.len);
  return DYB200_OK;
}

int dyb200_concatenate_bwd(DYB200_BWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)aux_mem; (void)fx;
  DYB_CHECK_ARG(ctx, attrs && (int)i < nxs && dEdf && dEdf->v && dEdxi && dEdxi->v, "Concatenate: bad backward arguments");
  const unsigned k = ((const dyb200_dim_attrs*)attrs)->dimension;
  DYB_CHECK_ARG(ctx, k < 4, "Concatenate: dimension %u out of range", k);
  const Split sf = split_at(dEdf, k);
  size_t off = 0;
  for (unsigned q = 0; q < i; ++q) off += t_dim(&xs[q], k);
  const Split sx = split_at(dEdxi, k);
  DYB_CHECK_ARG(ctx, sx.inner == sf.inner && sx.higher == sf.higher && off + sx.len <= sf.len, "Concatenate: gradient shape mismatch");
  const size_t row_len = sx.inner * sx.len;
  if (dEdxi->bd == dEdf->bd)
    return copy2d(ctx, dEdf->v + off * sf.inner, sf.inner * sf.len, sf.higher * dEdf->bd, dEdxi->v, row_len, row_len, sx.higher * dEdxi->bd, true);
  DYB_CHECK_ARG(ctx, dEdxi->bd == 1, "Concatenate: mismatched batch sizes");
  return batch_reduce_add(ctx, SliceOf{dEdf->v + off * sf.inner, sf.inner * sf.len, row_len, sf.higher}, row_len * sx.higher, dEdf->bd, dEdxi->v);
}

int dyb200_sum_fwd(DYB200_FWD_ARGS) {
  (void)aux_mem; (void)attrs;
  DYB_CHECK_ARG(ctx, nxs >= 1 && fx && fx->v, "Sum: at least one input required");
  const size_t n = t_size(fx);
  bool same = true;
  for (int q = 0; q < nxs; ++q) {
    DYB_CHECK_ARG(ctx, xs[q].v && t_batch_size(&xs[q]) == t_batch_size(fx) && (xs[q].bd == fx->bd || xs[q].bd == 1), "Sum: mismatched input dimensions (argument %d)", q);
    same = same && xs[q].bd == xs[0].bd;
  }
  if (n == 0) return DYB200_OK;
  const unsigned grid = stream_grid(ctx, n, kThreads);
  auto group = [&](int first, int count, bool acc) -> int {
    SumArgs a; a.n = count;
    for (int k = 0; k < 4; ++k) { a.x[k] = k < count ? xs[first + k].v : nullptr; a.size[k] = k < count ? t_size(&xs[first + k]) : 1; }
    if (acc) dyb_launch(k_sum_group<1>, grid, kThreads, 0, ctx, a, fx->v, n);
    else dyb_launch(k_sum_group<0>, grid, kThreads, 0, ctx, a, fx->v, n);
    DYB_LAUNCHED(ctx);
    return DYB200_OK;
  };
  int rc;
  if (same) {
    // the reference's unrolling: the first (up to) four, then the remainder of (n - 4) % 4, then groups of four
    const int head = nxs < 4 ? nxs : 4;
    if ((rc = group(0, head, false))) return rc;
    if (nxs <= 4) return DYB200_OK;
    const int rem = (nxs - 4) % 4;
    if (rem && (rc = group(4, rem, true))) return rc;
    for (int q = 4 + rem; q < nxs; q += 4) if ((rc = group(q, 4, true))) return rc;
    return DYB200_OK;
  }
  // mixed batch sizes: zero, then one accumulation per argument (batch-1 arguments broadcast)
  DYB_CUDA(ctx, cudaMemsetAsync(fx->v, 0, n * sizeof(float), ctx->stream));
  for (int q = 0; q < nxs; ++q) if ((rc = group(q, 1, true))) return rc;
  return DYB200_OK;
}

int dyb200_sum_bwd(DYB200_BWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)aux_mem; (void)attrs; (void)fx;
  DYB_CHECK_ARG(ctx, (int)i < nxs && dEdf && dEdf->v && dEdxi && dEdxi->v && t_batch_size(dEdxi) == t_batch_size(dEdf), "Sum: bad backward arguments");
  const size_t n = t_batch_size(dEdxi);
  if (dEdxi->bd == dEdf->bd) return copy2d(ctx, dEdf->v, n * dEdf->bd, 1, dEdxi->v, n * dEdf->bd, n * dEdf->bd, 1, true);
  DYB_CHECK_ARG(ctx, dEdxi->bd == 1, "Sum: mismatched batch sizes");
  return batch_reduce_add(ctx, BatchOf{dEdf->v, n}, n, dEdf->bd, dEdxi->v);
}

static int sum_dim_shape(dyb200_ctx* ctx, const dyb200_tensor* x, const dyb200_sum_dim_attrs* a, Dims4* s, size_t* n_out) {
  DYB_CHECK_ARG(ctx, x->nd <= 3, "SumDimension: input tensor has more than 3 dimensions");
  DYB_CHECK_ARG(ctx, a->ndims <= 2 && (a->ndims > 0 || a->include_batch_dim), "SumDimension: number of dimensions to reduce must be between 1 and 2");
  for (int k = 0; k < 3; ++k) { s->d[k] = t_dim(x, k); s->red[k] = 0; }
  s->d[3] = x->bd; s->red[3] = a->include_batch_dim ? 1 : 0;
  for (unsigned k = 0; k < a->ndims; ++k) {
    DYB_CHECK_ARG(ctx, a->dims[k] < 3, "SumDimension: dimension %u out of range", a->dims[k]);
    s->red[a->dims[k]] = 1;
  }
  *n_out = 1;
  for (int k = 0; k < 4; ++k) if (!s->red[k]) *n_out *= s->d[k];
  return DYB200_OK;
}

int dyb200_sum_dim_fwd(DYB200_FWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 1 && attrs && fx && fx->v && xs[0].v, "SumDimension: one input and attrs required");
  const dyb200_sum_dim_attrs* a = (const dyb200_sum_dim_attrs*)attrs;
  Dims4 s; size_t n_out;
  int rc = sum_dim_shape(ctx, &xs[0], a, &s, &n_out);
  if (rc) return rc;
  DYB_CHECK_ARG(ctx, t_size(fx) == n_out, "SumDimension: output size mismatch");
  if (t_size(&xs[0]) == 0) return DYB200_OK;
  if (a->ndims == 0) {   // sum_batches: deterministic two-stage reduction over the batch axis
    DYB_CUDA(ctx, cudaMemsetAsync(fx->v, 0, n_out * sizeof(float), ctx->stream));
    return batch_reduce_add(ctx, BatchOf{xs[0].v, n_out}, n_out, xs[0].bd, fx->v);
  }
  if (a->ndims == 1 && a->dims[0] == 0 && !a->include_batch_dim && s.d[0] >= 32) {
    dyb_launch(k_sum_dim0, stream_grid(ctx, n_out, kThreads / 32), kThreads, 0, ctx, xs[0].v, fx->v, s.d[0], n_out);
  } else {
    dyb_launch(k_sum_dims, stream_grid(ctx, n_out, kThreads), kThreads, 0, ctx, xs[0].v, fx->v, s, n_out);
  }
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_sum_dim_bwd(DYB200_BWD_ARGS) {
  (void)aux_mem; (void)fx;
  DYB_CHECK_ARG(ctx, nxs == 1 && i == 0 && attrs && dEdf && dEdf->v && dEdxi && dEdxi->v, "SumDimension: bad backward arguments");
  const dyb200_sum_dim_attrs* a = (const dyb200_sum_dim_attrs*)attrs;
  Dims4 s; size_t n_out;
  int rc = sum_dim_shape(ctx, dEdxi, a, &s, &n_out);
  if (rc) return rc;
  DYB_CHECK_ARG(ctx, t_size(dEdf) == n_out, "SumDimension: gradient size mismatch");
  const size_t n_in = t_size(dEdxi);
  if (n_in == 0) return DYB200_OK;
  dyb_launch(k_sum_dims_bwd, stream_grid(ctx, n_in, kThreads), kThreads, 0, ctx, dEdf->v, dEdxi->v, s, n_in);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_squared_norm_fwd(DYB200_FWD_ARGS) {
  (void)aux_mem; (void)attrs;
  DYB_CHECK_ARG(ctx, nxs == 1 && fx && fx->v && xs[0].v && t_size(fx) == xs[0].bd, "SquaredNorm: one input and a {1} x batch output required");
  if (xs[0].bd == 0) return DYB200_OK;
  dyb_launch(k_squared_norm, xs[0].bd, kThreads, 0, ctx, xs[0].v, fx->v, t_batch_size(&xs[0]));
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_squared_norm_bwd(DYB200_BWD_ARGS) {
  (void)aux_mem; (void)attrs; (void)fx;
  DYB_CHECK_ARG(ctx, nxs == 1 && i == 0 && dEdf && dEdf->v && dEdxi && dEdxi->v && t_size(dEdf) == xs[0].bd && t_size(dEdxi) == t_size(&xs[0]),
                "SquaredNorm: bad backward arguments");
  const size_t total = t_size(&xs[0]);
  if (total == 0) return DYB200_OK;
  dyb_launch(k_squared_norm_bwd, stream_grid(ctx, total, kThreads), kThreads, 0, ctx, xs[0].v, dEdf->v, dEdxi->v, t_batch_size(&xs[0]), total);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_random_bernoulli_fwd(DYB200_FWD_ARGS) {
  (void)aux_mem; (void)xs;
  DYB_CHECK_ARG(ctx, nxs == 0 && attrs && fx && fx->v, "RandomBernoulli: no inputs and attrs (p, scale, seed, offset) required");
  const dyb200_bernoulli_attrs* a = (const dyb200_bernoulli_attrs*)attrs;
  DYB_CHECK_ARG(ctx, a->p >= 0.f && a->p <= 1.f, "RandomBernoulli: p = %g is not a probability", (double)a->p);
  const size_t n = t_size(fx);
  if (n == 0) return DYB200_OK;
  dyb_launch(k_bernoulli, stream_grid(ctx, n / 4 + 1, kThreads), kThreads, 0, ctx, fx->v, n, a->p, a->scale, a->seed, a->offset);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

}  // extern "C"
