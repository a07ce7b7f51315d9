/*
 * CPU oracle: a plain-C, single-threaded, float32 restatement of the CPU (Eigen)
 * branches of DyNet's fused-layer nodes.  TEST INFRASTRUCTURE ONLY: it is the
 * checker the CUDA kernels are compared against and the timed CPU baseline; the
 * shipped library never links or calls it.
 *
 * Every function cites the reference file:line whose arithmetic and operation
 * order it follows.  Tensors are column-major float32 with the batch as the
 * slowest axis, exactly like dynet::Tensor (dynet/tensor-eigen.h:21-224).
 *
 * Third-party arithmetic: the reference evaluates tanh/exp/log and GEMM through
 * Eigen (un-vendored, pinned to hg commit b2e267dc99d4, README.md:58-66).  Eigen
 * is absent from the reference tree, so this file uses libm (tanhf/expf/logf)
 * and a straight k-ordered GEMM instead; both agree with Eigen's packet math to
 * a few ulp, far inside the 1e-5 / 1e-4 parity classes.  The logistic sigmoid is
 * the reference's own rational packet formula (dynet/simd-functors.h:81-125).
 * Long reductions (softmax / logsumexp / moment / norm sums) accumulate in double
 * and round once: Eigen reduces packet- and tree-wise, never as one sequential
 * float32 chain, and a sequential float32 sum (error growing with n, ~1e-3 at
 * n = 4M) would be a worse stand-in for it than the correctly rounded sum.
 *
 * Parity pin: checked against the golden values in the reference's own tests
 * (tests/test-rnn.cc:245-400, tests/test-nodes.cc:2383-2435,
 * tests/python/test.py:506-519) by tests/test_oracle_golden.py.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* scalar functors                                                     */
/* ------------------------------------------------------------------ */

/* dynet/simd-functors.h:81-125 (packetOp): clamp to [-18,18], odd/even rational. */
static inline float sigmoid_packet(float xin) {
  float x = fmaxf(fminf(xin, 18.0f), -18.0f);
  const float a1 = 2.48287947061529e-01f, a3 = 8.51377133304701e-03f,
              a5 = 6.08574864600143e-05f, a7 = 1.15627324459942e-07f,
              a9 = 4.37031012579801e-11f;
  const float b0 = 9.93151921023180e-01f, b2 = 1.16817656904453e-01f,
              b4 = 1.70198817374094e-03f, b6 = 6.29106785017040e-06f,
              b8 = 5.76102136993427e-09f, b10 = 6.10247389755681e-13f;
  float x2 = x * x;
  float p = fmaf(x2, a9, a7);
  p = fmaf(x2, p, a5);
  p = fmaf(x2, p, a3);
  p = fmaf(x2, p, a1);
  p = x * p;
  float q = fmaf(x2, b10, b8);
  q = fmaf(x2, q, b6);
  q = fmaf(x2, q, b4);
  q = fmaf(x2, q, b2);
  q = fmaf(x2, q, b0);
  return fmaxf(fminf(p / q + 0.5f, 1.0f), 0.0f);
}
/* dynet/simd-functors.h:76-79 (scalar operator(), used for the array tail). */
static inline float sigmoid_scalar(float x) { return 1.0f / (1.0f + expf(-x)); }

/* Eigen evaluates full packets with packetOp and the remainder with the scalar
 * op.  `packet` is the SIMD width assumed (8 = AVX); packet==0 selects the
 * scalar formula everywhere. */
static void sigmoid_array(const float* x, float* y, size_t n, int packet) {
  size_t nv = packet > 0 ? n - n % (size_t)packet : 0;
  for (size_t i = 0; i < nv; ++i) y[i] = sigmoid_packet(x[i]);
  for (size_t i = nv; i < n; ++i) y[i] = sigmoid_scalar(x[i]);
}

ORC_API float orc_sigmoid_packet(float x) { return sigmoid_packet(x); }
ORC_API float orc_sigmoid_scalar(float x) { return sigmoid_scalar(x); }

/* ------------------------------------------------------------------ */
/* A12: unary activations                                              */
/* ------------------------------------------------------------------ */

/* dynet/nodes-trig.cc:312-327 */
ORC_API void orc_tanh_fwd(const float* x, float* y, size_t n) {
  for (size_t i = 0; i < n; ++i) y[i] = tanhf(x[i]);
}
/* dynet/simd-functors.h:533-536: (1 - t*t) * d, accumulated */
ORC_API void orc_tanh_bwd(const float* y, const float* dy, float* dx, size_t n) {
  for (size_t i = 0; i < n; ++i) dx[i] += (1.0f - y[i] * y[i]) * dy[i];
}
/* dynet/nodes-activations.cc:64-79 */
ORC_API void orc_logistic_fwd(const float* x, float* y, size_t n, int packet) {
  sigmoid_array(x, y, n, packet);
}
/* dynet/simd-functors.h:509-515: (1 - t) * t * d */
ORC_API void orc_logistic_bwd(const float* y, const float* dy, float* dx, size_t n) {
  for (size_t i = 0; i < n; ++i) dx[i] += (1.0f - y[i]) * y[i] * dy[i];
}
/* dynet/nodes-activations.cc:30-45 */
ORC_API void orc_rectify_fwd(const float* x, float* y, size_t n) {
  for (size_t i = 0; i < n; ++i) y[i] = x[i] > 0.f ? x[i] : 0.f; /* cwiseMax(0) */
}
ORC_API void orc_rectify_bwd(const float* y, const float* dy, float* dx, size_t n) {
  /* cast<bool>().cast<float>(): 1 where fx != 0 */
  for (size_t i = 0; i < n; ++i) dx[i] += (y[i] != 0.f ? 1.f : 0.f) * dy[i];
}
/* dynet/nodes-activations.cc:166-181, dynet/functors.h:131-145 */
ORC_API void orc_elu_fwd(const float* x, float* y, size_t n, float alpha, float lambda) {
  for (size_t i = 0; i < n; ++i)
    y[i] = lambda * ((x[i] > 0.f) ? x[i] : alpha * expm1f(x[i]));
}
ORC_API void orc_elu_bwd(const float* x, const float* dy, float* dx, size_t n,
                         float alpha, float lambda) {
  for (size_t i = 0; i < n; ++i)
    dx[i] += dy[i] * ((x[i] > 0.f) ? lambda : lambda * alpha * expf(x[i]));
}

/* ------------------------------------------------------------------ */
/* A13: CwiseMultiply / CwiseSum / CwiseQuotient with broadcasting      */
/* ------------------------------------------------------------------ */
/* A shape is 4 dims + batch (dims beyond nd are 1), as tb<4> sees it
 * (dynet/nodes-arith-cwise.cc:196-307).  da/db are the two argument shapes;
 * the output shape is the element-wise max. */

static size_t shape_size(const uint32_t s[5]) {
  return (size_t)s[0] * s[1] * s[2] * s[3] * s[4];
}
static size_t bcast_index(const uint32_t idx[5], const uint32_t s[5]) {
  size_t off = 0, stride = 1;
  for (int k = 0; k < 5; ++k) {
    off += (s[k] == 1 ? 0 : idx[k]) * stride;
    stride *= s[k];
  }
  return off;
}
static void out_shape(const uint32_t a[5], const uint32_t b[5], uint32_t o[5]) {
  for (int k = 0; k < 5; ++k) o[k] = a[k] > b[k] ? a[k] : b[k];
}
#define FOR_EACH_OUT(o, idx)                                   \
  for (idx[4] = 0; idx[4] < o[4]; ++idx[4])                    \
    for (idx[3] = 0; idx[3] < o[3]; ++idx[3])                  \
      for (idx[2] = 0; idx[2] < o[2]; ++idx[2])                \
        for (idx[1] = 0; idx[1] < o[1]; ++idx[1])              \
          for (idx[0] = 0; idx[0] < o[0]; ++idx[0])

/* op: 0 = multiply, 1 = sum, 2 = quotient */
ORC_API void orc_cwise_fwd(int op, const float* a, const uint32_t sa[5], const float* b,
                           const uint32_t sb[5], float* y) {
  uint32_t o[5], idx[5];
  out_shape(sa, sb, o);
  size_t lin = 0;
  FOR_EACH_OUT(o, idx) {
    float av = a[bcast_index(idx, sa)], bv = b[bcast_index(idx, sb)];
    y[lin++] = op == 0 ? av * bv : (op == 1 ? av + bv : av / bv);
  }
}
/* Backward w.r.t. argument i (0 or 1), accumulated into dxi (shape of arg i).
 * Sums over broadcast axes in ascending linear order of the output, matching a
 * sequential Eigen reduction.  cmult: dynet/nodes-arith-cwise.cc:253-307;
 * csum: :99-157; cdiv: :354-412. */
ORC_API void orc_cwise_bwd(int op, const float* a, const uint32_t sa[5], const float* b,
                           const uint32_t sb[5], const float* dy, unsigned i, float* dxi) {
  uint32_t o[5], idx[5];
  out_shape(sa, sb, o);
  const uint32_t* si = i == 0 ? sa : sb;
  size_t ni = shape_size(si);
  float* acc = (float*)calloc(ni, sizeof(float));
  size_t lin = 0;
  FOR_EACH_OUT(o, idx) {
    float av = a[bcast_index(idx, sa)], bv = b[bcast_index(idx, sb)];
    float d = dy[lin++], g;
    if (op == 0) g = d * (i == 0 ? bv : av);
    else if (op == 1) g = d;
    else g = (i == 0) ? d / bv : -(d / (bv * bv) * av);
    acc[bcast_index(idx, si)] += g;
  }
  for (size_t k = 0; k < ni; ++k) dxi[k] += acc[k];
  free(acc);
}

/* ------------------------------------------------------------------ */
/* A6: Softmax                                                         */
/* ------------------------------------------------------------------ */
/* dynet/nodes-softmaxes.cc:40-87.  x is rows x cols per batch element. */
ORC_API void orc_softmax_fwd(const float* x, float* y, uint32_t rows, uint32_t cols,
                             uint32_t bd, unsigned dimension) {
  if (dimension == 0) { /* CPU branch :57-72, one column at a time */
    size_t ncols = (size_t)cols * bd;
    for (size_t c = 0; c < ncols; ++c) {
      const float* xc = x + c * rows;
      float* yc = y + c * rows;
      float m = xc[0];
      for (uint32_t r = 1; r < rows; ++r) m = xc[r] > m ? xc[r] : m;
      double zd = 0.0;
      for (uint32_t r = 0; r < rows; ++r) { yc[r] = expf(xc[r] - m); zd += yc[r]; }
      float z = (float)zd;
      for (uint32_t r = 0; r < rows; ++r) yc[r] = yc[r] / z;
    }
  } else { /* :73-85, reduce over dim 1 */
    for (uint32_t b = 0; b < bd; ++b)
      for (uint32_t r = 0; r < rows; ++r) {
        const float* xb = x + (size_t)b * rows * cols + r;
        float* yb = y + (size_t)b * rows * cols + r;
        float m = xb[0];
        for (uint32_t c = 1; c < cols; ++c) { float v = xb[(size_t)c * rows]; m = v > m ? v : m; }
        double zd = 0.0;
        for (uint32_t c = 0; c < cols; ++c) {
          float e = expf(xb[(size_t)c * rows] - m);
          yb[(size_t)c * rows] = e; zd += e;
        }
        float z = (float)zd;
        for (uint32_t c = 0; c < cols; ++c) yb[(size_t)c * rows] /= z;
      }
  }
}
/* dynet/nodes-softmaxes.cc:89-131: dx += (dy - sum(y*dy)) * y along `dimension` */
ORC_API void orc_softmax_bwd(const float* y, const float* dy, float* dx, uint32_t rows,
                             uint32_t cols, uint32_t bd, unsigned dimension) {
  if (dimension == 0) {
    size_t ncols = (size_t)cols * bd;
    for (size_t c = 0; c < ncols; ++c) {
      const float *yc = y + c * rows, *dc = dy + c * rows;
      float* xc = dx + c * rows;
      double zd = 0.0;
      for (uint32_t r = 0; r < rows; ++r) zd += yc[r] * dc[r];
      float z = (float)zd;
      for (uint32_t r = 0; r < rows; ++r) xc[r] += (dc[r] - z) * yc[r];
    }
  } else {
    for (uint32_t b = 0; b < bd; ++b)
      for (uint32_t r = 0; r < rows; ++r) {
        size_t base = (size_t)b * rows * cols + r;
        double zd = 0.0;
        for (uint32_t c = 0; c < cols; ++c) zd += y[base + (size_t)c * rows] * dy[base + (size_t)c * rows];
        float z = (float)zd;
        for (uint32_t c = 0; c < cols; ++c) {
          size_t k = base + (size_t)c * rows;
          dx[k] += (dy[k] - z) * y[k];
        }
      }
  }
}

/* ------------------------------------------------------------------ */
/* A7: logsumexp over an axis, LogSoftmax, LogSumExpDimension           */
/* ------------------------------------------------------------------ */
/* dynet/tensor.cc:468-507 (CPU branches :482-485, :497-505).  axis 0: one value
 * per column; axis 1: one per row.  m receives the maxima, z the result. */
ORC_API void orc_logsumexp_axis(const float* x, uint32_t rows, uint32_t cols, uint32_t bd,
                                unsigned axis, float* m, float* z) {
  uint32_t outer = axis == 0 ? cols : rows, inner = axis == 0 ? rows : cols;
  for (uint32_t b = 0; b < bd; ++b)
    for (uint32_t o = 0; o < outer; ++o) {
      const float* base = x + (size_t)b * rows * cols + (axis == 0 ? (size_t)o * rows : o);
      size_t stride = axis == 0 ? 1 : rows;
      float mv = base[0];
      for (uint32_t k = 1; k < inner; ++k) { float v = base[k * stride]; mv = v > mv ? v : mv; }
      double s = 0.0;
      for (uint32_t k = 0; k < inner; ++k) s += expf(base[k * stride] - mv);
      m[(size_t)b * outer + o] = mv;
      z[(size_t)b * outer + o] = logf((float)s) + mv;
    }
}
/* dynet/nodes-logsumexp.cc:136-146: dx += exp(x - z) * dz, broadcast along `axis` */
ORC_API void orc_logsumexp_dim_bwd(const float* x, const float* z, const float* dz, float* dx,
                                   uint32_t rows, uint32_t cols, uint32_t bd, unsigned axis) {
  uint32_t outer = axis == 0 ? cols : rows;
  for (uint32_t b = 0; b < bd; ++b)
    for (uint32_t c = 0; c < cols; ++c)
      for (uint32_t r = 0; r < rows; ++r) {
        size_t k = ((size_t)b * cols + c) * rows + r;
        size_t o = (size_t)b * outer + (axis == 0 ? c : r);
        dx[k] += expf(x[k] - z[o]) * dz[o];
      }
}
/* dynet/nodes-softmaxes.cc:156-183: y = x - logsumexp(column) */
ORC_API void orc_log_softmax_fwd(const float* x, float* y, uint32_t rows, uint32_t cols,
                                 uint32_t bd, float* z_aux, float* m_aux) {
  orc_logsumexp_axis(x, rows, cols, bd, 0, m_aux, z_aux);
  size_t ncols = (size_t)cols * bd;
  for (size_t c = 0; c < ncols; ++c)
    for (uint32_t r = 0; r < rows; ++r) y[c * rows + r] = x[c * rows + r] - z_aux[c];
}
/* dynet/nodes-softmaxes.cc:186-214: dx += exp(y) * -sum(dy) + dy */
ORC_API void orc_log_softmax_bwd(const float* y, const float* dy, float* dx, uint32_t rows,
                                 uint32_t cols, uint32_t bd) {
  size_t ncols = (size_t)cols * bd;
  for (size_t c = 0; c < ncols; ++c) {
    double zd = 0.0;
    for (uint32_t r = 0; r < rows; ++r) zd += dy[c * rows + r];
    float z = (float)zd;
    for (uint32_t r = 0; r < rows; ++r) {
      size_t k = c * rows + r;
      dx[k] += (expf(y[k]) * -z) + dy[k];
    }
  }
}

/* ------------------------------------------------------------------ */
/* A8: n-ary element-wise LogSumExp                                     */
/* ------------------------------------------------------------------ */
/* dynet/nodes-logsumexp.cc:37-73.  xs[k] has n elements per batch element and
 * batch size bds[k] in {1, bd}. */
ORC_API void orc_logsumexp_nary_fwd(const float* const* xs, const uint32_t* bds, unsigned k,
                                    size_t n, uint32_t bd, float* y) {
  size_t total = n * bd;
  if (k == 1) { memcpy(y, xs[0], total * sizeof(float)); return; }
  float* ms = (float*)malloc(total * sizeof(float));
  for (size_t e = 0; e < total; ++e) ms[e] = xs[0][bds[0] == bd ? e : e % n];
  for (unsigned j = 1; j < k; ++j)
    for (size_t e = 0; e < total; ++e) {
      float v = xs[j][bds[j] == bd ? e : e % n];
      ms[e] = v > ms[e] ? v : ms[e];
    }
  for (size_t e = 0; e < total; ++e) y[e] = expf(xs[0][bds[0] == bd ? e : e % n] - ms[e]);
  for (unsigned j = 1; j < k; ++j)
    for (size_t e = 0; e < total; ++e) y[e] += expf(xs[j][bds[j] == bd ? e : e % n] - ms[e]);
  for (size_t e = 0; e < total; ++e) y[e] = logf(y[e]) + ms[e];
  free(ms);
}
/* dynet/nodes-logsumexp.cc:75-98: dx_i += exp(x_i - y) * dy, batch-summed if x_i has bd 1 */
ORC_API void orc_logsumexp_nary_bwd(const float* xi, uint32_t bdi, unsigned k, const float* y,
                                    const float* dy, size_t n, uint32_t bd, float* dxi) {
  size_t total = n * bd;
  if (k == 1) { for (size_t e = 0; e < total; ++e) dxi[e] += dy[e]; return; }
  if (bdi == bd) {
    for (size_t e = 0; e < total; ++e) dxi[e] += expf(xi[e] - y[e]) * dy[e];
  } else {
    for (size_t r = 0; r < n; ++r) {
      float s = 0.f;
      for (uint32_t b = 0; b < bd; ++b) s += expf(xi[r] - y[b * n + r]) * dy[b * n + r];
      dxi[r] += s;
    }
  }
}

/* ------------------------------------------------------------------ */
/* A9: PickNegLogSoftmax                                                */
/* ------------------------------------------------------------------ */
/* dynet/nodes-pickneglogsoftmax.cc:78-118.  x is rows x bd; ids[b] < rows is
 * checked (returns -1 like the reference's DYNET_ARG_CHECK throws). */
ORC_API int orc_pnls_fwd(const float* x, uint32_t rows, uint32_t bd, const uint32_t* ids,
                         float* loss, float* z_aux, float* m_aux) {
  for (uint32_t b = 0; b < bd; ++b) if (ids[b] >= rows) return -1;
  orc_logsumexp_axis(x, rows, 1, bd, 0, m_aux, z_aux);
  for (uint32_t b = 0; b < bd; ++b) loss[b] = x[(size_t)b * rows + ids[b]];
  for (uint32_t b = 0; b < bd; ++b) loss[b] = z_aux[b] - loss[b];
  return 0;
}
/* dynet/nodes-pickneglogsoftmax.cc:120-146 (CPU loop :137-141) */
ORC_API void orc_pnls_bwd(const float* x, uint32_t rows, uint32_t bd, const uint32_t* ids,
                          const float* z_aux, const float* dE, float* dx) {
  for (uint32_t b = 0; b < bd; ++b) {
    for (uint32_t r = 0; r < rows; ++r) {
      size_t k = (size_t)b * rows + r;
      dx[k] += expf(x[k] - z_aux[b]) * dE[b];
    }
    dx[(size_t)b * rows + ids[b]] -= dE[b];
  }
}

/* ------------------------------------------------------------------ */
/* A10: WeightNormalization                                             */
/* ------------------------------------------------------------------ */
/* dynet/nodes-normalization.cc:28-41 */
ORC_API void orc_weight_norm_fwd(const float* w, float g, float* y, size_t n) {
  double ssd = 0.0;
  for (size_t i = 0; i < n; ++i) ssd += w[i] * w[i];
  float nrm = sqrtf((float)ssd);
  for (size_t i = 0; i < n; ++i) y[i] = (w[i] / nrm) * g;
}
/* dynet/nodes-normalization.cc:43-66 */
ORC_API void orc_weight_norm_bwd(const float* w, float g, const float* y, const float* dy,
                                 unsigned i, float* dxi, size_t n) {
  double ssd = 0.0, dotd = 0.0;
  for (size_t k = 0; k < n; ++k) { ssd += w[k] * w[k]; dotd += dy[k] * w[k]; }
  float ss = (float)ssd, dot = (float)dotd;
  if (i == 0) {
    float nrm = sqrtf(ss), t2 = dot / ss;
    for (size_t k = 0; k < n; ++k) dxi[k] += (dy[k] / nrm) * g - y[k] * t2;
  } else {
    dxi[0] += dot / sqrtf(ss);
  }
}

/* ------------------------------------------------------------------ */
/* A11: MomentDimension / StdDimension over dim 0 of a vector batch, and */
/*      the composite layer_norm                                        */
/* ------------------------------------------------------------------ */
/* The layer_norm composite (dynet/expr.cc:248-253) only uses dims = all
 * non-batch dims, include_batch_dim = false; x is viewed as n x bd. */

/* dynet/nodes-moments.cc:181-209 (order r, dims = all, no batch) */
ORC_API void orc_moment_elems_fwd(const float* x, size_t n, uint32_t bd, unsigned order, float* out) {
  for (uint32_t b = 0; b < bd; ++b) {
    double s = 0.0;
    for (size_t i = 0; i < n; ++i) {
      float v = x[b * n + i];
      s += order == 1 ? v : (order == 2 ? v * v : powf(v, (float)order));
    }
    out[b] = (float)s / (float)n;
  }
}
/* dynet/nodes-moments.cc:246-266 */
ORC_API void orc_moment_elems_bwd(const float* x, size_t n, uint32_t bd, unsigned order,
                                  const float* dE, float* dx) {
  float fn = (float)n;
  for (uint32_t b = 0; b < bd; ++b)
    for (size_t i = 0; i < n; ++i) {
      float v = x[b * n + i];
      if (order == 1) dx[b * n + i] += dE[b] / fn;
      else if (order == 2) dx[b * n + i] += (dE[b] * v) * (2.f / fn);
      else if (order == 3) dx[b * n + i] += (dE[b] * (v * v)) * (3.f / fn);
      else dx[b * n + i] += (dE[b] * powf(v, (float)order - 1)) * ((float)order / fn);
    }
}
/* dynet/nodes-moments.cc:434-463: population std, mean subtracted first */
ORC_API void orc_std_elems_fwd(const float* x, size_t n, uint32_t bd, float* out) {
  float fn = (float)n;
  for (uint32_t b = 0; b < bd; ++b) {
    double s = 0.0, q = 0.0;
    for (size_t i = 0; i < n; ++i) s += x[b * n + i];
    float mean = (float)s / fn;
    for (size_t i = 0; i < n; ++i) { float d = x[b * n + i] - mean; q += d * d; }
    out[b] = sqrtf((float)q / fn);
  }
}
/* dynet/nodes-moments.cc:498-530 with FSqrtBackward (dynet/simd-functors.h:212-226) */
ORC_API void orc_std_elems_bwd(const float* x, size_t n, uint32_t bd, const float* fx,
                               const float* dE, float* dx) {
  float fn = (float)n;
  for (uint32_t b = 0; b < bd; ++b) {
    double s = 0.0;
    for (size_t i = 0; i < n; ++i) s += x[b * n + i];
    float mean = (float)s / fn;
    float sb = dE[b] / (2.f * fx[b]);
    for (size_t i = 0; i < n; ++i) dx[b * n + i] += (2.f / fn) * (x[b * n + i] - mean) * sb;
  }
}
/* Moment / Std over the batch axis only (dims = {}, include_batch_dim = true):
 * dynet/nodes-moments.cc:192-200, :448-455.  Used by the std_dim_value golden test. */
ORC_API void orc_std_dim0_batch_fwd(const float* x, uint32_t d0, uint32_t d1, uint32_t bd, float* out) {
  /* reduce over dim 0 and the batch: out has d1 entries (nodes-moments.cc:464-471) */
  float fn = (float)d0 * (float)bd;
  for (uint32_t j = 0; j < d1; ++j) {
    double s = 0.0, q = 0.0;
    for (uint32_t b = 0; b < bd; ++b)
      for (uint32_t i = 0; i < d0; ++i) s += x[((size_t)b * d1 + j) * d0 + i];
    float mean = (float)s / fn;
    for (uint32_t b = 0; b < bd; ++b)
      for (uint32_t i = 0; i < d0; ++i) { float d = x[((size_t)b * d1 + j) * d0 + i] - mean; q += d * d; }
    out[j] = sqrtf((float)q / fn);
  }
}

/* layer_norm forward, node by node (dynet/expr.cc:248-253):
 *   mu = mean_elems(x); xc = x + (-mu); sigma = std_elems(x);
 *   y = cmult(g, cdiv(xc, sigma + 1e-8)) + b          (g, b have batch size 1) */
ORC_API void orc_layer_norm_fwd(const float* x, const float* g, const float* bias, float* y,
                                size_t n, uint32_t bd) {
  float* mu = (float*)malloc(bd * sizeof(float));
  float* sg = (float*)malloc(bd * sizeof(float));
  orc_moment_elems_fwd(x, n, bd, 1, mu);
  orc_std_elems_fwd(x, n, bd, sg);
  for (uint32_t b = 0; b < bd; ++b) {
    float neg = -mu[b], s2 = sg[b] + 1e-8f;
    for (size_t i = 0; i < n; ++i) {
      float xc = x[b * n + i] + neg;
      float q = xc / s2;
      y[b * n + i] = g[i] * q + bias[i];
    }
  }
  free(mu); free(sg);
}
/* layer_norm backward through the same eight nodes in reverse topological order
 * (dynet/exec.cc:166-284).  Accumulates into dx (n x bd), dg (n), db (n). */
ORC_API void orc_layer_norm_bwd(const float* x, const float* g, const float* dy, float* dx,
                                float* dg, float* db, size_t n, uint32_t bd) {
  float fn = (float)n;
  float* mu = (float*)malloc(bd * sizeof(float));
  float* sg = (float*)malloc(bd * sizeof(float));
  orc_moment_elems_fwd(x, n, bd, 1, mu);
  orc_std_elems_fwd(x, n, bd, sg);
  /* CwiseSum(y1, b): db += sum_b dy (nodes-arith-cwise.cc:117-119) */
  for (uint32_t b = 0; b < bd; ++b)
    for (size_t i = 0; i < n; ++i) db[i] += dy[b * n + i];
  /* CwiseMultiply(g, q): dg += sum_b dy*q (:270-272) */
  for (size_t i = 0; i < n; ++i) {
    double s = 0.0;
    for (uint32_t b = 0; b < bd; ++b) {
      float s2 = sg[b] + 1e-8f;
      float q = (x[b * n + i] + (-mu[b])) / s2;
      s += dy[b * n + i] * q;
    }
    dg[i] += (float)s;
  }
  for (uint32_t b = 0; b < bd; ++b) {
    float neg = -mu[b], s2 = sg[b] + 1e-8f;
    /* dq = dy * g;  cdiv i=1: ds2 -= sum(dq / s2^2 * xc) (:392-411) */
    float ssq = s2 * s2;
    double acc = 0.0, dneg = 0.0;
    for (size_t i = 0; i < n; ++i) {
      float dq = dy[b * n + i] * g[i];
      float xc = x[b * n + i] + neg;
      acc += dq / ssq * xc;
    }
    float dsigma = -(float)acc; /* ConstantPlusX passes the gradient through */
    /* StdDimension backward: dx += (2/n)(x - mean) * dsigma/(2 sigma) */
    float sb = dsigma / (2.f * sg[b]);
    for (size_t i = 0; i < n; ++i) dx[b * n + i] += (2.f / fn) * (x[b * n + i] - mu[b]) * sb;
    /* cdiv i=0 then CwiseSum(x, -mu): dx += dq / s2; dneg += sum(dq / s2) */
    for (size_t i = 0; i < n; ++i) {
      float dxc = (dy[b * n + i] * g[i]) / s2;
      dx[b * n + i] += dxc;
      dneg += dxc;
    }
    /* Negate then MomentDimension backward: dx += dmu / n */
    float dmu = -(float)dneg;
    for (size_t i = 0; i < n; ++i) dx[b * n + i] += dmu / fn;
  }
  free(mu); free(sg);
}

/* ------------------------------------------------------------------ */
/* A4/A5: LookupNode gather and gradient scatter-add                    */
/* ------------------------------------------------------------------ */
/* dynet/param-nodes.cc:304-329 (CPU branch :321-326).  Returns -1 on an
 * out-of-range id (the reference throws std::invalid_argument). */
ORC_API int orc_lookup_fwd(const float* table, uint32_t E, uint32_t V, const uint32_t* ids,
                           uint32_t n, float scale, float* out) {
  for (uint32_t b = 0; b < n; ++b) {
    if (ids[b] >= V) return -1;
    const float* row = table + (size_t)ids[b] * E;
    for (uint32_t e = 0; e < E; ++e) out[(size_t)b * E + e] = row[e] * scale;
  }
  return 0;
}
/* dynet/model.cc:728-743 (CPU branch): grads[ids[b]] += g[:, b], in order of b */
ORC_API void orc_lookup_accumulate_grads(float* all_grads, uint32_t E, const uint32_t* ids,
                                         uint32_t n, const float* g) {
  for (uint32_t b = 0; b < n; ++b) {
    float* row = all_grads + (size_t)ids[b] * E;
    for (uint32_t e = 0; e < E; ++e) row[e] += g[(size_t)b * E + e];
  }
}

/* ------------------------------------------------------------------ */
/* GEMM helpers (dynet/matrix-multiply.h CPU branches)                  */
/* ------------------------------------------------------------------ */
/* The loops are blocked so that each weight column is streamed once, but every
 * output element still accumulates its products in ascending k (or batch) order. */
/* y[M x N] += l[M x K] * r[K x N], all column-major (:45-55) */
static void gemm_nn_acc(const float* l, const float* r, float* y, size_t M, size_t K, size_t N) {
  const size_t MB = 256, NB = 32;
  for (size_t n0 = 0; n0 < N; n0 += NB) {
    size_t n1 = n0 + NB < N ? n0 + NB : N;
    for (size_t m0 = 0; m0 < M; m0 += MB) {
      size_t mb = (m0 + MB < M ? m0 + MB : M) - m0;
      for (size_t k = 0; k < K; ++k) {
        const float* lc = l + k * M + m0;
        for (size_t n = n0; n < n1; ++n) {
          float rv = r[n * K + k];
          float* yc = y + n * M + m0;
          for (size_t m = 0; m < mb; ++m) yc[m] += lc[m] * rv;
        }
      }
    }
  }
}
/* y[K x N] += l[M x K]^T * r[M x N]  (:120-125) */
static void gemm_tn_acc(const float* l, const float* r, float* y, size_t M, size_t K, size_t N) {
  for (size_t k = 0; k < K; ++k) {
    const float* lc = l + k * M;
    for (size_t n = 0; n < N; ++n) {
      const float* rc = r + n * M;
      float s = 0.f;
#pragma omp simd reduction(+ : s)
      for (size_t m = 0; m < M; ++m) s += lc[m] * rc[m];
      y[n * K + k] += s;
    }
  }
}
/* y[M x K] += l[M x N] * r[K x N]^T, i.e. summed over the N batch columns (:183-187) */
static void gemm_nt_acc(const float* l, const float* r, float* y, size_t M, size_t N, size_t K) {
  const size_t MB = 1024;
  for (size_t m0 = 0; m0 < M; m0 += MB) {
    size_t mb = (m0 + MB < M ? m0 + MB : M) - m0;
    for (size_t k = 0; k < K; ++k) {
      float* yc = y + k * M + m0;
      for (size_t n = 0; n < N; ++n) {
        float rv = r[n * K + k];
        const float* lc = l + n * M + m0;
        for (size_t m = 0; m < mb; ++m) yc[m] += lc[m] * rv;
      }
    }
  }
}
ORC_API void orc_gemm_nn_acc(const float* l, const float* r, float* y, size_t M, size_t K, size_t N) { gemm_nn_acc(l, r, y, M, K, N); }
ORC_API void orc_gemm_tn_acc(const float* l, const float* r, float* y, size_t M, size_t K, size_t N) { gemm_tn_acc(l, r, y, M, K, N); }
ORC_API void orc_gemm_nt_acc(const float* l, const float* r, float* y, size_t M, size_t N, size_t K) { gemm_nt_acc(l, r, y, M, N, K); }

/* ------------------------------------------------------------------ */
/* MatrixMultiply / AffineTransform nodes                               */
/* ------------------------------------------------------------------ */
/* A matrix argument: rows x cols x bd, column-major, batch slowest. */
typedef struct { const float* v; uint32_t rows, cols, bd; } orc_mat;
static const float* mat_batch(const orc_mat* t, uint32_t b) { return t->v + (size_t)(b % t->bd) * t->rows * t->cols; }

/* y = beta*y + l*r   (dynet/matrix-multiply.h:45-94, CPU branch without MKL) */
static void mm_fwd(const orc_mat* l, const orc_mat* r, float* y, uint32_t ybd, float beta) {
  size_t M = l->rows, K = l->cols, N = r->cols, ysz = M * N * ybd;
  for (size_t e = 0; e < ysz; ++e) y[e] = beta * y[e];
  if (l->bd == 1 && r->bd == ybd) gemm_nn_acc(l->v, r->v, y, M, K, N * ybd);
  else for (uint32_t b = 0; b < ybd; ++b) gemm_nn_acc(mat_batch(l, b), mat_batch(r, b), y + (size_t)b * M * N, M, K, N);
}
/* y += l^T * r   (dynet/matrix-multiply.h:117-156) */
static void mm_transp_l_acc(const orc_mat* l, const orc_mat* r, float* y, uint32_t ybd) {
  uint32_t max_b = l->bd > r->bd ? l->bd : r->bd;
  size_t M = l->rows, K = l->cols, N = r->cols;
  if (l->bd == 1 && ybd == r->bd) gemm_tn_acc(l->v, r->v, y, M, K, N * ybd);
  else for (uint32_t b = 0; b < max_b; ++b) gemm_tn_acc(mat_batch(l, b), mat_batch(r, b), y + (size_t)(b % ybd) * K * N, M, K, N);
}
/* y += l * r^T   (dynet/matrix-multiply.h:180-219) */
static void mm_transp_r_acc(const orc_mat* l, const orc_mat* r, float* y, uint32_t ybd) {
  uint32_t max_b = l->bd > r->bd ? l->bd : r->bd;
  size_t M = l->rows, N = l->cols, K = r->rows;
  if (ybd == 1 && l->bd == r->bd) gemm_nt_acc(l->v, r->v, y, M, N * l->bd, K);
  else for (uint32_t b = 0; b < max_b; ++b) gemm_nt_acc(mat_batch(l, b), mat_batch(r, b), y + (size_t)(b % ybd) * M * K, M, N, K);
}

/* AffineTransform::forward_dev_impl (dynet/nodes-affinetransform.cc:77-110): xs = {bias, A1, B1, A2, B2, ...};
 * the bias block is tiled over fx (CPU branch: bias.bd must be 1 when it is smaller than fx);
 * with nxs == 2 and a null bias this is MatrixMultiply::forward_dev_impl (dynet/nodes-matrixmultiply.cc:50-56). */
ORC_API int orc_affine_fwd(const orc_mat* xs, unsigned nxs, float* fx, uint32_t frows, uint32_t fcols, uint32_t fbd) {
  size_t fsz = (size_t)frows * fcols * fbd;
  if (xs[0].v) {
    size_t bsz = (size_t)xs[0].rows * xs[0].cols * xs[0].bd;
    if (bsz != fsz && xs[0].bd != 1) return 1;
    for (size_t o = 0; o < fsz; o += bsz) memcpy(fx + o, xs[0].v, sizeof(float) * (fsz - o < bsz ? fsz - o : bsz));
  } else {
    memset(fx, 0, sizeof(float) * fsz);
  }
  for (unsigned i = 1; i + 1 < nxs; i += 2) mm_fwd(&xs[i], &xs[i + 1], fx, fbd, 1.0f);
  return 0;
}
/* AffineTransform::backward_dev_impl (dynet/nodes-affinetransform.cc:112-157) and
 * MatrixMultiply::backward_dev_impl (dynet/nodes-matrixmultiply.cc:58-74); dxi accumulates. */
ORC_API int orc_affine_bwd(const orc_mat* xs, unsigned nxs, const float* dEdf, uint32_t frows, uint32_t fcols, uint32_t fbd,
                           unsigned i, float* dxi) {
  (void)nxs;
  orc_mat d = {dEdf, frows, fcols, fbd};
  if (i == 0) {
    size_t dx = (size_t)xs[0].rows * xs[0].cols * xs[0].bd, df = (size_t)frows * fcols * fbd;
    if (dx != df && xs[0].bd != 1) return 1;
    /* every output element sums its chunks in ascending order, in double, rounded once */
    for (size_t r = 0; r < dx; ++r) {
      double acc = 0.0;
      for (size_t o = r; o < df; o += dx) acc += dEdf[o];
      dxi[r] += (float)acc;
    }
  } else if (i % 2 == 1) {
    mm_transp_r_acc(&d, &xs[i + 1], dxi, xs[i].bd);
  } else {
    mm_transp_l_acc(&xs[i - 1], &d, dxi, xs[i].bd);
  }
  return 0;
}

/* ------------------------------------------------------------------ */
/* A1: VanillaLSTMGates                                                 */
/* ------------------------------------------------------------------ */
/* Inputs x_1..x_k (dims xdims[j], batch B) are concatenated along dim 0 to I
 * rows.  mask_x / mask_h may be NULL (no dropout) and have batch size
 * mask_*_bd in {1, B}.  dynet/nodes-lstm.cc:101-235. */
static float* concat_inputs(const float* const* xs, const uint32_t* xdims, unsigned k,
                            uint32_t I, uint32_t B) {
  float* x = (float*)malloc((size_t)I * B * sizeof(float));
  uint32_t off = 0;
  for (unsigned j = 0; j < k; ++j) {
    for (uint32_t b = 0; b < B; ++b)
      memcpy(x + (size_t)b * I + off, xs[j] + (size_t)b * xdims[j], xdims[j] * sizeof(float));
    off += xdims[j];
  }
  return x;
}
static void apply_mask(float* v, const float* mask, uint32_t n, uint32_t B, uint32_t mbd) {
  for (uint32_t b = 0; b < B; ++b)
    for (uint32_t i = 0; i < n; ++i)
      v[(size_t)b * n + i] *= mask[(mbd == B ? (size_t)b * n : 0) + i];
}

ORC_API void orc_lstm_gates_fwd(const float* const* xs, const uint32_t* xdims, unsigned k,
                                const float* h_tm1, const float* Wx, const float* Wh,
                                const float* bias, const float* mask_x, uint32_t mask_x_bd,
                                const float* mask_h, uint32_t mask_h_bd, uint32_t H, uint32_t I,
                                uint32_t B, float forget_bias, int skip_matmul, int packet,
                                float* fx) {
  size_t G = (size_t)4 * H;
  float* x = concat_inputs(xs, xdims, k, I, B);
  float* h = (float*)malloc((size_t)H * B * sizeof(float));
  memcpy(h, h_tm1, (size_t)H * B * sizeof(float));
  for (uint32_t b = 0; b < B; ++b) memcpy(fx + b * G, bias, G * sizeof(float)); /* :148-152 */
  for (uint32_t b = 0; b < B; ++b)
    for (uint32_t r = H; r < 2 * H; ++r) fx[b * G + r] += forget_bias;          /* :154 */
  if (mask_x) { apply_mask(x, mask_x, I, B, mask_x_bd); apply_mask(h, mask_h, H, B, mask_h_bd); }
  if (!skip_matmul) { /* weightnoise_std > 0 skips both products in the reference (:200-219) */
    gemm_nn_acc(Wx, x, fx, G, I, B);
    gemm_nn_acc(Wh, h, fx, G, H, B);
  }
  /* :222-232: the i,f,o rows are copied to a contiguous 3H x B buffer first, so
   * the packet/scalar split of the sigmoid applies to that buffer as a whole. */
  size_t n3 = (size_t)3 * H * B;
  float* ifo = (float*)malloc(n3 * sizeof(float));
  for (uint32_t b = 0; b < B; ++b) memcpy(ifo + (size_t)b * 3 * H, fx + b * G, 3 * H * sizeof(float));
  sigmoid_array(ifo, ifo, n3, packet);
  for (uint32_t b = 0; b < B; ++b) memcpy(fx + b * G, ifo + (size_t)b * 3 * H, 3 * H * sizeof(float));
  for (uint32_t b = 0; b < B; ++b)
    for (uint32_t r = 3 * H; r < 4 * H; ++r) fx[b * G + r] = tanhf(fx[b * G + r]);
  free(ifo); free(x); free(h);
}

/* Gate pre-activation gradient shared by every argument (:354-361). */
static float* gate_deriv(const float* fx, const float* dEdf, uint32_t H, uint32_t B) {
  size_t G = (size_t)4 * H;
  float* d = (float*)malloc(G * B * sizeof(float));
  for (uint32_t b = 0; b < B; ++b) {
    for (uint32_t r = 0; r < 3 * H; ++r) {
      float g = fx[b * G + r];
      d[b * G + r] = dEdf[b * G + r] * g * (1.f - g);
    }
    for (uint32_t r = 3 * H; r < 4 * H; ++r) {
      float g = fx[b * G + r];
      d[b * G + r] = dEdf[b * G + r] * (1.f - g * g);
    }
  }
  return d;
}

/* Backward w.r.t. argument i (numbering of the reference: 0..k-1 inputs, k = h_tm1,
 * k+1 = Wx, k+2 = Wh, k+3 = b), accumulated into dxi.  dynet/nodes-lstm.cc:237-527. */
ORC_API void orc_lstm_gates_bwd(const float* const* xs, const uint32_t* xdims, unsigned k,
                                const float* h_tm1, const float* Wx, const float* Wh,
                                const float* mask_x, uint32_t mask_x_bd, const float* mask_h,
                                uint32_t mask_h_bd, uint32_t H, uint32_t I, uint32_t B,
                                const float* fx, const float* dEdf, unsigned i, float* dxi) {
  size_t G = (size_t)4 * H;
  float* dg = gate_deriv(fx, dEdf, H, B);
  if (i < k) {
    uint32_t off = 0, di = xdims[i];
    for (unsigned j = 0; j < i; ++j) off += xdims[j];
    const float* Wslice = Wx + (size_t)off * G; /* columns [off, off+di) are contiguous */
    if (mask_x) {
      float* my = (float*)calloc((size_t)di * B, sizeof(float));
      gemm_tn_acc(Wslice, dg, my, G, di, B);
      for (uint32_t b = 0; b < B; ++b)
        for (uint32_t r = 0; r < di; ++r)
          dxi[(size_t)b * di + r] += my[(size_t)b * di + r] *
                                     mask_x[(mask_x_bd == B ? (size_t)b * I : 0) + off + r];
      free(my);
    } else {
      gemm_tn_acc(Wslice, dg, dxi, G, di, B);
    }
  } else if (i == k) {
    if (mask_h) {
      float* my = (float*)calloc((size_t)H * B, sizeof(float));
      gemm_tn_acc(Wh, dg, my, G, H, B);
      for (uint32_t b = 0; b < B; ++b)
        for (uint32_t r = 0; r < H; ++r)
          dxi[(size_t)b * H + r] += my[(size_t)b * H + r] *
                                    mask_h[(mask_h_bd == B ? (size_t)b * H : 0) + r];
      free(my);
    } else {
      gemm_tn_acc(Wh, dg, dxi, G, H, B);
    }
  } else if (i == k + 1) {
    float* x = concat_inputs(xs, xdims, k, I, B);
    if (mask_x) apply_mask(x, mask_x, I, B, mask_x_bd);
    gemm_nt_acc(dg, x, dxi, G, B, I);
    free(x);
  } else if (i == k + 2) {
    float* h = (float*)malloc((size_t)H * B * sizeof(float));
    memcpy(h, h_tm1, (size_t)H * B * sizeof(float));
    if (mask_h) apply_mask(h, mask_h, H, B, mask_h_bd);
    gemm_nt_acc(dg, h, dxi, G, B, H);
    free(h);
  } else if (i == k + 3) {
    for (size_t r = 0; r < G; ++r) {
      float s = 0.f;
      for (uint32_t b = 0; b < B; ++b) s += dg[b * G + r];
      dxi[r] += s;
    }
  }
  free(dg);
}

/* ------------------------------------------------------------------ */
/* A2/A3: VanillaLSTMC, VanillaLSTMH                                    */
/* ------------------------------------------------------------------ */
/* dynet/nodes-lstm.cc:562-589 */
ORC_API void orc_lstm_c_fwd(const float* c_tm1, const float* gates, uint32_t H, uint32_t B, float* c) {
  for (uint32_t b = 0; b < B; ++b) {
    const float* g = gates + (size_t)b * 4 * H;
    for (uint32_t j = 0; j < H; ++j)
      c[(size_t)b * H + j] = g[j] * g[3 * H + j] + g[H + j] * c_tm1[(size_t)b * H + j];
  }
}
/* dynet/nodes-lstm.cc:591-615 */
ORC_API void orc_lstm_c_bwd(const float* c_tm1, const float* gates, uint32_t H, uint32_t B,
                            const float* dc, unsigned i, float* dxi) {
  for (uint32_t b = 0; b < B; ++b) {
    const float* g = gates + (size_t)b * 4 * H;
    for (uint32_t j = 0; j < H; ++j) {
      float d = dc[(size_t)b * H + j];
      if (i == 0) {
        dxi[(size_t)b * H + j] += d * g[H + j];
      } else {
        float* o = dxi + (size_t)b * 4 * H;
        o[j] += d * g[3 * H + j];
        o[H + j] += d * c_tm1[(size_t)b * H + j];
        o[3 * H + j] += d * g[j];
      }
    }
  }
}
/* dynet/nodes-lstm.cc:650-668 */
ORC_API void orc_lstm_h_fwd(const float* c_t, const float* gates, uint32_t H, uint32_t B, float* h) {
  for (uint32_t b = 0; b < B; ++b)
    for (uint32_t j = 0; j < H; ++j)
      h[(size_t)b * H + j] = gates[(size_t)b * 4 * H + 2 * H + j] * tanhf(c_t[(size_t)b * H + j]);
}
/* dynet/nodes-lstm.cc:670-703 */
ORC_API void orc_lstm_h_bwd(const float* c_t, const float* gates, uint32_t H, uint32_t B,
                            const float* dh, unsigned i, float* dxi) {
  for (uint32_t b = 0; b < B; ++b)
    for (uint32_t j = 0; j < H; ++j) {
      float t = tanhf(c_t[(size_t)b * H + j]);
      float d = dh[(size_t)b * H + j];
      if (i == 0) dxi[(size_t)b * H + j] += d * gates[(size_t)b * 4 * H + 2 * H + j] * (1.f - t * t);
      else dxi[(size_t)b * 4 * H + 2 * H + j] += d * t;
    }
}

/* ------------------------------------------------------------------ */
/* A14: autobatch ragged gather / scatter-add                           */
/* ------------------------------------------------------------------ */
/* dynet/exec.cc:298-361 (CPU: memcpy per slice) and :363-411 (accumulate per slice) */
ORC_API void orc_parallel_memcpy(int num_seqs, const float* const* src, float* const* trg,
                                 const size_t* len) {
  for (int s = 0; s < num_seqs; ++s) memcpy(trg[s], src[s], len[s] * sizeof(float));
}
ORC_API void orc_parallel_accumulate(int num_seqs, const float* const* src, float* const* trg,
                                     const size_t* len) {
  for (int s = 0; s < num_seqs; ++s)
    for (size_t i = 0; i < len[s]; ++i) trg[s][i] += src[s][i];
}
