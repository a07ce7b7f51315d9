// MatrixMultiply and AffineTransform nodes on the 3xTF32 tensor-pipe GEMM.
//   MatrixMultiply   dynet/nodes-matrixmultiply.cc:50-74
//   AffineTransform  dynet/nodes-affinetransform.cc:77-157
// Both are thin drivers over the three product forms of dynet/matrix-multiply.h:
//   y  = [bias +] l * r      (MatrixMultiply,           :17-94)
//   y +=  l^T * r            (MatrixTranspMultiplyAcc,  :98-156)
//   y +=  l * r^T            (MatrixMultiplyTranspAcc,  :160-219)
// A left operand with one batch element multiplies all batch columns of the right operand in one
// product (N = cols * bd); otherwise the batch elements are multiplied one by one, a batch-1 operand
// being reused for every element (and a batch-1 result summed over them).
#include "common.cuh"
#include "gemm.cuh"
#include "reduce.cuh"

namespace {

constexpr int kThreads = 256;

// dst[e] = src[e % period]
__global__ void __launch_bounds__(kThreads) k_tile_copy(const float* __restrict__ src, size_t period, float* __restrict__ dst,
                                                        size_t n, int vec) {
  dyb_grid_dep_sync();
  if (vec) {
    const size_t n4 = n / 4;
    for (size_t q = (size_t)blockIdx.x * kThreads + threadIdx.x; q < n4; q += (size_t)gridDim.x * kThreads)
      st4(dst + 4 * q, ld4(src + (4 * q) % period));
    return;
  }
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < n; e += (size_t)gridDim.x * kThreads) dst[e] = src[e % period];
}

// dst[e] += src[e]
__global__ void __launch_bounds__(kThreads) k_add_into(const float* __restrict__ src, float* __restrict__ dst, size_t n, int vec) {
  dyb_grid_dep_sync();
  if (vec) {
    const size_t n4 = n / 4;
    for (size_t q = (size_t)blockIdx.x * kThreads + threadIdx.x; q < n4; q += (size_t)gridDim.x * kThreads) {
      float4 a = ld4_stream(src + 4 * q), o = ld4(dst + 4 * q);
      st4(dst + 4 * q, make_float4(o.x + a.x, o.y + a.y, o.z + a.z, o.w + a.w));
    }
    return;
  }
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < n; e += (size_t)gridDim.x * kThreads) dst[e] += src[e];
}

struct ChunkOf {   // f(r, b) = v[r + n * b]
  const float* v; size_t n;
  __device__ float operator()(size_t r, uint32_t b) const { return v[r + n * (size_t)b]; }
};

inline const float* batch_ptr(const dyb200_tensor* t, uint32_t b) { return t->v + (size_t)(b % t->bd) * t_rows(t) * t_cols(t); }

int check_matrix(dyb200_ctx* ctx, const dyb200_tensor* t, const char* what) {
  DYB_CHECK_ARG(ctx, t && t->v, "%s: null tensor", what);
  DYB_CHECK_ARG(ctx, t->nd <= 2, "%s: cannot multiply tensors of dimension higher than 2", what);
  DYB_CHECK_ARG(ctx, t->bd >= 1, "%s: empty batch", what);
  return DYB200_OK;
}

// y = epilogue(l * r); mode is EPI_STORE, EPI_ACCUM or EPI_BIAS (bias = column vector of rows(y))
int mm_fwd(dyb200_ctx* ctx, const dyb200_tensor* l, const dyb200_tensor* r, dyb200_tensor* y, int mode, const float* bias,
           int a_is_param) {
  const uint32_t M = t_rows(l), K = t_cols(l), N = t_cols(r);
  if (l->bd == 1 && r->bd == y->bd) {
    GemmPair p{l->v, M, 0, r->v, K, 0, K, nullptr, 0, 0, a_is_param};
    GemmEpilogue e{mode, y->v, M, bias, 0, 0.f, nullptr, 0, 0};
    return dyb200_gemm_fused(ctx, M, N * y->bd, 1, &p, e);
  }
  for (uint32_t b = 0; b < y->bd; ++b) {
    GemmPair p{batch_ptr(l, b), M, 0, batch_ptr(r, b), K, 0, K, nullptr, 0, 0, 0};
    GemmEpilogue e{mode, y->v + (size_t)b * M * N, M, bias, 0, 0.f, nullptr, 0, 0};
    int rc = dyb200_gemm_fused(ctx, M, N, 1, &p, e);
    if (rc) return rc;
  }
  return DYB200_OK;
}

// y += l^T * r   (l: M x K, r: M x N, y: K x N)
int mm_transp_l_acc(dyb200_ctx* ctx, const dyb200_tensor* l, const dyb200_tensor* r, dyb200_tensor* y, int a_is_param) {
  const uint32_t M = t_rows(l), K = t_cols(l), N = t_cols(r);
  const uint32_t max_b = l->bd > r->bd ? l->bd : r->bd;
  if (l->bd == 1 && y->bd == r->bd) {
    GemmPair p{l->v, M, 1, r->v, M, 0, M, nullptr, 0, 0, a_is_param};
    GemmEpilogue e{EPI_ACCUM, y->v, K, nullptr, 0, 0.f, nullptr, 0, 0};
    return dyb200_gemm_fused(ctx, K, N * y->bd, 1, &p, e);
  }
  for (uint32_t b = 0; b < max_b; ++b) {
    GemmPair p{batch_ptr(l, b), M, 1, batch_ptr(r, b), M, 0, M, nullptr, 0, 0, 0};
    GemmEpilogue e{EPI_ACCUM, y->v + (size_t)(b % y->bd) * K * N, K, nullptr, 0, 0.f, nullptr, 0, 0};
    int rc = dyb200_gemm_fused(ctx, K, N, 1, &p, e);
    if (rc) return rc;
  }
  return DYB200_OK;
}

// y += l * r^T   (l: M x N, r: K x N, y: M x K)
int mm_transp_r_acc(dyb200_ctx* ctx, const dyb200_tensor* l, const dyb200_tensor* r, dyb200_tensor* y) {
  const uint32_t M = t_rows(l), N = t_cols(l), K = t_rows(r);
  const uint32_t max_b = l->bd > r->bd ? l->bd : r->bd;
  if (y->bd == 1 && l->bd == r->bd) {
    GemmPair p{l->v, M, 0, r->v, K, 1, N * l->bd, nullptr, 0, 0, 0};
    GemmEpilogue e{EPI_ACCUM, y->v, M, nullptr, 0, 0.f, nullptr, 0, 0};
    return dyb200_gemm_fused(ctx, M, K, 1, &p, e);
  }
  for (uint32_t b = 0; b < max_b; ++b) {
    GemmPair p{batch_ptr(l, b), M, 0, batch_ptr(r, b), K, 1, N, nullptr, 0, 0, 0};
    GemmEpilogue e{EPI_ACCUM, y->v + (size_t)(b % y->bd) * M * K, M, nullptr, 0, 0.f, nullptr, 0, 0};
    int rc = dyb200_gemm_fused(ctx, M, K, 1, &p, e);
    if (rc) return rc;
  }
  return DYB200_OK;
}

int check_product(dyb200_ctx* ctx, const dyb200_tensor* l, const dyb200_tensor* r, const dyb200_tensor* y, const char* what) {
  int rc;
  if ((rc = check_matrix(ctx, l, what)) || (rc = check_matrix(ctx, r, what)) || (rc = check_matrix(ctx, y, what))) return rc;
  DYB_CHECK_ARG(ctx, t_cols(l) == t_rows(r), "%s: mismatched input dimensions (%u columns times %u rows)", what, t_cols(l), t_rows(r));
  DYB_CHECK_ARG(ctx, t_rows(y) == t_rows(l) && t_cols(y) == t_cols(r), "%s: bad output dimensions", what);
  // an AffineTransform result may have more batch elements than both operands of one of its products
  DYB_CHECK_ARG(ctx, (l->bd == 1 || l->bd == y->bd) && (r->bd == 1 || r->bd == y->bd),
                "%s: mismatched batch sizes %u, %u -> %u", what, l->bd, r->bd, y->bd);
  return DYB200_OK;
}

unsigned attr_flags(const void* attrs) { return attrs ? static_cast<const dyb200_affine_attrs*>(attrs)->flags : 0u; }

}  // namespace

extern "C" {

int dyb200_matmul_fwd(DYB200_FWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs == 2, "MatrixMultiply: failed input count check");
  int rc = check_product(ctx, &xs[0], &xs[1], fx, "MatrixMultiply");
  if (rc) return rc;
  return mm_fwd(ctx, &xs[0], &xs[1], fx, EPI_STORE, nullptr, (attr_flags(attrs) & DYB200_GEMM_A_IS_PARAM) ? 1 : 0);
}

int dyb200_matmul_bwd(DYB200_BWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)aux_mem; (void)fx;
  DYB_CHECK_ARG(ctx, nxs == 2 && i < 2, "MatrixMultiply: failed dimension check in backward");
  int rc = check_product(ctx, &xs[0], &xs[1], dEdf, "MatrixMultiply");
  if (rc) return rc;
  DYB_CHECK_ARG(ctx, dEdxi && dEdxi->v && t_batch_size(dEdxi) == t_batch_size(&xs[i]) && dEdxi->bd == xs[i].bd,
                "MatrixMultiply: gradient shape differs from argument %u", i);
  if (i == 0) return mm_transp_r_acc(ctx, dEdf, &xs[1], dEdxi);
  return mm_transp_l_acc(ctx, &xs[0], dEdf, dEdxi, (attr_flags(attrs) & DYB200_GEMM_A_IS_PARAM) ? 1 : 0);
}

int dyb200_affine_transform_fwd(DYB200_FWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)aux_mem;
  DYB_CHECK_ARG(ctx, nxs >= 1 && (nxs - 1) % 2 == 0, "AffineTransform: bad number of inputs (%d)", nxs);
  DYB_CHECK_ARG(ctx, fx && fx->v && xs[0].v, "AffineTransform: null tensor");
  const size_t b_size = t_size(&xs[0]), fx_size = t_size(fx);
  if (nxs == 1) {
    DYB_CHECK_ARG(ctx, b_size == fx_size, "AffineTransform: bad output dimensions");
    DYB_CUDA(ctx, cudaMemcpyAsync(fx->v, xs[0].v, fx_size * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    return DYB200_OK;
  }
  for (int k = 1; k < nxs; k += 2) {
    int rc = check_product(ctx, &xs[k], &xs[k + 1], fx, "AffineTransform");
    if (rc) return rc;
  }
  DYB_CHECK_ARG(ctx, t_rows(&xs[0]) == t_rows(fx) && b_size > 0 && fx_size % b_size == 0 && (b_size == fx_size || xs[0].bd == 1),
                "AffineTransform: broadcasting over columns with mini-batched inputs is not implemented yet");
  const int a_is_param = (attr_flags(attrs) & DYB200_GEMM_A_IS_PARAM) ? 1 : 0;
  int first = 1;
  if (b_size == t_rows(fx) && xs[0].bd == 1) {
    // column-vector bias: added in the epilogue of the first product
    int rc = mm_fwd(ctx, &xs[1], &xs[2], fx, EPI_BIAS, xs[0].v, a_is_param);
    if (rc) return rc;
    first = 3;
  } else if (b_size == fx_size) {
    DYB_CUDA(ctx, cudaMemcpyAsync(fx->v, xs[0].v, fx_size * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
  } else {
    const int vec = b_size % 4 == 0 && aligned16(xs[0].v) && aligned16(fx->v);
    dyb_launch(k_tile_copy, stream_grid(ctx, fx_size / 4 + 1, kThreads), kThreads, 0, ctx, xs[0].v, b_size, fx->v, fx_size, vec);
    DYB_LAUNCHED(ctx);
  }
  for (int k = first; k < nxs; k += 2) {
    int rc = mm_fwd(ctx, &xs[k], &xs[k + 1], fx, EPI_ACCUM, nullptr, a_is_param);
    if (rc) return rc;
  }
  return DYB200_OK;
}

int dyb200_affine_transform_bwd(DYB200_BWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)aux_mem; (void)fx;
  DYB_CHECK_ARG(ctx, nxs >= 1 && (nxs - 1) % 2 == 0 && (int)i < nxs, "AffineTransform: failed boundary check in backward");
  DYB_CHECK_ARG(ctx, dEdf && dEdf->v && dEdxi && dEdxi->v, "AffineTransform: null tensor");
  DYB_CHECK_ARG(ctx, t_batch_size(dEdxi) == t_batch_size(&xs[i]) && dEdxi->bd == xs[i].bd,
                "AffineTransform: gradient shape differs from argument %u", i);
  if (i == 0) {
    const size_t dx_size = t_size(dEdxi), df_size = t_size(dEdf);
    if (dx_size == df_size) {
      const int vec = dx_size % 4 == 0 && aligned16(dEdf->v) && aligned16(dEdxi->v);
      dyb_launch(k_add_into, stream_grid(ctx, dx_size / 4 + 1, kThreads), kThreads, 0, ctx, dEdf->v, dEdxi->v, dx_size, vec);
      DYB_LAUNCHED(ctx);
      return DYB200_OK;
    }
    DYB_CHECK_ARG(ctx, dEdxi->bd == 1 && dx_size > 0 && df_size % dx_size == 0,
                  "AffineTransform: broadcasting over columns with mini-batched inputs is not implemented yet");
    return batch_reduce_add(ctx, ChunkOf{dEdf->v, dx_size}, dx_size, (uint32_t)(df_size / dx_size), dEdxi->v);
  }
  const int k = (i % 2 == 1) ? (int)i : (int)i - 1;   // index of the left operand of this product
  int rc = check_product(ctx, &xs[k], &xs[k + 1], dEdf, "AffineTransform");
  if (rc) return rc;
  if (i % 2 == 1) return mm_transp_r_acc(ctx, dEdf, &xs[i + 1], dEdxi);
  return mm_transp_l_acc(ctx, &xs[i - 1], dEdf, dEdxi, (attr_flags(attrs) & DYB200_GEMM_A_IS_PARAM) ? 1 : 0);
}

}  // extern "C"
