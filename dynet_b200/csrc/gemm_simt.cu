// fp32 CUDA-core GEMM: the any-shape fallback behind dyb200_gemm_fused, and the dispatcher.
// 64x64 output tile per CTA, K step 16, 4x4 register micro-tile per thread.
#include "gemm.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__device__ __forceinline__ float load_a(const GemmPair& p, uint32_t m, uint32_t k, uint32_t M) {
  if (m >= M || k >= p.K) return 0.f;
  return p.transA ? p.A[k + (size_t)p.lda * m] : p.A[m + (size_t)p.lda * k];
}
__device__ __forceinline__ float load_b(const GemmPair& p, uint32_t k, uint32_t n, uint32_t N) {
  if (n >= N || k >= p.K) return 0.f;
  uint32_t r = p.transB ? n : k, c = p.transB ? k : n;
  float v = p.B[r + (size_t)p.ldb * c];
  if (p.maskB) v *= p.maskB[r + (p.mask_full ? (size_t)p.mask_ld * c : 0)];
  return v;
}

// gridDim.z > 1 (one pair only): split z covers k in [z kc, (z + 1) kc) and stores its partial product at epi.C + z M N
// (epi is then a plain store with leading dimension M); dyb200_splitk_reduce adds the splits and applies the real epilogue.
__global__ void __launch_bounds__(256) k_gemm_simt(uint32_t M, uint32_t N, int npairs, GemmPair p0, GemmPair p1,
                                                  GemmEpilogue epi, uint32_t kc) {
  dyb_grid_dep_sync();
  if (gridDim.z > 1) epi.C += (size_t)blockIdx.z * M * N;
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const uint32_t m0 = blockIdx.x * TM, n0 = blockIdx.y * TN;
  float acc[4][4] = {};
  for (int pi = 0; pi < npairs; ++pi) {
    const GemmPair& p = pi == 0 ? p0 : p1;
    const uint32_t k_lo = gridDim.z > 1 ? blockIdx.z * kc : 0u, k_hi = gridDim.z > 1 ? min(p.K, k_lo + kc) : p.K;
    for (uint32_t k0 = k_lo; k0 < k_hi; k0 += TK) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (p.transA) { int k = tid % 16, m = tid / 16 + 16 * j; As[k][m] = load_a(p, m0 + m, k0 + k, M); }
        else { int m = tid % 64, k = tid / 64 + 4 * j; As[k][m] = load_a(p, m0 + m, k0 + k, M); }
        if (p.transB) { int n = tid % 64, k = tid / 64 + 4 * j; Bs[k][n] = load_b(p, k0 + k, n0 + n, N); }
        else { int k = tid % 16, n = tid / 16 + 16 * j; Bs[k][n] = load_b(p, k0 + k, n0 + n, N); }
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < TK; ++k) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { a[i] = As[k][tx * 4 + i]; b[i] = Bs[k][ty * 4 + i]; }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t n = n0 + ty * 4 + j;
    if (n >= N) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t m = m0 + tx * 4 + i;
      if (m >= M) continue;
      float* c = epi.C + m + (size_t)epi.ldc * n;
      float v = acc[i][j];
      if (epi.mode == EPI_STORE) *c = v;
      else if (epi.mode == EPI_BIAS) *c = v + epi.bias[m];
      else if (epi.mode == EPI_ACCUM) *c += v;
      else if (epi.mode == EPI_GATES) {
        v += epi.bias[m];
        if (m >= epi.H && m < 2 * epi.H) v += epi.forget_bias;
        *c = m < 3 * epi.H ? gate_sigmoid(v) : gate_tanh(v);
      } else {
        *c = __fmaf_rn(v, epi.maskC[m + (epi.maskc_full ? (size_t)epi.maskc_ld * n : 0)], *c);
      }
    }
  }
}

}  // namespace

int dyb200_gemm_simt(dyb200_ctx* ctx, uint32_t M, uint32_t N, int npairs, const GemmPair* pairs, const GemmEpilogue& epi) {
  if (M == 0 || N == 0) return DYB200_OK;
  GemmPair p0 = pairs[0], p1 = npairs > 1 ? pairs[1] : pairs[0];
  dim3 grid((M + TM - 1) / TM, (N + TN - 1) / TN);
  DYB_CHECK_ARG(ctx, grid.y <= 65535, "gemm: N too large for the CUDA-core path");
  // A long reduction over a handful of tiles (the last time steps of a ragged batch: 128 x 21 x 1024 on two CTAs took
  // 190 us) is split along K: up to 32 splits of at least 64 k each, partial products to scratch, added in split order.
  const uint32_t K = pairs[0].K;
  if (npairs == 1 && grid.x * grid.y <= 16 && K >= 256 && epi.mode != EPI_GATES) {
    uint32_t S = K / 64;
    if (S > 32) S = 32;
    uint32_t kc = ((K + S - 1) / S + TK - 1) / TK * TK;   // whole k steps per split
    S = (K + kc - 1) / kc;
    void* part;
    int rc = dyb200_scratch(ctx, (size_t)S * M * N * sizeof(float), &part);
    if (rc) return rc;
    GemmEpilogue store{EPI_STORE, (float*)part, M, nullptr, 0, 0.f, nullptr, 0, 0};
    grid.z = S;
    dyb_launch(k_gemm_simt, grid, 256, 0, ctx, M, N, npairs, p0, p1, store, kc);
    DYB_LAUNCHED(ctx);
    return dyb200_splitk_reduce(ctx, (const float*)part, S, M, N, epi);
  }
  dyb_launch(k_gemm_simt, grid, 256, 0, ctx, M, N, npairs, p0, p1, epi, 0u);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_gemm_fused(dyb200_ctx* ctx, uint32_t M, uint32_t N, int npairs, const GemmPair* pairs, const GemmEpilogue& epi) {
  double flops = 0;
  for (int p = 0; p < npairs; ++p) flops += 2.0 * M * N * pairs[p].K;
  int handled = 0;
  int rc = dyb200_gemm_tc(ctx, M, N, npairs, pairs, epi, &handled);
  if (handled) return rc;
  GemmProfScope scope(ctx, flops, 0, M, N, pairs[0].K + (npairs > 1 ? pairs[1].K : 0), (uint32_t)epi.mode);
  return dyb200_gemm_simt(ctx, M, N, npairs, pairs, epi);
}

extern "C" int dyb200_gemm(int transA, int transB, uint32_t M, uint32_t N, uint32_t K, const float* A, uint32_t lda,
                           const float* B, uint32_t ldb, float* C, uint32_t ldc, int accumulate, unsigned flags,
                           dyb200_ctx* ctx) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  DYB_CHECK_ARG(ctx, A && B && C, "gemm: null pointer");
  DYB_CHECK_ARG(ctx, lda >= (transA ? K : M) && ldb >= (transB ? N : K) && ldc >= M, "gemm: leading dimension too small");
  GemmPair p{A, lda, transA, B, ldb, transB, K, nullptr, 0, 0, (flags & DYB200_GEMM_A_IS_PARAM) ? 1 : 0};
  GemmEpilogue e{accumulate ? EPI_ACCUM : EPI_STORE, C, ldc, nullptr, 0, 0.f, nullptr, 0, 0};
  return dyb200_gemm_fused(ctx, M, N, 1, &p, e);
}
