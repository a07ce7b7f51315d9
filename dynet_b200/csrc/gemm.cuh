// Internal GEMM interface shared by the LSTM nodes and dyb200_gemm.
//   C[M x N] = epilogue( sum_p op(A_p)[M x K_p] * (op(B_p) .* mask_p)[K_p x N] )
// All matrices are column-major fp32.  Up to two (A, B) pairs accumulate into the same
// tile, which is how the gate pre-activation Wx*x + Wh*h is formed in one kernel.
#pragma once
#include "common.cuh"

struct GemmPair {
  const float* A; uint32_t lda; int transA;   // op(A)(m,k) = transA ? A[k + lda*m] : A[m + lda*k]
  const float* B; uint32_t ldb; int transB;   // op(B)(k,n) = transB ? B[n + ldb*k] : B[k + ldb*n]
  uint32_t K;
  // optional multiplicative mask on B, indexed like B's storage: element at (row r, col c)
  // of the stored matrix uses mask[r + (mask_full ? mask_ld * c : 0)]  (dropout masks, bd 1 or B)
  const float* maskB; uint32_t mask_ld; int mask_full;
  int a_is_param;   // A is a parameter matrix: its packed form may be kept in the context's parameter cache
};

enum GemmEpiMode {
  EPI_STORE = 0,      // C = acc
  EPI_ACCUM = 1,      // C += acc
  EPI_GATES = 2,      // C = act(acc + bias[m] + (H <= m < 2H ? forget_bias : 0)); sigmoid for m < 3H, tanh above
  EPI_ACCUM_MASK = 3, // C += acc * maskC[m + (maskc_full ? maskc_ld * n : 0)]
  EPI_BIAS = 4        // C = acc + bias[m]   (column vector broadcast over the N columns)
};

struct GemmEpilogue {
  int mode;
  float* C; uint32_t ldc;
  const float* bias; uint32_t H; float forget_bias;
  const float* maskC; uint32_t maskc_ld; int maskc_full;
};

// fp32 CUDA-core path: any shape, any alignment.
int dyb200_gemm_simt(dyb200_ctx* ctx, uint32_t M, uint32_t N, int npairs, const GemmPair* pairs, const GemmEpilogue& epi);
// 3xTF32 tensor-pipe path (tcgen05 + TMEM + TMA); returns DYB200_ERUNTIME with *handled = 0
// when the shape/alignment is outside what it supports.
int dyb200_gemm_tc(dyb200_ctx* ctx, uint32_t M, uint32_t N, int npairs, const GemmPair* pairs, const GemmEpilogue& epi,
                   int* handled);
// Dispatcher: tensor path when eligible, else the CUDA-core path.
int dyb200_gemm_fused(dyb200_ctx* ctx, uint32_t M, uint32_t N, int npairs, const GemmPair* pairs, const GemmEpilogue& epi);

// ---- pieces of the tensor path, for entry points that reuse one packed operand in several products ----
struct PackedOp { float* hi; float* lo; uint32_t rows, K, pitch; };   // K-major TF32 hi / lo planes
// Packs `rows x K` (element (r, k) at src[k + ld*r] when k_is_fast, else src[r + ld*k]) times an optional mask
// into planes taken from the scratch arena (valid until the current entry point returns).
int dyb200_tc_pack(dyb200_ctx* ctx, const float* src, uint32_t ld, bool k_is_fast, uint32_t rows, uint32_t K,
                   const float* mask, uint32_t mask_ld, int mask_full, PackedOp* out);
// Same for a parameter matrix: served from the parameter cache when it is on.
int dyb200_tc_param(dyb200_ctx* ctx, const float* src, uint32_t ld, bool k_is_fast, uint32_t rows, uint32_t K, PackedOp* out);
int dyb200_tc_gemm_packed(dyb200_ctx* ctx, uint32_t M, uint32_t N, int npairs, const PackedOp* A, const PackedOp* B,
                          const GemmEpilogue& epi);
bool dyb200_tc_eligible(uint32_t M, uint32_t N, double flops);
struct dyb200_wgrad;
