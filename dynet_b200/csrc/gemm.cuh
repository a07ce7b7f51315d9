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
  EPI_BIAS = 4,       // C = acc + bias[m]   (column vector broadcast over the N columns)
  // The A operand was packed with interleaved gate rows (dyb200_tc_param_gates): tile t, row 32 q + l is gate q
  // (i, f, o, g) of hidden unit u = 32 t + l.  gates[q H + u, n] = act(acc + bias + forget bias) as in EPI_GATES,
  // then c_out[u, n] = i g + f c_prev[u, n] and h_out[u, n] = o tanh(c) (VanillaLSTMC / VanillaLSTMH forward).
  EPI_LSTM_CELL = 5
};

struct GemmEpilogue {
  int mode;
  float* C; uint32_t ldc;
  const float* bias; uint32_t H; float forget_bias;
  const float* maskC; uint32_t maskc_ld; int maskc_full;
  // Optional second destination: rows m >= split_m go to C2 (row m - split_m) with their own leading dimension and
  // mask; split_m = 0 disables it.  Lets one product with stacked A operands ([Wx; Wh]^T) feed two tensors.
  uint32_t split_m = 0;
  float* C2 = nullptr; uint32_t ldc2 = 0;
  const float* maskC2 = nullptr; uint32_t maskc2_ld = 0; int maskc2_full = 0;
  // EPI_LSTM_CELL only: previous cell state and the two outputs, all H x N with leading dimension H
  const float* c_prev = nullptr; float* c_out = nullptr; float* h_out = nullptr;
  // EPI_LSTM_CELL, optional: h .* hmask also goes out as split operand planes (row = batch column, H values each): the
  // K-major right operand of the next time step's gate product and, read MN-major, the right operand of the layer's
  // weight-gradient product.  16-byte aligned, H % 4 == 0.
  float* hn_hi = nullptr; float* hn_lo = nullptr; uint32_t hn_pitch = 0;
  const float* hmask = nullptr; uint32_t hmask_ld = 0; int hmask_full = 0;
};
#ifdef __CUDACC__
// h .* mask of four hidden units [u, u + 4) of batch column n, written as operand planes (see GemmEpilogue::hn_hi).
__device__ __forceinline__ void epi_emit_h(const GemmEpilogue& epi, uint32_t u, uint32_t n, float4 h) {
  if (epi.hmask) {
    const float4 mk = *reinterpret_cast<const float4*>(epi.hmask + u + (epi.hmask_full ? (size_t)epi.hmask_ld * n : 0));
    h.x *= mk.x; h.y *= mk.y; h.z *= mk.z; h.w *= mk.w;
  }
  float4 hi, lo;
  split_tf32(h.x, hi.x, lo.x); split_tf32(h.y, hi.y, lo.y); split_tf32(h.z, hi.z, lo.z); split_tf32(h.w, hi.w, lo.w);
  *reinterpret_cast<float4*>(epi.hn_hi + (size_t)n * epi.hn_pitch + u) = hi;
  *reinterpret_cast<float4*>(epi.hn_lo + (size_t)n * epi.hn_pitch + u) = lo;
}
#endif
// Row m of the product -> destination pointer of column 0, leading dimension and mask of that row.
struct EpiRow { float* c; uint32_t ldc; const float* mask; uint32_t mask_ld; int mask_full; };
__host__ __device__ inline EpiRow epi_row(const GemmEpilogue& e, uint32_t m) {
  if (e.split_m && m >= e.split_m) {
    const uint32_t r = m - e.split_m;
    return EpiRow{e.C2 + r, e.ldc2, e.maskC2 ? e.maskC2 + r : nullptr, e.maskc2_ld, e.maskc2_full};
  }
  return EpiRow{e.C + m, e.ldc, e.maskC ? e.maskC + m : nullptr, e.maskc_ld, e.maskc_full};
}

// fp32 CUDA-core path: any shape, any alignment.
int dyb200_gemm_simt(dyb200_ctx* ctx, uint32_t M, uint32_t N, int npairs, const GemmPair* pairs, const GemmEpilogue& epi);
// 3xTF32 tensor-pipe path (tcgen05 + TMEM + TMA); returns DYB200_ERUNTIME with *handled = 0
// when the shape/alignment is outside what it supports.
int dyb200_gemm_tc(dyb200_ctx* ctx, uint32_t M, uint32_t N, int npairs, const GemmPair* pairs, const GemmEpilogue& epi,
                   int* handled);
// Dispatcher: tensor path when eligible, else the CUDA-core path.
int dyb200_gemm_fused(dyb200_ctx* ctx, uint32_t M, uint32_t N, int npairs, const GemmPair* pairs, const GemmEpilogue& epi);

// ---- pieces of the tensor path, for entry points that reuse one packed operand in several products ----
// TF32 hi / lo planes of an operand: `rows` rows (m or n) of K values.  K-major (mn_major = 0): element (r, k) at
// plane[r * pitch + k].  MN-major (left operands of dyb200_tc_gemm_packed only): element (r, k) at plane[k * pitch + r] -
// the K-major planes of the transposed matrix, used as they are.
struct PackedOp { float* hi; float* lo; uint32_t rows, K, pitch; uint32_t mn_major = 0; };
// A queue of packing work that one kernel launch executes (several small operands per launch).
constexpr int kMaxPackJobs = 8;
constexpr int kLayoutGates = 2;
struct PackJob {
  const float* src; const float* mask; float* hi; float* lo;
  uint32_t ld, rows, K, mask_ld, pitch, gx, perm_H;
  uint32_t mask_period;   // > 0: a full mask repeats every mask_period batch columns (one mask for every time step of a sequence)
  int k_is_fast, mask_full, vec;
};
struct PackJobs { PackJob job[kMaxPackJobs]; uint32_t start[kMaxPackJobs + 1]; int n; };
inline void dyb200_tc_pack_begin(PackJobs* b) { b->n = 0; b->start[0] = 0; }
int dyb200_tc_pack_flush(dyb200_ctx* ctx, PackJobs* batch);
// Packs `rows x K` (element (r, k) at src[k + ld*r] when k_is_fast, else src[r + ld*k]) times an optional mask
// into planes taken from the scratch arena (valid until the current entry point returns).  With a batch the work is
// only queued: the planes are filled when the batch is flushed.
int dyb200_tc_pack(dyb200_ctx* ctx, const float* src, uint32_t ld, bool k_is_fast, uint32_t rows, uint32_t K,
                   const float* mask, uint32_t mask_ld, int mask_full, PackedOp* out, PackJobs* batch = nullptr);
// Same for a parameter matrix: served from the parameter cache when it is on.
int dyb200_tc_param(dyb200_ctx* ctx, const float* src, uint32_t ld, bool k_is_fast, uint32_t rows, uint32_t K, PackedOp* out);
// A gate weight matrix (rows = 4H, element (r, k) at src[r + ld * k]) with its rows interleaved for EPI_LSTM_CELL.
int dyb200_tc_param_gates(dyb200_ctx* ctx, const float* src, uint32_t ld, uint32_t rows, uint32_t K, PackedOp* out);
// Number of K splits dyb200_tc_gemm_packed will use for this shape (1 = the epilogue runs in the MMA kernel).
uint32_t dyb200_tc_splits(const dyb200_ctx* ctx, uint32_t M, uint32_t N, uint32_t kb_total);
// Two parameter matrices with the same K and leading dimension stacked along the rows: rows [0, rows) from src,
// rows [rows, rows + rows2) from src2.
int dyb200_tc_param2(dyb200_ctx* ctx, const float* src, uint32_t rows, const float* src2, uint32_t rows2, uint32_t ld,
                     bool k_is_fast, uint32_t K, PackedOp* out);
// force_splits > 0: that many K splits (normalised so that no split is empty) instead of the cost model's choice.
int dyb200_tc_gemm_packed(dyb200_ctx* ctx, uint32_t M, uint32_t N, int npairs, const PackedOp* A, const PackedOp* B,
                          const GemmEpilogue& epi, uint32_t force_splits = 0);
int dyb200_splitk_reduce(dyb200_ctx* ctx, const float* part, uint32_t S, uint32_t M, uint32_t N, const GemmEpilogue& epi);
// Tiling of the backward recurrence of an LSTM layer (dx_t, dh_{t-1} += [Wx; Wh]^T dgates_t), shared by the per-step call
// and the sequence kernel so that both add the same partial sums: tile width, batch-column blocks per CTA of the sequence
// kernel (1 or 2) and K splits.  False when the shape does not suit the sequence kernel (the per-step call then lets the
// cost model choose).
struct LstmBwdTiling { uint32_t bn, ncb, S; };
bool dyb200_lstm_bwd_tiling(const dyb200_ctx* ctx, uint32_t I, uint32_t H, uint32_t B, LstmBwdTiling* out);
bool dyb200_tc_eligible(uint32_t M, uint32_t N, double flops);
// Planes of `rows x K` taken from the scratch arena, left for the caller's kernel to fill.
int dyb200_tc_planes(dyb200_ctx* ctx, uint32_t rows, uint32_t K, PackedOp* out);
struct dyb200_wgrad;
// The accumulator's A planes (dgates of all columns) are MN-major: one row of `pitch` floats per column, M values each.  The
// reserve calls hand out the rows of k columns for the caller's kernel to fill (a_hi / a_lo point at the first of them);
// the same rows are a K-major right operand (rows = columns, K = M) for the caller's own products.
int dyb200_wgrad_reserve(dyb200_wgrad* w, uint32_t k, float** a_hi, float** a_lo, uint32_t* pitch, const float* b0, uint32_t ldb0,
                         const float* mask0, int mask0_full, const float* b1, uint32_t ldb1, const float* mask1, int mask1_full,
                         dyb200_ctx* ctx, PackJobs* batch);
int dyb200_wgrad_push_b_at(dyb200_wgrad* w, uint32_t col, uint32_t k, const float* b0, uint32_t ldb0, const float* mask0, int mask0_full,
                           const float* b1, uint32_t ldb1, const float* mask1, int mask1_full, dyb200_ctx* ctx, PackJobs* batch);
int dyb200_wgrad_reserve_a_at(dyb200_wgrad* w, uint32_t col, uint32_t k, float** a_hi, float** a_lo, uint32_t* pitch, dyb200_ctx* ctx);
int dyb200_wgrad_pack_a_at(dyb200_wgrad* w, uint32_t col, uint32_t k, const float* a, uint32_t lda, dyb200_ctx* ctx, PackJobs* batch);
uint32_t dyb200_wgrad_rows(const dyb200_wgrad* w);
// Pre-split sequence inputs (dyb200_wgrad_pack_inputs): the forward operand planes of the step that starts at column `col`,
// when they are available.  x: rows [col, col + k) of the planes filled by dyb200_wgrad_pack_inputs; h: the planes the
// previous step's LSTM epilogue wrote for this column.  Return false when the caller has to split that input itself.
bool dyb200_wgrad_x_planes(const dyb200_wgrad* w, uint32_t col, uint32_t k, PackedOp* out);
bool dyb200_wgrad_h_planes(const dyb200_wgrad* w, uint32_t col, uint32_t k, PackedOp* out);
// Destinations for the split planes of the NEXT step's h input (the step that starts at column col + k), or false when
// there is no next step or the inputs were not pre-split.  Marks those planes as the h input of column col + k.
bool dyb200_wgrad_next_h(dyb200_wgrad* w, uint32_t col, uint32_t k, GemmEpilogue* epi);
uint32_t dyb200_wgrad_fill(const dyb200_wgrad* w);
int dyb200_wgrad_push_batched(dyb200_wgrad* w, uint32_t k, const float* a, uint32_t lda, const float* b0, uint32_t ldb0,
                              const float* mask0, int mask0_full, const float* b1, uint32_t ldb1, const float* mask1,
                              int mask1_full, dyb200_ctx* ctx, PackJobs* batch);

// ---- sequence kernels (lstm_seq.cu) ----
// Operand planes of a whole sequence held by an accumulator after dyb200_wgrad_pack_inputs: X = x .* mask_x (row = column
// of the sequence, K = I), Hs = h_tm1 .* mask_h (row = column, K = H; rows [c, c + step) are the input of the step that
// starts at column c).  False when they are not in place for `steps` steps of `step` columns.
struct SeqPlanes { PackedOp X, Hs; };
bool dyb200_wgrad_seq_planes(const dyb200_wgrad* w, uint32_t steps, uint32_t step, SeqPlanes* out);
int dyb200_wgrad_seq_h0(dyb200_wgrad* w, const float* h0, const float* mh, int mh_full, dyb200_ctx* ctx, PackJobs* batch);
void dyb200_wgrad_seq_done(dyb200_wgrad* w);
// A 2-D tensor map (CUtensorMap, 128 bytes at `map`) over a K-major plane: box = 32 floats of K x box_rows rows, 128-byte swizzle.
int dyb200_tc_make_tmap(dyb200_ctx* ctx, void* map, float* plane, uint32_t rows, uint32_t K, uint32_t pitch, uint32_t box_rows);
uint32_t dyb200_tc_tile_cols(uint32_t N);   // width of the output tile the tensor path uses for N columns (64 or 128)
