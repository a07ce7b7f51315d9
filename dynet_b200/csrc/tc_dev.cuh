// Device-side building blocks of the 3xTF32 tensor-pipe kernels (tcgen05 / TMEM / TMA), shared by the GEMM kernels
// (gemm_tc.cu) and the sequence-persistent LSTM kernels (lstm_seq.cu): tile constants, mbarrier / TMA / tcgen05 wrappers, the
// 12 MMAs of a k-block, and the cooperative epilogue pass over a tile parked in shared memory.
#pragma once
#include <cuda.h>
#include <math.h>

#include "gemm.cuh"

namespace {


constexpr int BM = 128, BN = 128, BK = 32, STAGES = 3;
constexpr int TILE_BYTES = BM * BK * 4;          // 16 KiB, rows of 128 bytes
constexpr int STAGE_BYTES = 4 * TILE_BYTES;      // A_hi, A_lo, B_hi, B_lo
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;   // + slack to align the ring to 1 KiB
constexpr int kThreads = 320;              // TMA warp, MMA warp, 8 epilogue warps
constexpr uint32_t kWaitLimit = 1u << 20;
constexpr uint32_t kTmemCols = 256;       // two 128-column accumulators, used alternately       // two 128-column accumulators, used alternately
// k-blocks accumulated in TMEM before the sum moves to registers.  Measured against a float64 product (randn operands,
// worst element / rms of the result): one unbroken chain 1.9e-5 at K = 2048 and 1.6e-4 at K = 17920 (biased towards
// zero); chains of 8 k-blocks 8.7e-6 at both, against 2.6e-6 .. 9.3e-6 for cuBLAS SGEMM.  Each flush costs about
// 0.4 us of tensor-pipe time (4 % at this setting).
constexpr uint32_t kChunkKB = 8;
constexpr uint32_t kEpiWarps = 8;

// pair p: t[4p] = A_hi, A_lo, B_hi, B_lo.  a_mn != 0 (one pair only): the A planes are MN-major - element (m, k) at
// plane[k * pitch + m], the layout of a K x M row-major matrix - and t[0], t[1] are 3-D maps over (m within a group of 32,
// k, group) with a box of 32 x 32 x 4; see load_a_tile / umma_desc_mn.  b_mn: the same for the B planes (t[2], t[3]; the
// box holds as many groups as the tile has columns / 32).
struct TmapPack { CUtensorMap t[8]; uint32_t a_mn, b_mn; };

// The k-blocks of K split z of S: [b0, b0 + n0) of pair 0, then [b1, b1 + n1) of pair 1 (each pair cut into S equal shares).
struct KSplit { uint32_t b0, n0, b1, n1; };
__device__ __forceinline__ KSplit k_split(uint32_t kb0, uint32_t kb1, uint32_t z, uint32_t S) {
  const uint32_t per0 = (kb0 + S - 1) / S, per1 = (kb1 + S - 1) / S;
  KSplit k;
  k.b0 = min(z * per0, kb0); k.n0 = min(k.b0 + per0, kb0) - k.b0;
  k.b1 = min(z * per1, kb1); k.n1 = min(k.b1 + per1, kb1) - k.b1;
  return k;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done = 0;
  for (uint32_t it = 0; it < kWaitLimit; ++it) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                        // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                        // layout: SWIZZLE_128B
  return d;
}
// Same for an MN-major A tile of 128 m x 32 k as load_a_tile lays it out: four groups of 32 m (128 bytes) x 32 k rows, 4096
// bytes apart (the leading byte offset = distance between 32-element groups along m).  32-bit MN-major operands exist in
// one shared-memory layout only, the 128-byte swizzle with 32-byte atoms (layout type 1; the tensor map's
// SWIZZLE_128B_ATOM_32B): its pattern repeats every 4 k rows, so the stride byte offset - the distance between 4-k groups -
// is 512 bytes, and one MMA (k = 8) advances the start address by 1024 bytes.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(4096 >> 4) << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)1 << 61;
  return d;
}
// One plane of the A tile (m0 .., k-block kblk) into `st`: one box of 16 KB in either layout (MN-major: the box's innermost
// extent is one 128-byte swizzle span = 32 m, its outermost the four groups of the tile).  k rows past the plane's extent
// arrive as zeros.
__device__ __forceinline__ void load_a_tile(unsigned char* st, const CUtensorMap* map, uint64_t* bar, uint32_t kblk, uint32_t m0,
                                            uint32_t a_mn) {
  if (a_mn) {
    tma_load_3d(st, map, bar, 0, (int)(kblk * 32), (int)(m0 / 32));
  } else {
    tma_load_2d(st, map, bar, (int)(kblk * 32), (int)m0);
  }
}
__device__ __forceinline__ void load_b_tile(unsigned char* st, const CUtensorMap* map, uint64_t* bar, uint32_t kblk, uint32_t n0,
                                            uint32_t b_mn) {
  if (b_mn) tma_load_3d(st, map, bar, 0, (int)(kblk * 32), (int)(n0 / 32));
  else tma_load_2d(st, map, bar, (int)(kblk * 32), (int)n0);
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// The 12 MMAs of one 32-wide k-block (3 products x 4 k-steps of 8) as one block of PTX.  The first MMA accumulates iff
// `accumulate` is non-zero (0 opens a new accumulation chain).  a_step: what one k-step adds to the A descriptors, in
// descriptor units of 16 bytes (2 = 32 bytes of a K-major row; 64 = one 8-k group of an MN-major tile); b_step: the same
// for the B descriptors.
__device__ __forceinline__ void issue_kblock(uint32_t acc, uint64_t a_hi, uint64_t a_lo, uint64_t b_hi, uint64_t b_lo,
                                             uint32_t idesc, uint32_t accumulate, uint64_t a_step = 2, uint64_t b_step = 2) {
  // one MMA consumes 8 tf32 = 32 bytes of K: +2 in descriptor units per k8 step of a K-major operand
  asm volatile(
      "{\n\t.reg .pred pf, pt;\n\t.reg .b64 xa, xb, ya, yb;\n\t"
      "setp.ne.b32 pf, %6, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %2, %3, %5, pf;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %4, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %3, %5, pt;\n\t"
      "add.s64 xa, %1, %7;\n\tadd.s64 xb, %2, %7;\n\tadd.s64 ya, %3, %8;\n\tadd.s64 yb, %4, %8;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], xb, ya, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], xa, yb, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], xa, ya, %5, pt;\n\t"
      "add.s64 xa, xa, %7;\n\tadd.s64 xb, xb, %7;\n\tadd.s64 ya, ya, %8;\n\tadd.s64 yb, yb, %8;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], xb, ya, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], xa, yb, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], xa, ya, %5, pt;\n\t"
      "add.s64 xa, xa, %7;\n\tadd.s64 xb, xb, %7;\n\tadd.s64 ya, ya, %8;\n\tadd.s64 yb, yb, %8;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], xb, ya, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], xa, yb, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], xa, ya, %5, pt;\n\t}"
      ::"r"(acc), "l"(a_hi), "l"(a_lo), "l"(b_hi), "l"(b_lo), "r"(idesc), "r"(accumulate), "l"(a_step), "l"(b_step)
      : "memory");
}

// The cooperative pass over NC finished columns parked in shared memory (column-major, BM rows per column): called by
// NT epilogue threads (te = 0..NT-1).  mt is the tile's row-block index (m0 = BM mt), n0 the global column of the first
// parked column, cprev the previous cell states the caller fetched for EPI_LSTM_CELL (hidden units
// [32 mt + 4 (te % 8), +4), columns n0 + te / 8 + (NT / 8) k).
// Only columns [c_lo, c_hi) of the parked tile are written out (the whole tile: 0, NC).
template <int NC, int NT>
__device__ __forceinline__ void epilogue_pass(const GemmEpilogue& epi, const float* tile, uint32_t te, uint32_t mt, uint32_t m0,
                                              uint32_t n0, uint32_t M, uint32_t N, const float4 (&cprev)[4],
                                              uint32_t c_lo = 0, uint32_t c_hi = NC) {
  if (epi.mode == EPI_LSTM_CELL) {
    // rows 32 q + l of the tile are gate q (i, f, o, g) of hidden unit 32 mt + l
    const uint32_t l = 4 * (te & 7), u = mt * 32 + l;
    float4 bias[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      bias[q] = ld4(epi.bias + (size_t)q * epi.H + u);
      if (q == 1) { bias[q].x += epi.forget_bias; bias[q].y += epi.forget_bias; bias[q].z += epi.forget_bias; bias[q].w += epi.forget_bias; }
    }
#pragma unroll
    for (int k = 0; k < NC / (NT / 8); ++k) {
      const uint32_t c = (te >> 3) + (NT / 8) * k, n = n0 + c;
      if (n < N && c >= c_lo && c < c_hi) {
        float4 g[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 a = ld4(tile + (size_t)c * BM + 32 * q + l);
          const float4 x = make_float4(a.x + bias[q].x, a.y + bias[q].y, a.z + bias[q].z, a.w + bias[q].w);
          g[q] = q == 3 ? make_float4(gate_tanh(x.x), gate_tanh(x.y), gate_tanh(x.z), gate_tanh(x.w))
                        : make_float4(gate_sigmoid(x.x), gate_sigmoid(x.y), gate_sigmoid(x.z), gate_sigmoid(x.w));
          st4(epi.C + (size_t)q * epi.H + u + (size_t)epi.ldc * n, g[q]);
        }
        const size_t e = u + (size_t)epi.H * n;
        const float4 cn = make_float4(lstm_cell_c(g[0].x, g[3].x, g[1].x, cprev[k].x), lstm_cell_c(g[0].y, g[3].y, g[1].y, cprev[k].y),
                                      lstm_cell_c(g[0].z, g[3].z, g[1].z, cprev[k].z), lstm_cell_c(g[0].w, g[3].w, g[1].w, cprev[k].w));
        st4(epi.c_out + e, cn);
        const float4 hv = make_float4(lstm_cell_h(g[2].x, cn.x), lstm_cell_h(g[2].y, cn.y), lstm_cell_h(g[2].z, cn.z), lstm_cell_h(g[2].w, cn.w));
        st4(epi.h_out + e, hv);
        if (epi.hn_hi) epi_emit_h(epi, u, n, hv);
      }
    }
  } else {
    const bool vec = (M & 3) == 0 && (epi.split_m & 3) == 0 && (epi.ldc & 3) == 0 && aligned16(epi.C) &&
                     (epi.split_m == 0 || ((epi.ldc2 & 3) == 0 && aligned16(epi.C2))) &&
                     (epi.mode != EPI_BIAS || aligned16(epi.bias)) && (epi.mode != EPI_GATES || (aligned16(epi.bias) && (epi.H & 3) == 0)) &&
                     (epi.mode != EPI_ACCUM_MASK ||
                      (aligned16(epi.maskC) && (!epi.maskc_full || (epi.maskc_ld & 3) == 0) &&
                       (epi.split_m == 0 || (aligned16(epi.maskC2) && (!epi.maskc2_full || (epi.maskc2_ld & 3) == 0)))));
    if (vec) {
      // 32 row quads x NC columns; a thread keeps its row quad and walks the columns te / 32 + (NT / 32) k
      const uint32_t rq = te & 31, m = m0 + 4 * rq;
      if (m < M) {
        const EpiRow row = epi_row(epi, m);
        const size_t ldc = row.ldc;
        float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
        if (epi.mode == EPI_BIAS || epi.mode == EPI_GATES) bias = ld4(epi.bias + m);
        if (epi.mode == EPI_GATES && m >= epi.H && m < 2 * epi.H) { bias.x += epi.forget_bias; bias.y += epi.forget_bias; bias.z += epi.forget_bias; bias.w += epi.forget_bias; }
        const bool is_tanh = m >= 3 * epi.H;
        const size_t mstep = row.mask_full ? (size_t)row.mask_ld : 0;
#pragma unroll 1
        for (uint32_t c0 = c_lo + (te >> 5); c0 < c_hi; c0 += 8 * (NT / 32)) {   // batches of 8 columns, loads first
          float4 v[8], old[8], mk[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t c = c0 + (NT / 32) * k, n = n0 + c;
            const bool live = n < N && c < c_hi;
            v[k] = ld4(tile + (size_t)min(c, (uint32_t)NC - 1) * BM + 4 * rq);
            if (epi.mode == EPI_ACCUM || epi.mode == EPI_ACCUM_MASK) old[k] = live ? __ldcg(reinterpret_cast<const float4*>(row.c + ldc * n)) : v[k];
            if (epi.mode == EPI_ACCUM_MASK) mk[k] = live ? ld4(row.mask + mstep * n) : v[k];
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t c = c0 + (NT / 32) * k, n = n0 + c;
            if (n >= N || c >= c_hi) continue;
            float4 r = v[k];
            if (epi.mode == EPI_BIAS) { r.x += bias.x; r.y += bias.y; r.z += bias.z; r.w += bias.w; }
            else if (epi.mode == EPI_GATES) {
              r = make_float4(r.x + bias.x, r.y + bias.y, r.z + bias.z, r.w + bias.w);
              r = is_tanh ? make_float4(gate_tanh(r.x), gate_tanh(r.y), gate_tanh(r.z), gate_tanh(r.w))
                          : make_float4(gate_sigmoid(r.x), gate_sigmoid(r.y), gate_sigmoid(r.z), gate_sigmoid(r.w));
            } else if (epi.mode == EPI_ACCUM) { r.x += old[k].x; r.y += old[k].y; r.z += old[k].z; r.w += old[k].w; }
            else if (epi.mode == EPI_ACCUM_MASK) {
              // (explicit fused multiply-adds: every kernel that applies this epilogue rounds alike)
              r = make_float4(__fmaf_rn(r.x, mk[k].x, old[k].x), __fmaf_rn(r.y, mk[k].y, old[k].y), __fmaf_rn(r.z, mk[k].z, old[k].z), __fmaf_rn(r.w, mk[k].w, old[k].w));
            }
            st4(row.c + ldc * n, r);
          }
        }
      }
    } else {
      // any shape / alignment: one row per thread pair of columns, scalar accesses
      const uint32_t r = te & 127, m = m0 + r;
      if (m < M) {
        const EpiRow row = epi_row(epi, m);
        const size_t ldc = row.ldc;
        float bias = 0.f;
        if (epi.mode == EPI_BIAS || epi.mode == EPI_GATES) bias = epi.bias[m];
        if (epi.mode == EPI_GATES && m >= epi.H && m < 2 * epi.H) bias += epi.forget_bias;
        const bool is_tanh = m >= 3 * epi.H;
        const size_t mstep = row.mask_full ? (size_t)row.mask_ld : 0;
#pragma unroll 4
        for (uint32_t c = c_lo + (te >> 7); c < c_hi; c += NT / 128) {
          const uint32_t n = n0 + c;
          if (n >= N) break;
          float v = tile[(size_t)c * BM + r];
          float* dst = row.c + ldc * n;
          if (epi.mode == EPI_STORE) *dst = v;
          else if (epi.mode == EPI_BIAS) *dst = v + bias;
          else if (epi.mode == EPI_GATES) *dst = is_tanh ? gate_tanh(v + bias) : gate_sigmoid(v + bias);
          else if (epi.mode == EPI_ACCUM) *dst += v;
          else *dst = __fmaf_rn(v, row.mask[mstep * n], *dst);
        }
      }
    }
  }
}

__device__ __forceinline__ void bar_sync(uint32_t id, uint32_t count) { asm volatile("barrier.cta.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void bar_arrive(uint32_t id, uint32_t count) { asm volatile("barrier.cta.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }

}  // namespace
