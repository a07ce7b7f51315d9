// One LSTM layer's backward pass over all time steps of a sequence in one kernel: what T calls of
// dyb200_vanilla_lstm_bwd_fused_at compute, i.e. per step the backward passes of VanillaLSTMH, VanillaLSTMC and
// VanillaLSTMGates (dynet/nodes-lstm.cc:262-330, 415-470, 530-580) in the order in which the executor's backward sweep
// visits a CompactVanillaLSTMBuilder layer (dynet/lstm.cc:1044-1080 built them; dynet/exec.cc:96-140 walks them back).
//
// Per step t the per-step form launches a cell pass (dgates from dh_t, dc_t, the saved gates and cell states; also
// dc_{t-1} += ...) and one 3xTF32 product [Wx; Wh]^T dgates whose rows go to dx_t and dh_{t-1}.  Here the CTAs of that
// product stay resident: CTA (mt, nt, split) owns rows [128 mt, +128) of [dx; dh] x BNT batch columns in every step, and
// its eight epilogue warps also run a share of the cell pass of its column block.  The two hand-overs of a step are
// counters in global memory, one pair per column block (column blocks never wait for one another):
//   cell_done[nt]  += 1 per finished cell tile   -> the TMA warps wait for all tiles of the step before reading dgates
//   gemm_done[nt]  += 1 per finished product CTA -> the cell pass of the next step waits for all CTAs (dh_{t-1} complete,
//                                                   the dgates planes free to be overwritten)
// K splits exchange their partial tiles through a workspace in global memory (L2) and a counter per tile; rank r of a
// tile's S CTAs adds the S partial tiles of its slice of the columns in split order and runs the epilogue on it.
//
// Every wait is bounded: on expiry the CTA sets DYB200_FLAG_WAIT_TIMEOUT, stops storing, keeps signalling so that nothing
// else stalls longer than its own bound, frees its TMEM and returns.
//
// Values are bit for bit those of the per-step calls: the cell arithmetic of the per-step pass (lstm_cell.cuh), per-tile row
// sums of dgates added per step in tile order and the steps in sweep order (k_seq_db_reduce), the same k-blocks in the same
// accumulation chains (cut every kChunkKB k-blocks), the same K splits (dyb200_lstm_bwd_tiling, which the per-step call
// also asks) added in split order, the epilogue of the product kernels (epilogue_pass).
#include "lstm_cell.cuh"
#include "seq_dev.cuh"

namespace {

struct SeqBwd {
  uint32_t T, B, H, I;              // the kernel runs steps t = T - 1 .. 0
  uint32_t kb;                      // k-blocks of the product: 4H / 32
  uint32_t ncb;                     // column blocks per CTA (1 or 2)
  const float* gates; const float* cs;      // saved by the forward pass: step t at + t * 4H * B / + t * H * B
  const float* c0;                  // the cell state before step 0
  float* dh; float* dc; float* dx;          // H x (T B), H x (T B), I x (T B); all accumulate
  // operand planes of dgates of all steps: row = t B + batch column, K = 4H.  The K-major right operand of each step's
  // product and, read MN-major by the deferred weight-gradient products, their left operand (the accumulator's A planes).
  float *dn_hi, *dn_lo; uint32_t dn_pitch;
  float* part;                      // per-tile row sums of dgates: [step][B / 32][4H]
  const float* mx; int mx_full; const float* mh; int mh_full;   // dropout masks of the layer's inputs (null: none)
  float* ws;                        // split exchange: [tile][split][BNT columns][128 rows]
  uint32_t* cell_done; uint32_t* gemm_done; uint32_t* sent;   // [B / BNT], [B / BNT], [tiles]; zero at launch
  uint32_t* flags;
};

constexpr int kCellB = 32;   // batch columns of one cell tile

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// The cell pass of one tile (JT = 32 or 64 hidden units from j0, 32 batch columns from b0) of step t, by the 256 epilogue
// threads (tid = 0..255); the arithmetic of k_lstm_cell_bwd_tiled, minus its sum over batch tiles (the per-tile row sums
// go to a.part).  `tile` holds 4 x JT x 32 floats, un-padded, for those row sums; element (gate, unit, column) sits at
// column ^ (unit & 31) of its row, which keeps both the element-wise writes (8 or 16 units per warp, one column) and the
// row-wise reads (one unit, 32 columns) free of bank conflicts.
template <int JT>
__device__ __forceinline__ void cell_bwd_tile(const SeqBwd& a, uint32_t t, uint32_t step, uint32_t j0, uint32_t b0, uint32_t tid, float* tile) {
  constexpr int kQuads = JT / 4, kLanes = 256 / kQuads, kCols = kCellB / kLanes;   // 8 x 32 x 1 or 16 x 16 x 2
  const uint32_t H = a.H, B = a.B;
  const size_t HB = (size_t)H * B;
  const float* gates = a.gates + (size_t)t * 4 * HB;
  const float* c_t = a.cs + (size_t)t * HB;
  const float* c_tm1 = t ? a.cs + (size_t)(t - 1) * HB : a.c0;
  const float* dEdh = a.dh + (size_t)t * HB;
  const float* dEdc = a.dc + (size_t)t * HB;
  float* dc_tm1 = t ? a.dc + (size_t)(t - 1) * HB : nullptr;   // (step 0 has no earlier step to hand dE/dc to)
  const uint32_t tq = tid % kQuads, tb = tid / kQuads;
  const uint32_t j = j0 + 4 * tq;
  float4 gi[kCols], gf[kCols], go[kCols], gg[kCols], c[kCols], cp[kCols], dh[kCols], dcin[kCols], dcp[kCols];
#pragma unroll
  for (int k = 0; k < kCols; ++k) {   // all loads of the tile first
    const uint32_t b = b0 + tb + kLanes * k;
    const size_t e = (size_t)b * H + j;
    const float* g = gates + (size_t)b * 4 * H + j;
    gi[k] = ld4(g); gf[k] = ld4(g + H); go[k] = ld4(g + 2 * H); gg[k] = ld4(g + 3 * H);
    c[k] = ld4(c_t + e); cp[k] = ld4(c_tm1 + e);
    // (dh_t and dc_t were finished by other CTAs / earlier in this kernel: read them from L2)
    dh[k] = __ldcg(reinterpret_cast<const float4*>(dEdh + e)); dcin[k] = __ldcg(reinterpret_cast<const float4*>(dEdc + e));
    dcp[k] = t ? __ldcg(reinterpret_cast<const float4*>(dc_tm1 + e)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int k = 0; k < kCols; ++k) {
    const uint32_t bl = tb + kLanes * k, b = b0 + bl;
    const size_t e = (size_t)b * H + j;
    float pi[4], pf[4], po[4], pg[4];
    const float gi_[4] = {gi[k].x, gi[k].y, gi[k].z, gi[k].w}, gf_[4] = {gf[k].x, gf[k].y, gf[k].z, gf[k].w},
                go_[4] = {go[k].x, go[k].y, go[k].z, go[k].w}, gg_[4] = {gg[k].x, gg[k].y, gg[k].z, gg[k].w},
                c_[4] = {c[k].x, c[k].y, c[k].z, c[k].w}, cp_[4] = {cp[k].x, cp[k].y, cp[k].z, cp[k].w},
                dh_[4] = {dh[k].x, dh[k].y, dh[k].z, dh[k].w}, dci_[4] = {dcin[k].x, dcin[k].y, dcin[k].z, dcin[k].w};
    float dcp_[4] = {dcp[k].x, dcp[k].y, dcp[k].z, dcp[k].w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      lstm_cell_grad(gi_[q], gf_[q], go_[q], gg_[q], c_[q], cp_[q], dh_[q], dci_[q], true, dcp_[q], pi[q], pf[q], po[q], pg[q]);
      const uint32_t u = 4 * tq + q, col = bl ^ (u & 31);
      tile[(0 * JT + u) * kCellB + col] = pi[q]; tile[(1 * JT + u) * kCellB + col] = pf[q];
      tile[(2 * JT + u) * kCellB + col] = po[q]; tile[(3 * JT + u) * kCellB + col] = pg[q];
    }
    if (t) st4(dc_tm1 + e, make_float4(dcp_[0], dcp_[1], dcp_[2], dcp_[3]));
    const size_t o = ((size_t)t * B + b) * a.dn_pitch + j;
    float hi[4], lo[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) split_tf32(pi[q], hi[q], lo[q]);
    st4(a.dn_hi + o, make_float4(hi[0], hi[1], hi[2], hi[3])); st4(a.dn_lo + o, make_float4(lo[0], lo[1], lo[2], lo[3]));
#pragma unroll
    for (int q = 0; q < 4; ++q) split_tf32(pf[q], hi[q], lo[q]);
    st4(a.dn_hi + o + H, make_float4(hi[0], hi[1], hi[2], hi[3])); st4(a.dn_lo + o + H, make_float4(lo[0], lo[1], lo[2], lo[3]));
#pragma unroll
    for (int q = 0; q < 4; ++q) split_tf32(po[q], hi[q], lo[q]);
    st4(a.dn_hi + o + 2 * H, make_float4(hi[0], hi[1], hi[2], hi[3])); st4(a.dn_lo + o + 2 * H, make_float4(lo[0], lo[1], lo[2], lo[3]));
#pragma unroll
    for (int q = 0; q < 4; ++q) split_tf32(pg[q], hi[q], lo[q]);
    st4(a.dn_hi + o + 3 * H, make_float4(hi[0], hi[1], hi[2], hi[3])); st4(a.dn_lo + o + 3 * H, make_float4(lo[0], lo[1], lo[2], lo[3]));
  }
  bar_sync(1, 256);
  // row sums over the 32 columns, one row per thread, added in the order of a butterfly reduction over the columns (the
  // order of the per-step pass's warp_sum, seen from lane 0)
  if (tid < 4 * JT) {
    const uint32_t gate = tid / JT, jl = tid % JT;
    const float* rowp = tile + (size_t)tid * kCellB;
    float v[32];
#pragma unroll
    for (int cc = 0; cc < 32; ++cc) v[cc] = rowp[cc ^ (jl & 31)];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int cc = 0; cc < o; ++cc) v[cc] += v[cc + o];
    float* part = a.part + ((size_t)step * (B / kCellB) + b0 / kCellB) * 4 * H;
    part[(size_t)gate * H + j0 + jl] = v[0];
  }
}

// Requests the lines of the saved gates and cell states that the cell tile (j0, b0) of step t will read into L2 (they come
// from HBM: 35 steps of gates do not stay in L2), so that the pass itself only waits for L2.
template <int JT>
__device__ __forceinline__ void cell_prefetch(const SeqBwd& a, uint32_t t, uint32_t j0, uint32_t b0, uint32_t tid) {
  constexpr int kQuads = JT / 4, kLanes = 256 / kQuads, kCols = kCellB / kLanes;
  const uint32_t H = a.H;
  const size_t HB = (size_t)H * a.B;
  const uint32_t tq = tid % kQuads, tb = tid / kQuads;
  if (tq % 8 != 0) return;   // one request per 128-byte line (8 threads x 16 bytes)
  const uint32_t j = j0 + 4 * tq;
#pragma unroll
  for (int k = 0; k < kCols; ++k) {
    const uint32_t b = b0 + tb + kLanes * k;
    const size_t e = (size_t)b * H + j;
    const float* g = a.gates + (size_t)t * 4 * HB + (size_t)b * 4 * H + j;
    prefetch_l2(g); prefetch_l2(g + H); prefetch_l2(g + 2 * H); prefetch_l2(g + 3 * H);
    prefetch_l2(a.cs + (size_t)t * HB + e); prefetch_l2(t ? a.cs + (size_t)(t - 1) * HB + e : a.c0 + e);
  }
}

// SPLIT: gridDim.z > 1 (its own instantiation: the unsplit epilogue, which parks a 128-column tile in two rounds, would
// cost the split one registers).
template <int BNT, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1) k_lstm_seq_bwd(const __grid_constant__ TmapPack tm, const SeqBwd a) {
  constexpr int kStages = BNT == 64 ? 4 : 3;
  constexpr int kStageBytes = 2 * TILE_BYTES + 2 * BNT * BK * 4;
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], acc_full[kSeqBufs], acc_empty[kSeqBufs];
  __shared__ uint32_t tmem_base_slot;
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* park = reinterpret_cast<float*>(ring + (size_t)kStages * kStageBytes);   // 64 columns x BM rows; also the cell tile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int TILE_B_BYTES = BNT * BK * 4;
  constexpr int STAGE_TX = 2 * TILE_BYTES + 2 * TILE_B_BYTES;
  const uint32_t S = gridDim.z, rank = blockIdx.z;
  const uint32_t m0 = blockIdx.x * BM;
  const KSplit ks = k_split(a.kb, 0, rank, S);
  const uint32_t total = ks.n0;                   // k-blocks of this CTA per product
  const uint32_t N = a.B;
  const uint32_t steps = a.T, ncb = a.ncb;
  // the CTAs that serve a column block share its cell tiles: (H / 32) x (BNT / 32) per step
  const uint32_t n_cta = gridDim.x * S, my_cta = blockIdx.x * S + rank;
  // (64-unit tiles when there are more 32-unit tiles than CTAs to take them: one round of loads instead of two)
  const uint32_t cell_j = (a.H / 32) * (BNT / kCellB) > n_cta && a.H % 64 == 0 ? 64u : 32u;
  const uint32_t n_cell = (a.H / cell_j) * (BNT / kCellB);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (uint32_t q = 0; q < kSeqBufs; ++q) { mbar_init(&acc_full[q], 1); mbar_init(&acc_empty[q], kEpiWarps); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (threadIdx.x == 32 * 2) {
#pragma unroll
    for (int q = 0; q < 4; ++q) asm volatile("prefetch.tensormap [%0];" ::"l"(&tm.t[q]) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kSeqBufs * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {
      // TMA producer.  Every product reads rows [m0, m0 + 128) of [Wx; Wh]^T and rows [t B + n0, + BNT) of the dgates planes.
      uint32_t s = 0, ph = 0;
      bool fail = false;
      bool ready = false;   // the cell pass of the product about to start has already been seen complete
      for (uint32_t step = 0; step < steps && !fail; ++step) {
        for (uint32_t cb = 0; cb < ncb && !fail; ++cb) {
          const uint32_t nt = blockIdx.y * ncb + cb, n0 = nt * BNT;
          const int brow = (int)((a.T - 1 - step) * a.B + n0);   // this step's rows of the dgates planes
          uint32_t it0 = 0;
          if (!ready) {
            // the weight tiles of the first k-blocks do not depend on this step's cell pass: request them before the wait
            const uint32_t pre = min((uint32_t)kStages, total);
            uint32_t s2 = s, ph2 = ph;
            for (uint32_t j = 0; j < pre; ++j) {
              if (!mbar_wait(&empty_bar[s2], ph2 ^ 1)) { fail = true; break; }
              unsigned char* st = ring + (size_t)s2 * kStageBytes;
              mbar_expect_tx(&full_bar[s2], STAGE_TX);
              tma_load_2d(st, &tm.t[0], &full_bar[s2], (int)((ks.b0 + j) * BK), (int)m0);
              tma_load_2d(st + TILE_BYTES, &tm.t[1], &full_bar[s2], (int)((ks.b0 + j) * BK), (int)m0);
              if (++s2 == kStages) { s2 = 0; ph2 ^= 1; }
            }
            if (fail) break;
            if (!wait_counter(a.cell_done + nt, (step + 1) * n_cell)) { fail = true; break; }
            asm volatile("fence.proxy.async.global;" ::: "memory");   // generic-proxy stores of other CTAs -> this CTA's TMA reads
            for (uint32_t j = 0; j < pre; ++j) {
              unsigned char* st = ring + (size_t)s * kStageBytes;
              tma_load_2d(st + 2 * TILE_BYTES, &tm.t[2], &full_bar[s], (int)((ks.b0 + j) * BK), brow);
              tma_load_2d(st + 2 * TILE_BYTES + TILE_B_BYTES, &tm.t[3], &full_bar[s], (int)((ks.b0 + j) * BK), brow);
              if (++s == kStages) { s = 0; ph ^= 1; }
            }
            it0 = pre;
          }
          ready = false;
          // With two chains the next product's cell pass has normally finished long before this product's loads are all
          // issued: one look at its counter, a ring's length before the end, lets the next product start without a gap.
          const bool last_cb = cb + 1 == ncb;
          const uint32_t nstep = last_cb ? step + 1 : step, nnt = blockIdx.y * ncb + (last_cb ? 0 : cb + 1);
          const uint32_t peek_at = total > (uint32_t)kStages ? total - kStages : total;
          for (uint32_t it = it0; it < total; ++it) {
            if (it == peek_at && nstep < steps && peek_counter(a.cell_done + nnt) >= (nstep + 1) * n_cell) {
              ready = true;
              asm volatile("fence.proxy.async.global;" ::: "memory");
            }
            if (!mbar_wait(&empty_bar[s], ph ^ 1)) { fail = true; break; }
            const uint32_t kblk = ks.b0 + it;
            unsigned char* st = ring + (size_t)s * kStageBytes;
            mbar_expect_tx(&full_bar[s], STAGE_TX);
            tma_load_2d(st, &tm.t[0], &full_bar[s], (int)(kblk * BK), (int)m0);
            tma_load_2d(st + TILE_BYTES, &tm.t[1], &full_bar[s], (int)(kblk * BK), (int)m0);
            tma_load_2d(st + 2 * TILE_BYTES, &tm.t[2], &full_bar[s], (int)(kblk * BK), brow);
            tma_load_2d(st + 2 * TILE_BYTES + TILE_B_BYTES, &tm.t[3], &full_bar[s], (int)(kblk * BK), brow);
            if (++s == kStages) { s = 0; ph ^= 1; }
          }
        }
      }
      if (fail) atomicOr(a.flags, DYB200_FLAG_WAIT_TIMEOUT);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BNT >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      uint64_t d_a_hi[kStages], d_a_lo[kStages], d_b_hi[kStages], d_b_lo[kStages];
#pragma unroll
      for (int q = 0; q < kStages; ++q) {
        const uint32_t base = smem_u32(ring + (size_t)q * kStageBytes);
        d_a_hi[q] = umma_desc(base); d_a_lo[q] = umma_desc(base + TILE_BYTES);
        d_b_hi[q] = umma_desc(base + 2 * TILE_BYTES); d_b_lo[q] = umma_desc(base + 2 * TILE_BYTES + TILE_B_BYTES);
      }
      // stage, phase and chunk counters run on across products; an accumulation chain never crosses a product
      uint32_t s = 0, ph = 0, chunk = 0, buf = 0;
      bool fail = false;
      for (uint32_t prod = 0; prod < steps * ncb && !fail; ++prod) {
        uint32_t in_chunk = 0;
        for (uint32_t it = 0; it < total; ++it) {
          if (in_chunk == 0 && chunk >= kSeqBufs) {
            if (!mbar_wait(&acc_empty[buf], ((chunk / kSeqBufs) - 1) & 1)) { fail = true; break; }
          }
          if (!mbar_wait(&full_bar[s], ph)) { fail = true; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          uint64_t a_hi, a_lo, b_hi, b_lo;   // select without dynamic register indexing
          if (s == 0) { a_hi = d_a_hi[0]; a_lo = d_a_lo[0]; b_hi = d_b_hi[0]; b_lo = d_b_lo[0]; }
          else if (s == 1) { a_hi = d_a_hi[1]; a_lo = d_a_lo[1]; b_hi = d_b_hi[1]; b_lo = d_b_lo[1]; }
          else if (s == 2 || kStages == 3) { a_hi = d_a_hi[2]; a_lo = d_a_lo[2]; b_hi = d_b_hi[2]; b_lo = d_b_lo[2]; }
          else { a_hi = d_a_hi[kStages - 1]; a_lo = d_a_lo[kStages - 1]; b_hi = d_b_hi[kStages - 1]; b_lo = d_b_lo[kStages - 1]; }
          issue_kblock(tmem_base + buf * BN, a_hi, a_lo, b_hi, b_lo, idesc, in_chunk);
          umma_commit(&empty_bar[s]);
          const bool chunk_ends = in_chunk == kChunkKB - 1 || it == total - 1;
          if (chunk_ends) { umma_commit(&acc_full[buf]); in_chunk = 0; ++chunk; buf = chunk % kSeqBufs; }
          else ++in_chunk;
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
      if (fail) atomicOr(a.flags, DYB200_FLAG_WAIT_TIMEOUT);
    }
  } else {
    // warps 2..9: the epilogue of each product, and this CTA's share of the cell tiles of its column blocks
    const uint32_t quarter = warp & 3, half = (warp - 2) >> 2;
    const uint32_t te = threadIdx.x - 64;
    const bool has_cols = 64 * half < BNT;
    const uint32_t nchunks = (total + kChunkKB - 1) / kChunkKB;
    // The BNT columns of a tile are finished by its S CTAs, w columns each (S > 1: at most 64, one exchange buffer full).
    const uint32_t w = ((BNT + S - 1) / S + 7) & ~7u;
    const uint32_t c_lo = min(rank * w, (uint32_t)BNT), c_hi = min(c_lo + w, (uint32_t)BNT);
    const size_t HB = (size_t)a.H * a.B, IB = (size_t)a.I * a.B;
    GemmEpilogue epi{a.mx ? EPI_ACCUM_MASK : EPI_ACCUM, nullptr, a.I, nullptr, 0, 0.f, a.mx, a.I, a.mx_full};
    epi.split_m = a.I; epi.ldc2 = a.H; epi.maskC2 = a.mh; epi.maskc2_ld = a.H; epi.maskc2_full = a.mh_full;
    const float4 no_cprev[4] = {};
    uint32_t cg = 0;
    bool ok = true;   // the same for all 256 threads after every bar_and below

    // the cell tiles of column block nt for `step` that fall to this CTA; each finished tile is published on its own
    auto cell_pass = [&](uint32_t nt, uint32_t step) {
      const uint32_t t = a.T - 1 - step;
      for (uint32_t blk = my_cta; blk < n_cell; blk += n_cta) {
        const uint32_t j0 = (blk / (BNT / kCellB)) * cell_j, b0 = nt * BNT + (blk % (BNT / kCellB)) * kCellB;
        if (!ok) bar_sync(1, 256);
        else if (cell_j == 64) cell_bwd_tile<64>(a, t, step, j0, b0, te, park);
        else cell_bwd_tile<32>(a, t, step, j0, b0, te, park);
        bar_sync(1, 256);   // all stores of the tile are issued; the tile buffer may be reused
        if (te == 0) {
          // One thread publishes: its release orders all stores it has observed, through the barrier, before the counter
          // update (cumulativity), for the generic and for the async proxy (the readers are TMA loads).
          asm volatile("fence.proxy.async.global;" ::: "memory");
          signal_counter(a.cell_done + nt);
        }
      }
    };
    for (uint32_t cb = 0; cb < ncb; ++cb) cell_pass(blockIdx.y * ncb + cb, 0);

#pragma unroll 1
    for (uint32_t step = 0; step < steps; ++step) {
      const uint32_t t = a.T - 1 - step;
#pragma unroll 1
      for (uint32_t cb = 0; cb < ncb; ++cb) {
        const uint32_t nt = blockIdx.y * ncb + cb, n0 = nt * BNT;
        const uint32_t tile_id = nt * gridDim.x + blockIdx.x;
        float* const ws_tile = a.ws + (size_t)tile_id * S * BNT * BM;   // (unused when S == 1)
        // While the product runs: ask L2 for what this chain needs next from HBM - the saved gates / cell states of the cell
        // tiles of its next step, and the current values of the dx / dh entries this CTA is about to add to.
        if (step + 1 < steps) {
          for (uint32_t blk = my_cta; blk < n_cell; blk += n_cta) {
            const uint32_t j0 = (blk / (BNT / kCellB)) * cell_j, b0 = nt * BNT + (blk % (BNT / kCellB)) * kCellB;
            if (cell_j == 64) cell_prefetch<64>(a, t - 1, j0, b0, te);
            else cell_prefetch<32>(a, t - 1, j0, b0, te);
          }
        }
        if (m0 + 4 * (te & 31) < (t ? a.I + a.H : a.I)) {
          const uint32_t m = m0 + 4 * (te & 31);
          const float* base = m < a.I ? a.dx + (size_t)t * IB + m : a.dh + (size_t)(t - 1) * HB + (m - a.I);
          const size_t ld = m < a.I ? a.I : a.H;
          if ((te & 7) == 0)
            for (uint32_t c = c_lo + (te >> 5); c < c_hi; c += 8) prefetch_l2(base + ld * (n0 + c));
        }
        // With at most 32 columns per CTA (4 per thread in the epilogue's layout: row quad te % 32, columns c_lo + te / 32 + 8 k)
        // the current dx / dh values and the mask values are fetched into registers now, so that the epilogue after the exchange
        // only waits for shared memory.
        const bool pre_epi = SPLIT && c_hi - c_lo <= 32;
        float4 old4[4];
        const uint32_t m_epi = m0 + 4 * (te & 31);
        const bool epi_row_live = pre_epi && m_epi < (t ? a.I + a.H : a.I);
        const bool to_dx = m_epi < a.I;
        float* const cbase = to_dx ? a.dx + (size_t)t * IB + m_epi : a.dh + (size_t)(t ? t - 1 : 0) * HB + (m_epi - a.I);
        const uint32_t ld_epi = to_dx ? a.I : a.H;
        if (epi_row_live) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t c = c_lo + (te >> 5) + 8 * k, n = n0 + c;
            old4[k] = (c < c_hi && n < N) ? __ldcg(reinterpret_cast<const float4*>(cbase + (size_t)ld_epi * n)) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
        // ---- drain the accumulation chains of this product ----
        float sum[64];
#pragma unroll
        for (int q = 0; q < 64; ++q) sum[q] = 0.f;
#pragma unroll 1
        for (uint32_t c = 0; c < nchunks; ++c, ++cg) {
          const uint32_t buf = cg % kSeqBufs;
          if (!ok) continue;
          if (!mbar_wait(&acc_full[buf], (cg / kSeqBufs) & 1)) { ok = false; continue; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (has_cols) {
            float v[32];
            const uint32_t taddr = tmem_base + buf * BN + ((quarter * 32) << 16) + 2 * half * 32;
            tmem_ld32(taddr, v);
#pragma unroll
            for (int q = 0; q < 32; ++q) sum[q] += v[q];
            tmem_ld32(taddr + 32, v);
#pragma unroll
            for (int q = 0; q < 32; ++q) sum[32 + q] += v[q];
          }
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        epi.C = a.dx + (size_t)t * IB;
        epi.C2 = t ? a.dh + (size_t)(t - 1) * HB : nullptr;
        const uint32_t M = t ? a.I + a.H : a.I;   // step 0 has no dE/dh_{t-1}: the rows of the product beyond dx are dropped
        if (SPLIT) {
          // this split's partial tile -> the workspace (column-major like C: a warp stores 32 consecutive rows of a column)
          if (has_cols) {
            float* col = ws_tile + ((size_t)rank * BNT + 64 * half) * BM + quarter * 32 + lane;
#pragma unroll
            for (int q = 0; q < 64; ++q) __stcg(col + (size_t)q * BM, sum[q]);
          }
          ok = bar_and(1, 256, ok) != 0;
          bool got = true;
          if (te == 0) {
            signal_counter(a.sent + tile_id);
            got = wait_counter(a.sent + tile_id, (step + 1) * S);
          }
          ok = bar_and(1, 256, ok && got) != 0;
        }
        if (SPLIT) {
          // the S partial tiles of this CTA's slice, added in split order: all loads of a piece are issued before the adds
          const uint32_t f_lo = c_lo * (BM / 4), f_hi = c_hi * (BM / 4);   // 16-byte pieces of the slice
          const float4* src = reinterpret_cast<const float4*>(ws_tile);
          float4* dst = reinterpret_cast<float4*>(park) - f_lo;          // (the buffer starts at column c_lo)
          if (S <= 4) {
            // two pieces per round: 2 S <= 8 loads in flight
            for (uint32_t f = f_lo + te; ok && f < f_hi; f += 512) {
              const uint32_t f2 = f + 256 < f_hi ? f + 256 : f;   // (the last round may have one piece: it is then read twice)
              float4 pv[8];
#pragma unroll
              for (uint32_t r = 0; r < 4; ++r)
                if (r < S) {
                  pv[r] = __ldcg(src + (size_t)r * BNT * (BM / 4) + f);
                  pv[4 + r] = __ldcg(src + (size_t)r * BNT * (BM / 4) + f2);
                }
              float4 acc = pv[0], acc2 = pv[4];
#pragma unroll
              for (uint32_t r = 1; r < 4; ++r)
                if (r < S) {
                  acc.x += pv[r].x; acc.y += pv[r].y; acc.z += pv[r].z; acc.w += pv[r].w;
                  acc2.x += pv[4 + r].x; acc2.y += pv[4 + r].y; acc2.z += pv[4 + r].z; acc2.w += pv[4 + r].w;
                }
              dst[f] = acc;
              dst[f2] = acc2;
            }
          } else {
            for (uint32_t f = f_lo + te; ok && f < f_hi; f += 256) {
              float4 pv[8];
#pragma unroll
              for (uint32_t r = 0; r < 8; ++r)
                if (r < S) pv[r] = __ldcg(src + (size_t)r * BNT * (BM / 4) + f);
              float4 acc = pv[0];
#pragma unroll
              for (uint32_t r = 1; r < 8; ++r)
                if (r < S) { acc.x += pv[r].x; acc.y += pv[r].y; acc.z += pv[r].z; acc.w += pv[r].w; }
              dst[f] = acc;
            }
          }
          ok = bar_and(1, 256, ok) != 0;
          if (ok && pre_epi) {
            // dx / dh = old + sum .* mask (the arithmetic of epilogue_pass for EPI_ACCUM / EPI_ACCUM_MASK) on the prefetched values
            if (epi_row_live) {
              const float* mbase = to_dx ? a.mx : a.mh;
              const uint32_t mrow = to_dx ? m_epi : m_epi - a.I;
              const bool mfull = to_dx ? a.mx_full : a.mh_full;
              float4 mk4[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint32_t c = c_lo + (te >> 5) + 8 * k, n = n0 + c;
                mk4[k] = (mbase && c < c_hi && n < N) ? ld4(mbase + mrow + (mfull ? (size_t)ld_epi * n : 0)) : make_float4(1.f, 1.f, 1.f, 1.f);
              }
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint32_t cs = (te >> 5) + 8 * k, n = n0 + c_lo + cs;   // cs: column within the slice
                if (c_lo + cs < c_hi && n < N) {
                  const float4 v = ld4(park + (size_t)cs * BM + 4 * (te & 31));
                  float4 r;
                  if (mbase) r = make_float4(__fmaf_rn(v.x, mk4[k].x, old4[k].x), __fmaf_rn(v.y, mk4[k].y, old4[k].y),
                                             __fmaf_rn(v.z, mk4[k].z, old4[k].z), __fmaf_rn(v.w, mk4[k].w, old4[k].w));
                  else r = make_float4(v.x + old4[k].x, v.y + old4[k].y, v.z + old4[k].z, v.w + old4[k].w);
                  st4(cbase + (size_t)ld_epi * n, r);
                }
              }
            }
          } else if (ok) {
            epilogue_pass<BNT, 256>(epi, park - (size_t)c_lo * BM, te, blockIdx.x, m0, n0, M, N, no_cprev, c_lo, c_hi);
          }
          bar_sync(1, 256);   // the exchange buffer may be overwritten; every thread's stores of dx / dh are issued
        } else {
#pragma unroll 1
          for (uint32_t hh = 0; hh < BNT / 64; ++hh) {
            if (half == hh) {
              float* col = park + quarter * 32 + lane;
#pragma unroll
              for (int q = 0; q < 64; ++q) col[(size_t)q * BM] = sum[q];
            }
            ok = bar_and(1, 256, ok) != 0;
            if (ok) epilogue_pass<64, 256>(epi, park, te, blockIdx.x, m0, n0 + 64 * hh, M, N, no_cprev);
            bar_sync(1, 256);
          }
        }
        if (te == 0) signal_counter(a.gemm_done + nt);
        // ---- the cell pass of this chain's next step: needs dh complete (every product CTA of the column block through
        // with this step) ----
        if (step + 1 < steps) {
          if (my_cta < n_cell) {
            bool got = true;
            if (te == 0) got = wait_counter(a.gemm_done + nt, (step + 1) * n_cta);
            ok = bar_and(1, 256, ok && got) != 0;
          }
          cell_pass(nt, step + 1);
        }
      }
    }
    if (!ok && lane == 0) atomicOr(a.flags, DYB200_FLAG_WAIT_TIMEOUT);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kSeqBufs * BN) : "memory");
  }
}

// db += the row sums of dgates of all steps: per step the batch tiles in ascending order, then the steps in sweep order (a
// fixed order, so the result is the same from run to run).  A CTA owns 32 gate rows; its 8 warps take the steps s, s + 8, ...
// in parallel (lane = row, all tiles of a step in flight), leave the per-step sums in shared memory, and warp 0 adds them up.
constexpr uint32_t kDbMaxSteps = 256;
__global__ void __launch_bounds__(256) k_seq_db_reduce(const float* __restrict__ part, uint32_t steps, uint32_t tiles, uint32_t G,
                                                       float* __restrict__ db) {
  dyb_grid_dep_sync();
  __shared__ float per_step[kDbMaxSteps][32];
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t row = blockIdx.x * 32 + lane;
  if (row < G) {
    for (uint32_t s = warp; s < steps; s += 8) {
      const float* p = part + (size_t)s * tiles * G + row;
      float acc = 0.f;
      uint32_t t = 0;
      for (; t + 8 <= tiles; t += 8) {
        float v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) v[q] = __ldcg(p + (size_t)(t + q) * G);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc += v[q];
      }
      for (; t < tiles; ++t) acc += __ldcg(p + (size_t)t * G);
      per_step[s][lane] = acc;
    }
  }
  __syncthreads();
  if (warp == 0 && row < G) {
    float d = db[row];
    for (uint32_t s = 0; s < steps; ++s) d += per_step[s][lane];
    db[row] = d;
  }
}

}  // namespace

// ---- host side ---------------------------------------------------------------------------------------------------------
namespace {

template <int BNT, bool SPLIT>
int launch_seq_bwd(dyb200_ctx* ctx, const TmapPack& tm, const SeqBwd& a, dim3 grid, double flops) {
  const uint32_t bit = (BNT == 64 ? (1u << 20) : (1u << 21)) << (SPLIT ? 2 : 0);
  if (!(ctx->func_attr_done & bit)) {
    DYB_CUDA(ctx, cudaFuncSetAttribute(k_lstm_seq_bwd<BNT, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_SEQ_BYTES));
    ctx->func_attr_done |= bit;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid; cfg.blockDim = dim3(kThreads, 1, 1); cfg.dynamicSmemBytes = SMEM_SEQ_BYTES; cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  // All CTAs wait on one another, so they have to be resident together: the grid never exceeds one CTA per SM (checked by
  // the caller), and the cooperative attribute makes the driver schedule them as one gang.  A driver that refuses the
  // attribute gets a plain launch (the waits are bounded either way).
  if (ctx->seq_coop >= 0) {
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    GemmProfScope scope(ctx, flops, 1, a.I + a.H, a.B * a.T, a.kb * BK, EPI_ACCUM_MASK);
    cudaError_t e = cudaLaunchKernelEx(&cfg, k_lstm_seq_bwd<BNT, SPLIT>, tm, a);
    if (e == cudaSuccess) { ctx->seq_coop = 1; ctx->launches++; return DYB200_OK; }
    (void)cudaGetLastError();
    if (ctx->seq_coop == 1) return dyb200_fail(ctx, DYB200_ECUDA, "sequence kernel launch failed: %s", cudaGetErrorString(e));
    ctx->seq_coop = -1;
  }
  cfg.attrs = nullptr; cfg.numAttrs = 0;
  GemmProfScope scope(ctx, flops, 1, a.I + a.H, a.B * a.T, a.kb * BK, EPI_ACCUM_MASK);
  cudaLaunchKernelEx(&cfg, k_lstm_seq_bwd<BNT, SPLIT>, tm, a);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

}  // namespace

extern "C" {

int dyb200_vanilla_lstm_seq_bwd(const dyb200_tensor* x_all, const dyb200_tensor* h0, const dyb200_tensor* c0,
                                const dyb200_tensor* Wx, const dyb200_tensor* Wh, const dyb200_tensor* mask_x,
                                const dyb200_tensor* mask_h, const dyb200_lstm_gates_attrs* attrs, const dyb200_tensor* gates_all,
                                const dyb200_tensor* c_all, const dyb200_tensor* h_all, dyb200_tensor* dh_all, dyb200_tensor* dc_all,
                                dyb200_tensor* dx_all, dyb200_tensor* dWx, dyb200_tensor* dWh, dyb200_tensor* db,
                                dyb200_wgrad* deferred, uint32_t steps, dyb200_ctx* ctx) {
  DYB_CHECK_ARG(ctx, x_all && h0 && c0 && Wx && Wh && attrs && gates_all && c_all && h_all && dh_all && dc_all && db && steps > 0 &&
                         (deferred || (dWx && dWh)), "lstm_seq_bwd: null argument");
  DYB_CHECK_ARG(ctx, (attrs->dropout != 0) == (mask_x != nullptr && mask_h != nullptr), "lstm_seq_bwd: masks must be given exactly when dropout is set");
  DYB_CHECK_ARG(ctx, x_all->nd == 1 && x_all->bd % steps == 0, "lstm_seq_bwd: x_all must be Dim({I}, steps * batch)");
  const uint32_t T = steps, B = x_all->bd / T, I = t_dim(x_all, 0), H = t_dim(h0, 0), G = 4 * H;
  const size_t HB = (size_t)H * B, IB = (size_t)I * B;
  DYB_CHECK_ARG(ctx, h0->nd == 1 && h0->bd == B && c0->bd == B && t_dim(c0, 0) == H, "lstm_seq_bwd: h0 / c0 must be Dim({H}, batch)");
  DYB_CHECK_ARG(ctx, t_size(gates_all) == 4 * HB * T && t_size(c_all) == HB * T && t_size(h_all) == HB * T && t_size(dh_all) == HB * T &&
                         t_size(dc_all) == HB * T && (!dx_all || t_size(dx_all) == IB * T), "lstm_seq_bwd: the state tensors must hold all %u steps", T);
  if (HB == 0) return DYB200_OK;
  int rc;
  const float* mx = attrs->dropout ? mask_x->v : nullptr;
  const float* mh = attrs->dropout ? mask_h->v : nullptr;
  const int mx_full = mx ? mask_x->bd == B : 0, mh_full = mh ? mask_h->bd == B : 0;

  // ---- all steps in one kernel, when its CTAs can all be resident ----
  uint32_t first = T;   // steps [0, first) run as per-step calls below
  LstmBwdTiling tl{64, 1, 1};
  const uint32_t Imin = I < H ? I : H;
  const double flops_small = 2.0 * Imin * (double)B * G;
  const bool persistent = ctx->seq_kernels && deferred && dx_all && T >= 2 && T <= kDbMaxSteps && attrs->weightnoise_std == 0.f &&
                          dyb200_lstm_bwd_tiling(ctx, I, H, B, &tl) && dyb200_tc_eligible(Imin, B, flops_small) &&
                          dyb200_tc_eligible(G, Imin, flops_small) && Wx->nd == 2 && Wx->d[0] == G && Wx->d[1] == I && Wh->nd == 2 &&
                          Wh->d[0] == G && Wh->d[1] == H && t_size(db) == G && aligned16(gates_all->v) && aligned16(c_all->v) &&
                          aligned16(c0->v) && aligned16(dh_all->v) && aligned16(dc_all->v) && aligned16(dx_all->v) &&
                          (!mx || (aligned16(mx) && aligned16(mh) && (mask_x->bd == B || mask_x->bd == 1) &&
                                   (mask_h->bd == B || mask_h->bd == 1) && t_dim(mask_x, 0) == I && t_dim(mask_h, 0) == H));
  const uint32_t bn = tl.bn, ncb = tl.ncb, S = tl.S;
  const uint32_t tiles_m = (I + H + BM - 1) / BM, tiles_n = B / bn, kb = G / 32;
  if (persistent) {
    { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
    DYB_CHECK_ARG(ctx, dyb200_wgrad_rows(deferred) == G, "lstm_seq_bwd: the deferred accumulator has %u rows, the layer %u", dyb200_wgrad_rows(deferred), G);
    PackedOp wT, dn;
    if ((rc = dyb200_tc_param2(ctx, Wx->v, I, Wh->v, H, G, true, G, &wT))) return rc;
    // the gate-gradient planes of all steps are the accumulator's A planes (columns [0, T B))
    dn.rows = T * B; dn.K = G;
    if ((rc = dyb200_wgrad_reserve_a_at(deferred, 0, T * B, &dn.hi, &dn.lo, &dn.pitch, ctx))) return rc;
    const uint32_t btiles = B / 32, tiles = tiles_m * tiles_n;
    void *pp, *pw = nullptr, *pc;
    if ((rc = dyb200_scratch(ctx, (size_t)T * btiles * G * sizeof(float), &pp))) return rc;
    if (S > 1 && (rc = dyb200_scratch(ctx, (size_t)tiles * S * bn * BM * sizeof(float), &pw))) return rc;
    if ((rc = dyb200_scratch(ctx, 256 * sizeof(uint32_t), &pc))) return rc;
    DYB_CUDA(ctx, cudaMemsetAsync(pc, 0, 256 * sizeof(uint32_t), ctx->stream));
    TmapPack tm;
    memset(&tm, 0, sizeof(tm));
    if ((rc = dyb200_tc_make_tmap(ctx, &tm.t[0], wT.hi, I + H, G, wT.pitch, BM))) return rc;
    if ((rc = dyb200_tc_make_tmap(ctx, &tm.t[1], wT.lo, I + H, G, wT.pitch, BM))) return rc;
    if ((rc = dyb200_tc_make_tmap(ctx, &tm.t[2], dn.hi, T * B, G, dn.pitch, bn))) return rc;
    if ((rc = dyb200_tc_make_tmap(ctx, &tm.t[3], dn.lo, T * B, G, dn.pitch, bn))) return rc;
    SeqBwd a;
    memset(&a, 0, sizeof(a));
    a.T = T; a.B = B; a.H = H; a.I = I; a.kb = kb; a.ncb = ncb;
    a.gates = gates_all->v; a.cs = c_all->v; a.c0 = c0->v; a.dh = dh_all->v; a.dc = dc_all->v; a.dx = dx_all->v;
    a.dn_hi = dn.hi; a.dn_lo = dn.lo; a.dn_pitch = dn.pitch;
    a.part = (float*)pp;
    a.mx = mx; a.mx_full = mx_full; a.mh = mh; a.mh_full = mh_full;
    a.ws = (float*)pw;
    a.cell_done = (uint32_t*)pc; a.gemm_done = a.cell_done + 32; a.sent = a.cell_done + 64;
    a.flags = ctx->dev_flags;
    const dim3 grid(tiles_m, tiles_n / ncb, S);
    const double flops = 2.0 * (I + H) * (double)B * G * T;
    if (S > 1) rc = bn == 64 ? launch_seq_bwd<64, true>(ctx, tm, a, grid, flops) : launch_seq_bwd<128, true>(ctx, tm, a, grid, flops);
    else rc = bn == 64 ? launch_seq_bwd<64, false>(ctx, tm, a, grid, flops) : launch_seq_bwd<128, false>(ctx, tm, a, grid, flops);
    if (rc) return rc;
    dyb_launch(k_seq_db_reduce, (G + 31) / 32, 256, 0, ctx, (const float*)pp, T, btiles, G, db->v);
    DYB_LAUNCHED(ctx);
    first = 0;
  }

  // ---- without the kernel: one call per time step ----
  for (uint32_t t = first; t-- > 0;) {
    dyb200_tensor x = *x_all, hp = *h0, cp = *c0, g = *gates_all, c = *c_all, dh = *dh_all, dc = *dc_all, dx, dhp = *dh_all, dcp = *dc_all;
    x.bd = B; x.v = x_all->v + (size_t)t * IB;
    g.bd = B; g.v = gates_all->v + (size_t)t * 4 * HB;
    c.bd = B; c.v = c_all->v + (size_t)t * HB;
    dh.bd = B; dh.v = dh_all->v + (size_t)t * HB;
    dc.bd = B; dc.v = dc_all->v + (size_t)t * HB;
    if (dx_all) { dx = *dx_all; dx.bd = B; dx.v = dx_all->v + (size_t)t * IB; }
    if (t > 0) {
      hp.v = h_all->v + (size_t)(t - 1) * HB; cp.v = c_all->v + (size_t)(t - 1) * HB;
      dhp.bd = B; dhp.v = dh_all->v + (size_t)(t - 1) * HB;
      dcp.bd = B; dcp.v = dc_all->v + (size_t)(t - 1) * HB;
    }
    if ((rc = dyb200_vanilla_lstm_bwd_fused_at(&x, &hp, &cp, Wx, Wh, mask_x, mask_h, &g, &c, &dh, &dc, dx_all ? &dx : nullptr,
                                               t > 0 ? &dhp : nullptr, t > 0 ? &dcp : nullptr, dWx, dWh, db, attrs, deferred,
                                               deferred ? t * B : DYB200_WGRAD_APPEND, ctx)))
      return rc;
  }
  return DYB200_OK;
}

}  // extern "C"
