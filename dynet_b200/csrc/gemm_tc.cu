// 3xTF32 GEMM on the 5th-generation tensor cores: tcgen05.mma (kind::tf32) with the accumulator
// in TMEM, operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle, no
// multicast), one CTA per 128 x 128 output tile.
//
// fp32 accuracy from TF32 hardware: every operand x is split as x = hi + lo with hi = tf32(x) and
// lo = tf32(x - hi); the product a*b is accumulated as a_lo*b_hi + a_hi*b_lo + a_hi*b_hi (the
// lo*lo term, ~2^-22 relative, is dropped).  The split is done once per operand by a packing
// kernel that also brings the operand to K-major order (the reduction index contiguous) and
// applies the dropout mask, so the GEMM kernel itself only moves tiles and issues MMAs:
//   warp 0     TMA producer: 4 tiles (A_hi, A_lo, B_hi, B_lo) per 32-wide k-block, 3-stage ring
//   warp 1     allocates TMEM, issues 3 MMAs per 8-wide k-step, commits to the ring's mbarriers;
//              the accumulation chain is cut every kChunkKB k-blocks (two TMEM accumulators, used alternately)
//   warps 2-9  add every finished chunk (tcgen05.ld of their 32 accumulator lanes x 64 columns) into fp32
//              registers, park the finished tile in the idle operand ring and run the epilogue as a short
//              cooperative loop over it: 16-byte accesses along the rows (whole 512-byte tile columns per warp),
//              read-modify-write epilogues with 8 loads in flight; the LSTM epilogue reads the four gates of a
//              hidden unit from the tile and also forms c and h
// Products with few output tiles are split along K over blockIdx.z; the splits store raw partial
// tiles and a second kernel adds them in split order and applies the epilogue (deterministic).
// Products with more tiles than SMs run on a persistent variant (one CTA per SM walks the tiles) whose
// epilogue overlaps the next tile's main loop.
// Every mbarrier wait is bounded; a wait that runs out sets DYB200_FLAG_WAIT_TIMEOUT and the
// kernel still frees its TMEM and returns.

#include "tc_dev.cuh"

namespace {

// BNT = columns of the output tile: 128, or 64 for products with N <= 64 (small per-GPU batches), where a 128-wide tile
// would spend half of every MMA and half of the B traffic on padding.
// CLUSTER: the gridDim.z K-splits of a tile form one thread-block cluster (1 x 1 x S); every CTA parks its partial tile in
// its own shared memory, and CTA r adds all partial tiles of its 1 / S of the columns through distributed shared memory, in
// split order, and runs the epilogue on that slice - no workspace round trip and no second kernel.
template <int BNT, bool CLUSTER>
__global__ void __launch_bounds__(kThreads, 1) k_gemm_tc(const __grid_constant__ TmapPack tm, uint32_t M, uint32_t N,
                                                         uint32_t kb0, uint32_t kb1, uint32_t kb_per_split,
                                                         GemmEpilogue epi, uint32_t* flags) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // (the wait comes after the prologue, below)
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int TILE_B_BYTES = BNT * BK * 4;                      // one B plane of a stage
  constexpr int STAGE_TX = 2 * TILE_BYTES + 2 * TILE_B_BYTES;     // bytes a stage receives (stages stay STAGE_BYTES apart)
  const uint32_t m0 = blockIdx.x * BM, n0 = blockIdx.y * BNT;
  // K splits: split z of S takes the z-th share of EACH pair's k-blocks (pair 0 first, then pair 1), so that in
  // Wx x + Wh h every split holds the same mix of the two products (the sequence-persistent LSTM kernel relies on
  // it: only the Wh h share of a split waits for the previous time step).  With one pair this is the plain contiguous cut.
  const KSplit ks = k_split(kb0, kb1, blockIdx.z, gridDim.z);
  const uint32_t total = ks.n0 + ks.n1;
  (void)kb_per_split;
  const uint32_t nchunks = (total + kChunkKB - 1) / kChunkKB;
  if (!CLUSTER && gridDim.z > 1) epi.C += (size_t)blockIdx.z * epi.ldc * N;   // raw partial tile of this split (mode is EPI_STORE)
  __shared__ uint32_t split_ok;   // CLUSTER: this CTA's partial tile is complete

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int q = 0; q < 2; ++q) { mbar_init(&acc_full[q], 1); mbar_init(&acc_empty[q], kEpiWarps); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (threadIdx.x == 32 * 2) {   // (an epilogue thread, idle until the first chunk is done) descriptors of the first loads
#pragma unroll
    for (int q = 0; q < 8; ++q) asm volatile("prefetch.tensormap [%0];" ::"l"(&tm.t[q]) : "memory");
  }
  if (warp == 1) {   // the whole warp allocates the accumulator columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  // Barrier initialisation and the TMEM allocation above may overlap the previous kernel of the stream; nothing below
  // (TMA loads, c_prev prefetch, stores) starts before that kernel has completed.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      for (uint32_t it = 0; it < total; ++it) {
        if (!mbar_wait(&empty_bar[s], ph ^ 1)) { atomicOr(flags, DYB200_FLAG_WAIT_TIMEOUT); break; }
        const uint32_t pair = it < ks.n0 ? 0 : 1, kblk = pair ? ks.b1 + (it - ks.n0) : ks.b0 + it;
        unsigned char* st = ring + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_TX);
        load_a_tile(st, &tm.t[4 * pair + 0], &full_bar[s], kblk, m0, tm.a_mn);
        load_a_tile(st + TILE_BYTES, &tm.t[4 * pair + 1], &full_bar[s], kblk, m0, tm.a_mn);
        load_b_tile(st + 2 * TILE_BYTES, &tm.t[4 * pair + 2], &full_bar[s], kblk, n0, tm.b_mn);
        load_b_tile(st + 2 * TILE_BYTES + TILE_B_BYTES, &tm.t[4 * pair + 3], &full_bar[s], kblk, n0, tm.b_mn);
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
    if (CLUSTER) {   // all lanes: the two cluster barriers of the epilogue warps (see there)
      __syncwarp();
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // This one thread issues every MMA of the tile, and the tensor pipe is only as busy as this loop is short:
      // descriptors of the three stages are built once, stage / phase / chunk counters are carried instead of divided,
      // and the 12 MMAs of a k-block go out in one block of PTX.
      // instruction descriptor: D = f32, A = B = tf32, both K-major, N = BNT, M = 128
      // (bits 15 / 16: A / B is MN-major)
      const uint32_t a_mn = tm.a_mn, b_mn = tm.b_mn;
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BNT >> 3) << 17) | ((uint32_t)(BM >> 4) << 24) |
                             (a_mn ? 1u << 15 : 0u) | (b_mn ? 1u << 16 : 0u);
      const uint64_t a_step = a_mn ? 64 : 2, b_step = b_mn ? 64 : 2;
      uint64_t d_a_hi[STAGES], d_a_lo[STAGES], d_b_hi[STAGES], d_b_lo[STAGES];
#pragma unroll
      for (int q = 0; q < STAGES; ++q) {
        const uint32_t base = smem_u32(ring + (size_t)q * STAGE_BYTES);
        d_a_hi[q] = a_mn ? umma_desc_mn(base) : umma_desc(base);
        d_a_lo[q] = a_mn ? umma_desc_mn(base + TILE_BYTES) : umma_desc(base + TILE_BYTES);
        d_b_hi[q] = b_mn ? umma_desc_mn(base + 2 * TILE_BYTES) : umma_desc(base + 2 * TILE_BYTES);
        d_b_lo[q] = b_mn ? umma_desc_mn(base + 2 * TILE_BYTES + TILE_B_BYTES) : umma_desc(base + 2 * TILE_BYTES + TILE_B_BYTES);
      }
      // The tensor core truncates when it aligns addends to the accumulator, a bias that grows with the length of
      // the accumulation chain.  So the chain is cut every kChunkKB k-blocks: chunk c accumulates into TMEM buffer
      // c & 1 from zero, and the epilogue warps add finished chunks into fp32 registers with ordinary rounding.
      uint32_t s = 0, ph = 0, in_chunk = 0, chunk = 0, buf = 0;
      for (uint32_t it = 0; it < total; ++it) {
        if (in_chunk == 0 && chunk >= 2) {   // buffer reuse: the epilogue warps must have drained chunk - 2
          if (!mbar_wait(&acc_empty[buf], ((chunk >> 1) - 1) & 1)) { atomicOr(flags, DYB200_FLAG_WAIT_TIMEOUT); break; }
        }
        if (!mbar_wait(&full_bar[s], ph)) { atomicOr(flags, DYB200_FLAG_WAIT_TIMEOUT); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint64_t a_hi, a_lo, b_hi, b_lo;   // select without dynamic register indexing
        if (s == 0) { a_hi = d_a_hi[0]; a_lo = d_a_lo[0]; b_hi = d_b_hi[0]; b_lo = d_b_lo[0]; }
        else if (s == 1) { a_hi = d_a_hi[1]; a_lo = d_a_lo[1]; b_hi = d_b_hi[1]; b_lo = d_b_lo[1]; }
        else { a_hi = d_a_hi[2]; a_lo = d_a_lo[2]; b_hi = d_b_hi[2]; b_lo = d_b_lo[2]; }
        const uint32_t acc = tmem_base + buf * BN;
        issue_kblock(acc, a_hi, a_lo, b_hi, b_lo, idesc, in_chunk, a_step, b_step);
        umma_commit(&empty_bar[s]);   // frees the stage once these MMAs have read it
        const bool chunk_ends = in_chunk == kChunkKB - 1 || it == total - 1;
        if (chunk_ends) { umma_commit(&acc_full[buf]); in_chunk = 0; ++chunk; buf ^= 1; }
        else ++in_chunk;
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
    if (CLUSTER) {
      __syncwarp();
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
  } else {
    // epilogue warps 2..9: TMEM lanes 32*(warp % 4) .. +31 (row of the tile = lane of TMEM); warps 2-5
    // take columns 0-63, warps 6-9 columns 64-127
    const uint32_t quarter = warp & 3, half = (warp - 2) >> 2;
    const uint32_t te = threadIdx.x - 64;   // 0..255 among the epilogue threads
    // EPI_LSTM_CELL: in the cooperative pass below this thread owns hidden units [4 (te % 8), +4) of the tile's 32 for
    // the columns te / 8 + 32 k; their previous cell states are fetched now, while the MMAs run
    float4 cprev[4];
    if (epi.mode == EPI_LSTM_CELL) {
      const uint32_t u = blockIdx.x * 32 + 4 * (te & 7);
#pragma unroll
      for (int k = 0; k < BNT / 32; ++k) {
        const uint32_t n = n0 + (te >> 3) + 32 * k;
        cprev[k] = n < N ? ld4(epi.c_prev + u + (size_t)epi.H * n) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    float sum[64];   // this thread's row of the tile, columns [64 half, 64 half + 64)
#pragma unroll
    for (int j = 0; j < 64; ++j) sum[j] = 0.f;
    bool ok = true;
#pragma unroll 1
    for (uint32_t c = 0; c < nchunks; ++c) {
      const uint32_t buf = c & 1;
      if (!mbar_wait(&acc_full[buf], (c >> 1) & 1)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (64 * half < BNT) {   // (with a 64-column tile the second column half does not exist)
        // (two 32-column loads: one 64-column load per flush measured slower)
        float v[32];
        const uint32_t taddr = tmem_base + buf * BN + ((quarter * 32) << 16) + 2 * half * 32;
        tmem_ld32(taddr, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[j] += v[j];
        tmem_ld32(taddr + 32, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[32 + j] += v[j];
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (!ok && lane == 0) atomicOr(flags, DYB200_FLAG_WAIT_TIMEOUT);
    // The tile goes through shared memory (the operand ring is idle once the last chunk has been drained: every MMA
    // has completed and no TMA load is in flight), stored like C: column-major, 128 rows per column.  The pass that
    // follows is a short rolled loop in which consecutive threads take consecutive rows, so global accesses are
    // 16-byte vectors covering whole 512-byte columns of the tile.  Every epilogue warp reaches the named barrier,
    // whatever its waits did; a failed wait anywhere cancels the stores.
    float* tile = reinterpret_cast<float*>(ring);
    if (64 * half < BNT) {
      float* col = tile + (size_t)(64 * half) * BM + quarter * 32 + lane;
#pragma unroll
      for (int j = 0; j < 64; ++j) col[(size_t)j * BM] = sum[j];
    }
    uint32_t all_ok;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.cta.red.and.pred p, 1, 256, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(all_ok) : "r"((uint32_t)ok) : "memory");
    if (!CLUSTER) {
      if (all_ok) epilogue_pass<BNT, 256>(epi, tile, te, blockIdx.x, m0, n0, M, N, cprev);
    } else {
      // every thread of every CTA of the cluster takes part in the two cluster barriers below (the TMA and MMA warps
      // reach them further down); between them rank 0 reads the other CTAs' tiles
      if (te == 0) split_ok = all_ok;
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
      {
        // Rank r (= blockIdx.z: the cluster is 1 x 1 x gridDim.z) finishes columns [c_lo, c_hi) of the tile: it adds the
        // S partial tiles of that slice in split order (the order of the split-K reduction kernel), its own from its
        // shared memory and the others through distributed shared memory, and runs the epilogue on the slice.
        const uint32_t S = gridDim.z, rank = blockIdx.z;
        const uint32_t w = ((BNT + S - 1) / S + 7) & ~7u;
        const uint32_t c_lo = min(rank * w, (uint32_t)BNT), c_hi = min(c_lo + w, (uint32_t)BNT);
        uint32_t ok_all = all_ok, base[8];
        for (uint32_t r = 0; r < S; ++r) {
          uint32_t ra, v;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(&split_ok)), "r"(r));
          asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(ra) : "memory");
          ok_all &= v;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(base[r & 7]) : "r"(smem_u32(tile)), "r"(r));
        }
        if (ok_all) {
          const uint32_t f_lo = c_lo * (BM / 4), f_hi = c_hi * (BM / 4);   // 16-byte pieces of the slice
          float4* t4 = reinterpret_cast<float4*>(tile);
          for (uint32_t f = f_lo + te; f < f_hi; f += 256) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t r = 0; r < S; ++r) {
              float4 pv;
              asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                           : "=f"(pv.x), "=f"(pv.y), "=f"(pv.z), "=f"(pv.w) : "r"(base[r & 7] + 16u * f) : "memory");
              if (r == 0) acc = pv;
              else { acc.x += pv.x; acc.y += pv.y; acc.z += pv.z; acc.w += pv.w; }
            }
            t4[f] = acc;
          }
          asm volatile("barrier.cta.sync 1, 256;" ::: "memory");   // the pass below reads other threads' pieces
          epilogue_pass<BNT, 256>(epi, tile, te, blockIdx.x, m0, n0, M, N, cprev, c_lo, c_hi);
        } else if (te == 0 && rank == 0) {
          atomicOr(flags, DYB200_FLAG_WAIT_TIMEOUT);
        }
      }
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");   // every tile stays until all ranks have read it
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---- persistent variant for products with more tiles than SMs -----------------------------------------------------------
// One CTA per SM walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ... (the same order in which the one-tile kernel's
// CTAs would run, so CTAs that share operand tiles still work on the same k-blocks at the same time).  The epilogue of a
// tile runs while the TMA and MMA warps are already on the next one: the finished tile waits in the epilogue warps'
// registers (the TMEM accumulators are free again as soon as their last chunk is drained) and goes through a 32 KiB
// staging buffer beside the operand ring, one 64-column half at a time: warps 2-5 park and write out columns 0-63, then
// warps 6-9 columns 64-127.  What this saves is the pipeline fill and the epilogue of every tile but the last, about
// 9 us per tile: a third of the time of the output layer's product (K = 1024, 75 tiles per SM).
constexpr int SMEM_PERSIST_BYTES = SMEM_BYTES + BM * 64 * 4;
// Four accumulators (all 512 TMEM columns): the MMA warp may run four chunks - a whole tile of the output layer's
// product - ahead of the epilogue warps, which drain nothing while they write out the previous tile.
constexpr uint32_t kPersistBufs = 4;

// Tile order.  gm == 0: row block fastest (the launch order of the one-tile kernel).  gm > 0: groups of gm row blocks, row
// block fastest within a group, then the column block, then the next group.  The 148 tiles in flight then touch gm A
// blocks and ~148 / gm B blocks instead of all A blocks and two B blocks, and the A blocks of a group stay in L2 while
// the B blocks stream past them (output layer, gm = 16: 25 MB of operands per round instead of 83 MB).
__device__ __forceinline__ void persist_tile_coords(uint32_t tile, uint32_t tiles_m, uint32_t tiles_n, uint32_t gm, uint32_t& mt,
                                                    uint32_t& nt) {
  if (gm == 0) { mt = tile % tiles_m; nt = tile / tiles_m; return; }
  const uint32_t per_group = gm * tiles_n;
  const uint32_t g = tile / per_group, r = tile - g * per_group;
  const uint32_t rows = min(gm, tiles_m - g * gm);   // the last group may be lower
  nt = r / rows;
  mt = g * gm + r % rows;
}

// The two single-thread roles are functions of their own: their loops pace the tensor pipe and keep their own registers.
template <int BNT>
__device__ __noinline__ void persist_producer(const TmapPack* tm, unsigned char* ring, uint64_t* full_bar, uint64_t* empty_bar,
                                              uint32_t tiles, uint32_t tiles_m, uint32_t tiles_n, uint32_t gm, uint32_t kb0,
                                              uint32_t kb1, uint32_t S, uint32_t* flags) {
  constexpr int TILE_B_BYTES = BNT * BK * 4;
  constexpr int STAGE_TX = 2 * TILE_BYTES + 2 * TILE_B_BYTES;
  uint32_t s = 0, ph = 0;
  bool fail = false;
  // work item w = (K split z, tile): all tiles of split 0 first, so that the CTAs of a round share operand k-blocks
  for (uint32_t w = blockIdx.x; w < tiles * S && !fail; w += gridDim.x) {
    const uint32_t z = w / tiles, tile = w - z * tiles;
    const KSplit ks = k_split(kb0, kb1, z, S);
    uint32_t mt, nt;
    persist_tile_coords(tile, tiles_m, tiles_n, gm, mt, nt);
    const uint32_t m0 = mt * BM, n0 = nt * BNT;
    for (uint32_t g = 0; g < ks.n0 + ks.n1; ++g) {
      if (!mbar_wait(&empty_bar[s], ph ^ 1)) { fail = true; break; }
      const uint32_t pair = g < ks.n0 ? 0 : 1, kblk = pair ? ks.b1 + (g - ks.n0) : ks.b0 + g;
      unsigned char* st = ring + (size_t)s * STAGE_BYTES;
      mbar_expect_tx(&full_bar[s], STAGE_TX);
      load_a_tile(st, &tm->t[4 * pair + 0], &full_bar[s], kblk, m0, tm->a_mn);
      load_a_tile(st + TILE_BYTES, &tm->t[4 * pair + 1], &full_bar[s], kblk, m0, tm->a_mn);
      load_b_tile(st + 2 * TILE_BYTES, &tm->t[4 * pair + 2], &full_bar[s], kblk, n0, tm->b_mn);
      load_b_tile(st + 2 * TILE_BYTES + TILE_B_BYTES, &tm->t[4 * pair + 3], &full_bar[s], kblk, n0, tm->b_mn);
      if (++s == STAGES) { s = 0; ph ^= 1; }
    }
  }
  if (fail) atomicOr(flags, DYB200_FLAG_WAIT_TIMEOUT);
}

template <int BNT>
__device__ __noinline__ void persist_issue(unsigned char* ring, uint64_t* full_bar, uint64_t* empty_bar, uint64_t* acc_full,
                                           uint64_t* acc_empty, uint32_t tmem_base, uint32_t tiles, uint32_t kb0, uint32_t kb1, uint32_t S,
                                           uint32_t a_mn, uint32_t b_mn, uint32_t* flags) {
  constexpr int TILE_B_BYTES = BNT * BK * 4;
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BNT >> 3) << 17) | ((uint32_t)(BM >> 4) << 24) |
                         (a_mn ? 1u << 15 : 0u) | (b_mn ? 1u << 16 : 0u);
  const uint64_t a_step = a_mn ? 64 : 2, b_step = b_mn ? 64 : 2;
  uint64_t d_a_hi[STAGES], d_a_lo[STAGES], d_b_hi[STAGES], d_b_lo[STAGES];
#pragma unroll
  for (int q = 0; q < STAGES; ++q) {
    const uint32_t base = smem_u32(ring + (size_t)q * STAGE_BYTES);
    d_a_hi[q] = a_mn ? umma_desc_mn(base) : umma_desc(base);
    d_a_lo[q] = a_mn ? umma_desc_mn(base + TILE_BYTES) : umma_desc(base + TILE_BYTES);
    d_b_hi[q] = b_mn ? umma_desc_mn(base + 2 * TILE_BYTES) : umma_desc(base + 2 * TILE_BYTES);
    d_b_lo[q] = b_mn ? umma_desc_mn(base + 2 * TILE_BYTES + TILE_B_BYTES) : umma_desc(base + 2 * TILE_BYTES + TILE_B_BYTES);
  }
  // stage, phase and chunk counters run on across tiles; an accumulation chain never crosses a tile boundary
  uint32_t s = 0, ph = 0, chunk = 0, buf = 0;
  bool fail = false;
  for (uint32_t w = blockIdx.x; w < tiles * S && !fail; w += gridDim.x) {
    const KSplit ks = k_split(kb0, kb1, w / tiles, S);
    const uint32_t kb = ks.n0 + ks.n1;
    uint32_t in_chunk = 0;
    for (uint32_t it = 0; it < kb; ++it) {
      if (in_chunk == 0 && chunk >= kPersistBufs) {
        if (!mbar_wait(&acc_empty[buf], ((chunk / kPersistBufs) - 1) & 1)) { fail = true; break; }
      }
      if (!mbar_wait(&full_bar[s], ph)) { fail = true; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint64_t a_hi, a_lo, b_hi, b_lo;
      if (s == 0) { a_hi = d_a_hi[0]; a_lo = d_a_lo[0]; b_hi = d_b_hi[0]; b_lo = d_b_lo[0]; }
      else if (s == 1) { a_hi = d_a_hi[1]; a_lo = d_a_lo[1]; b_hi = d_b_hi[1]; b_lo = d_b_lo[1]; }
      else { a_hi = d_a_hi[2]; a_lo = d_a_lo[2]; b_hi = d_b_hi[2]; b_lo = d_b_lo[2]; }
      const uint32_t acc = tmem_base + buf * BN;
      issue_kblock(acc, a_hi, a_lo, b_hi, b_lo, idesc, in_chunk, a_step, b_step);
      umma_commit(&empty_bar[s]);
      const bool chunk_ends = in_chunk == kChunkKB - 1 || it == kb - 1;
      if (chunk_ends) { umma_commit(&acc_full[buf]); in_chunk = 0; ++chunk; buf = chunk % kPersistBufs; }
      else ++in_chunk;
      if (++s == STAGES) { s = 0; ph ^= 1; }
    }
  }
  if (fail) atomicOr(flags, DYB200_FLAG_WAIT_TIMEOUT);
}


template <int BNT>
__global__ void __launch_bounds__(kThreads, 1) k_gemm_persist(const __grid_constant__ TmapPack tm, uint32_t M, uint32_t N,
                                                              uint32_t kb0, uint32_t kb1, uint32_t tiles_m, uint32_t tiles,
                                                              uint32_t gm, uint32_t S, GemmEpilogue epi, uint32_t* flags) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[kPersistBufs], acc_empty[kPersistBufs];
  __shared__ uint32_t tmem_base_slot;
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* stage = reinterpret_cast<float*>(ring + (size_t)STAGES * STAGE_BYTES);   // 64 columns x BM rows
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (uint32_t q = 0; q < kPersistBufs; ++q) { mbar_init(&acc_full[q], 1); mbar_init(&acc_empty[q], kEpiWarps); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kPersistBufs * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) persist_producer<BNT>(&tm, ring, full_bar, empty_bar, tiles, tiles_m, (N + BNT - 1) / BNT, gm, kb0, kb1, S, flags);
  } else if (warp == 1) {
    if (lane == 0) persist_issue<BNT>(ring, full_bar, empty_bar, acc_full, acc_empty, tmem_base, tiles, kb0, kb1, S, tm.a_mn, tm.b_mn, flags);
  } else {
    // epilogue warps 2..9: TMEM lanes 32 (warp % 4) .. +31; warps 2-5 hold columns 0-63 of the tile, warps 6-9 columns 64-127
    const uint32_t quarter = warp & 3, half = (warp - 2) >> 2;
    const uint32_t th = (threadIdx.x - 64) & 127;   // 0..127 within this half's four warps
    const bool has_cols = 64 * half < BNT;
    uint32_t cg = 0;   // chunks drained so far (selects the TMEM buffer and the barrier phase)
    bool ok = true;
#pragma unroll 1
    for (uint32_t w = blockIdx.x, j = 0; w < tiles * S; w += gridDim.x, ++j) {
      const uint32_t z = w / tiles, tile = w - z * tiles;
      const KSplit ks = k_split(kb0, kb1, z, S);
      const uint32_t nchunks = (ks.n0 + ks.n1 + kChunkKB - 1) / kChunkKB;
      // (K splits: epi is a plain store with ldc = M into S partial products side by side, so split z writes columns z N ..)
      const uint32_t n_shift = z * N;
      uint32_t mt, nt;
      persist_tile_coords(tile, tiles_m, (N + BNT - 1) / BNT, gm, mt, nt);
      const uint32_t m0 = mt * BM, n0 = nt * BNT + 64 * half;
      float sum[64];
#pragma unroll
      for (int q = 0; q < 64; ++q) sum[q] = 0.f;
#pragma unroll 1
      for (uint32_t c = 0; c < nchunks; ++c, ++cg) {
        const uint32_t buf = cg % kPersistBufs;
        if (!ok) continue;
        if (!mbar_wait(&acc_full[buf], (cg / kPersistBufs) & 1)) { ok = false; continue; }
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
      if (!has_cols) continue;   // (64-column tiles: warps 6-9 only take part in the accumulator hand-shake)
      // The staging buffer is free once the other half has written out its columns of the previous turn (128-column
      // tiles), or once this half's own warps have all left the previous pass (64-column tiles).
      if (BNT == 128) {
        if (half == 1) bar_sync(2, 256);
        else if (j > 0) bar_sync(4, 256);
      } else if (j > 0) {
        bar_sync(2, 128);
      }
      {
        float* col = stage + quarter * 32 + lane;
#pragma unroll
        for (int q = 0; q < 64; ++q) col[(size_t)q * BM] = sum[q];
      }
      float4 cprev[4];
      if (epi.mode == EPI_LSTM_CELL) {
        const uint32_t u = mt * 32 + 4 * (th & 7);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t n = n0 + (th >> 3) + 16 * k;
          cprev[k] = n < N ? ld4(epi.c_prev + u + (size_t)epi.H * n) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      uint32_t all_ok;
      asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.cta.red.and.pred p, %2, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(all_ok) : "r"((uint32_t)ok), "r"(1u + 2u * half) : "memory");
      if (all_ok) epilogue_pass<64, 128>(epi, stage, th, mt, m0, n0 + n_shift, M, N + n_shift, cprev);
      if (BNT == 128) {
        if (half == 0) bar_arrive(2, 256);
        else if (w + gridDim.x < tiles * S) bar_arrive(4, 256);
      }
    }
    if (!ok && lane == 0) atomicOr(flags, DYB200_FLAG_WAIT_TIMEOUT);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kPersistBufs * BN) : "memory");
  }
}

// ---- split-K second stage: C = epilogue(sum_s part[s]) in ascending split order ----------------
__global__ void __launch_bounds__(256) k_splitk_reduce(const float* __restrict__ part, uint32_t S, uint32_t M, uint32_t N,
                                                      GemmEpilogue epi, int vec) {
  dyb_grid_dep_sync();
  const size_t MN = (size_t)M * N;
  if (vec) {   // M % 4 == 0 and 16-byte aligned C / mask: four rows of one column per thread
    const size_t MN4 = MN / 4;
    for (size_t q = (size_t)blockIdx.x * 256 + threadIdx.x; q < MN4; q += (size_t)gridDim.x * 256) {
      const size_t e = 4 * q;
      const uint32_t m = (uint32_t)(e % M), n = (uint32_t)(e / M);
      float4 acc = ld4_stream(part + e);
      for (uint32_t s2 = 1; s2 < S; ++s2) {
        float4 v = ld4_stream(part + (size_t)s2 * MN + e);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      const EpiRow row = epi_row(epi, m);   // split_m is a multiple of 4 here: the four rows share a destination
      float* dst = row.c + (size_t)row.ldc * n;
      if (epi.mode == EPI_STORE) st4(dst, acc);
      else if (epi.mode == EPI_BIAS) {
        float4 b = ld4(epi.bias + m);
        st4(dst, make_float4(acc.x + b.x, acc.y + b.y, acc.z + b.z, acc.w + b.w));
      } else if (epi.mode == EPI_ACCUM) {
        float4 o = ld4(dst);
        st4(dst, make_float4(o.x + acc.x, o.y + acc.y, o.z + acc.z, o.w + acc.w));
      } else {   // EPI_ACCUM_MASK
        float4 o = ld4(dst), mk = ld4(row.mask + (row.mask_full ? (size_t)row.mask_ld * n : 0));
        st4(dst, make_float4(__fmaf_rn(acc.x, mk.x, o.x), __fmaf_rn(acc.y, mk.y, o.y), __fmaf_rn(acc.z, mk.z, o.z), __fmaf_rn(acc.w, mk.w, o.w)));
      }
    }
    return;
  }
  for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < MN; e += (size_t)gridDim.x * 256) {
    const uint32_t m = (uint32_t)(e % M), n = (uint32_t)(e / M);
    float acc = 0.f;
    for (uint32_t s2 = 0; s2 < S; ++s2) acc += part[(size_t)s2 * MN + e];
    const EpiRow row = epi_row(epi, m);
    float* dst = row.c + (size_t)row.ldc * n;
    if (epi.mode == EPI_STORE) *dst = acc;
    else if (epi.mode == EPI_BIAS) *dst = acc + epi.bias[m];
    else if (epi.mode == EPI_ACCUM) *dst += acc;
    else if (epi.mode == EPI_GATES) {
      acc += epi.bias[m] + ((m >= epi.H && m < 2 * epi.H) ? epi.forget_bias : 0.f);
      *dst = m < 3 * epi.H ? gate_sigmoid(acc) : gate_tanh(acc);   // (the activations of every gate epilogue)
    } else {
      *dst = __fmaf_rn(acc, row.mask[row.mask_full ? (size_t)row.mask_ld * n : 0], *dst);
    }
  }
}

// Split-K second stage of the LSTM forward product (EPI_LSTM_CELL): rows are the interleaved gate rows of
// dyb200_tc_param_gates.  One thread owns four consecutive hidden units of one column: it adds the partial tiles in
// split order, applies bias + sigmoid / tanh, writes the four gate rows and forms c and h.
__global__ void __launch_bounds__(256) k_splitk_reduce_cell(const float* __restrict__ part, uint32_t S, uint32_t M, uint32_t N,
                                                           GemmEpilogue epi) {
  dyb_grid_dep_sync();
  const uint32_t H = epi.H, H4 = H / 4;
  const size_t MN = (size_t)M * N, total = (size_t)H4 * N;
  for (size_t q = (size_t)blockIdx.x * 256 + threadIdx.x; q < total; q += (size_t)gridDim.x * 256) {
    const uint32_t u = 4 * (uint32_t)(q % H4), n = (uint32_t)(q / H4);
    const uint32_t row0 = 128 * (u / 32) + (u % 32);   // interleaved row of gate 0; gate g is 32 g rows further
    float4 a[4];
    // all loads of up to four splits are issued before the first add (this kernel is latency-bound at small batch)
    for (uint32_t s0 = 0; s0 < S; s0 += 4) {
      float4 v[4][4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int g = 0; g < 4; ++g)
          v[k][g] = s0 + k < S ? ld4_stream(part + row0 + 32 * g + (size_t)M * n + (size_t)(s0 + k) * MN) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (s0 == 0) a[g] = v[0][g];
        else { a[g].x += v[0][g].x; a[g].y += v[0][g].y; a[g].z += v[0][g].z; a[g].w += v[0][g].w; }
#pragma unroll
        for (int k = 1; k < 4; ++k)
          if (s0 + k < S) { a[g].x += v[k][g].x; a[g].y += v[k][g].y; a[g].z += v[k][g].z; a[g].w += v[k][g].w; }
      }
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const float4 b = ld4(epi.bias + (size_t)g * H + u);
      const float fb = g == 1 ? epi.forget_bias : 0.f;
      a[g].x += b.x + fb; a[g].y += b.y + fb; a[g].z += b.z + fb; a[g].w += b.w + fb;
      if (g == 3) a[g] = make_float4(gate_tanh(a[g].x), gate_tanh(a[g].y), gate_tanh(a[g].z), gate_tanh(a[g].w));
      else a[g] = make_float4(gate_sigmoid(a[g].x), gate_sigmoid(a[g].y), gate_sigmoid(a[g].z), gate_sigmoid(a[g].w));
      st4(epi.C + (size_t)g * H + u + (size_t)epi.ldc * n, a[g]);
    }
    const size_t e = u + (size_t)H * n;
    const float4 cp = ld4(epi.c_prev + e);
    const float4 c = make_float4(lstm_cell_c(a[0].x, a[3].x, a[1].x, cp.x), lstm_cell_c(a[0].y, a[3].y, a[1].y, cp.y),
                                 lstm_cell_c(a[0].z, a[3].z, a[1].z, cp.z), lstm_cell_c(a[0].w, a[3].w, a[1].w, cp.w));
    st4(epi.c_out + e, c);
    const float4 hv = make_float4(lstm_cell_h(a[2].x, c.x), lstm_cell_h(a[2].y, c.y), lstm_cell_h(a[2].z, c.z), lstm_cell_h(a[2].w, c.w));
    st4(epi.h_out + e, hv);
    if (epi.hn_hi) epi_emit_h(epi, u, n, hv);
  }
}

// ---- operand packing: fp32 (masked, possibly transposed) -> K-major hi / lo planes ------------
// One launch packs up to kMaxPackJobs operands.  A job is cut into units of one CTA each: for a source whose
// k index is fast (element (r, k) at src[k + ld * r]) a unit is 1024 consecutive k of one row; for a source whose
// row index is fast (element (r, k) at src[r + ld * k]) a unit is a 32 x 32 tile transposed through shared memory.
__global__ void __launch_bounds__(256) k_pack_multi(const PackJobs jobs) {
  dyb_grid_dep_sync();
  __shared__ float tile[32][33];
  int j = 0;
#pragma unroll
  for (int q = 1; q < kMaxPackJobs; ++q) if (q < jobs.n && blockIdx.x >= jobs.start[q]) j = q;
  const PackJob& job = jobs.job[j];
  const uint32_t unit = blockIdx.x - jobs.start[j];
  const float* __restrict__ src = job.src;
  const float* __restrict__ mask = job.mask;
  float* __restrict__ hi = job.hi;
  float* __restrict__ lo = job.lo;
  const uint32_t ld = job.ld, rows = job.rows, K = job.K, pitch = job.pitch, mask_ld = job.mask_ld;
  const int mask_full = job.mask_full;
  const uint32_t mask_period = job.mask_period;
  if (job.k_is_fast) {
    const uint32_t r = unit / job.gx, bx = unit % job.gx;
    const uint32_t mr = mask_period ? r % mask_period : r;   // batch column of the mask
    if (job.vec) {
      const uint32_t k = (bx * 256 + threadIdx.x) * 4;
      if (k < K) {
        float4 v = ld4(src + k + (size_t)ld * r);
        if (mask) {
          float4 mk = ld4(mask + k + (mask_full ? (size_t)mask_ld * mr : 0));
          v.x *= mk.x; v.y *= mk.y; v.z *= mk.z; v.w *= mk.w;
        }
        float4 h, l;
        split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y); split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
        st4(hi + k + (size_t)pitch * r, h);
        st4(lo + k + (size_t)pitch * r, l);
      }
    } else {
      for (uint32_t k = bx * 1024 + threadIdx.x; k < min(K, (bx + 1) * 1024); k += 256) {
        float v = src[k + (size_t)ld * r];
        if (mask) v *= mask[k + (mask_full ? (size_t)mask_ld * mr : 0)];
        float h, l;
        split_tf32(v, h, l);
        hi[k + (size_t)pitch * r] = h;
        lo[k + (size_t)pitch * r] = l;
      }
    }
    return;
  }
  const uint32_t r0 = (unit % job.gx) * 32, k0 = (unit / job.gx) * 32;
  const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t r = r0 + tx, k = k0 + ty + 8 * i;
    float v = 0.f;
    if (r < rows && k < K) {
      v = src[r + (size_t)ld * k];
      if (mask) v *= mask[r + (mask_full ? (size_t)mask_ld * (mask_period ? k % mask_period : k) : 0)];
    }
    tile[ty + 8 * i][tx] = v;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t r = r0 + ty + 8 * i, k = k0 + tx;
    if (r < rows && k < K) {
      float h, l;
      split_tf32(tile[tx][ty + 8 * i], h, l);
      uint32_t rd = r;
      if (job.perm_H) { const uint32_t q = r / job.perm_H, u = r % job.perm_H; rd = 128 * (u / 32) + 32 * q + (u % 32); }
      hi[k + (size_t)pitch * rd] = h;
      lo[k + (size_t)pitch * rd] = l;
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encoder(dyb200_ctx* ctx, EncodeTiledFn* fn) {
  if (!ctx->encode_tiled) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    DYB_CUDA(ctx, cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || !p) return dyb200_fail(ctx, DYB200_ECUDA, "cuTensorMapEncodeTiled is not available in this driver");
    ctx->encode_tiled = p;
  }
  *fn = (EncodeTiledFn)ctx->encode_tiled;
  return DYB200_OK;
}

// Plane of `rows` rows and K valid floats per row, row pitch `pitch` floats; box = 32 (k) x 128 (rows).
int make_map(dyb200_ctx* ctx, EncodeTiledFn enc, CUtensorMap* map, float* plane, uint32_t rows, uint32_t K, uint32_t pitch,
             uint32_t box_rows = BM) {
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch * sizeof(float)};
  cuuint32_t box[2] = {BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, plane, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return dyb200_fail(ctx, DYB200_ECUDA, "cuTensorMapEncodeTiled failed with code %d (rows %u, K %u, pitch %u)", (int)r, rows, K, pitch);
  return DYB200_OK;
}

// MN-major plane: element (m, k) at plane[k * pitch + m], `rows` valid m and K valid k, as a 3-D tensor (m within a group
// of 32, k, group): one box = 4 groups x 32 k x 32 m, in the 128-byte swizzle with 32-byte atoms that umma_desc_mn describes.
// The last group may reach past `rows` into the pitch (those rows of the product are never stored).
int make_map_mn(dyb200_ctx* ctx, EncodeTiledFn enc, CUtensorMap* map, float* plane, uint32_t rows, uint32_t K, uint32_t pitch,
                uint32_t box_rows = BM) {
  // (32 m, k, group of 32 m): one box brings box_rows / 32 groups x 32 k rows x 128 bytes, group after group
  cuuint64_t dims[3] = {32, K, (rows + 31) / 32};
  cuuint64_t strides[2] = {(cuuint64_t)pitch * sizeof(float), 128};
  cuuint32_t box[3] = {32, BK, box_rows / 32};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, plane, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return dyb200_fail(ctx, DYB200_ECUDA, "cuTensorMapEncodeTiled failed with code %d (MN-major, rows %u, K %u, pitch %u)", (int)r, rows, K, pitch);
  return DYB200_OK;
}

int pack_flush_impl(dyb200_ctx* ctx, PackJobs* jobs) {
  if (jobs->n == 0) return DYB200_OK;
  const uint32_t total = jobs->start[jobs->n];
  dyb_launch(k_pack_multi, total, 256, 0, ctx, *jobs);
  jobs->n = 0;
  jobs->start[0] = 0;
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

// Queues one operand in `batch` (launching the queue first when it is full); with batch == nullptr it is packed at once.
// layout: 0 = the row index is fast in the source, 1 = the k index is fast, kLayoutGates = row index fast and the
// rows = 4H gate rows are written interleaved (destination row 128 t + 32 q + l <- source row q H + 32 t + l) so that
// every 128-row tile holds the four gates of 32 hidden units.
int pack(dyb200_ctx* ctx, const float* src, uint32_t ld, int layout, uint32_t rows, uint32_t K, const float* mask,
         uint32_t mask_ld, int mask_full, float* hi, float* lo, uint32_t pitch, PackJobs* batch = nullptr,
         uint32_t mask_period = 0) {
  const bool k_is_fast = layout == 1;
  if (rows == 0 || K == 0) return DYB200_OK;
  PackJobs local;
  local.n = 0; local.start[0] = 0;
  PackJobs* q = batch ? batch : &local;
  if (q->n == kMaxPackJobs) { int rc = pack_flush_impl(ctx, q); if (rc) return rc; }
  PackJob& j = q->job[q->n];
  j.src = src; j.mask = mask; j.hi = hi; j.lo = lo;
  j.ld = ld; j.rows = rows; j.K = K; j.mask_ld = mask_ld; j.pitch = pitch;
  j.k_is_fast = k_is_fast ? 1 : 0; j.mask_full = mask_full; j.mask_period = mask_period;
  j.perm_H = layout == kLayoutGates ? rows / 4 : 0;
  uint64_t units;
  if (k_is_fast) {
    j.vec = (K % 4 == 0) && (ld % 4 == 0) && aligned16(src) && (!mask || ((mask_ld % 4 == 0 || !mask_full) && aligned16(mask)));
    j.gx = (K + 1023) / 1024;
    units = (uint64_t)j.gx * rows;
  } else {
    j.vec = 0;
    j.gx = (rows + 31) / 32;
    units = (uint64_t)j.gx * ((K + 31) / 32);
  }
  DYB_CHECK_ARG(ctx, (uint64_t)q->start[q->n] + units < 0x7fffffffull, "pack: operand too large (%u x %u)", rows, K);
  q->start[q->n + 1] = q->start[q->n] + (uint32_t)units;
  q->n++;
  return batch ? DYB200_OK : pack_flush_impl(ctx, q);
}

inline uint32_t round_up(uint32_t x, uint32_t m) { return (x + m - 1) / m * m; }

// Returns the cached packed form of a parameter matrix, packing it first if it is new or stale.
int cached_param_pack(dyb200_ctx* ctx, const float* src, uint32_t ld, int k_is_fast, uint32_t rows, uint32_t K, uint32_t pitch,
                      float** hi, float** lo, const float* src2 = nullptr, uint32_t rows2 = 0) {
  const int cap = (int)(sizeof(ctx->param_pack) / sizeof(ctx->param_pack[0]));
  dyb200_ctx::ParamPack* hit = nullptr;
  dyb200_ctx::ParamPack* victim = &ctx->param_pack[0];
  for (int k = 0; k < cap; ++k) {
    dyb200_ctx::ParamPack* e = &ctx->param_pack[k];
    if (e->hi && e->src == src && e->src2 == src2 && e->rows2 == rows2 && e->ld == ld && e->rows == rows && e->K == K && e->k_is_fast == (int)k_is_fast) { hit = e; break; }
    if (!e->hi) { if (victim->hi) victim = e; }
    else if (victim->hi && e->last_use < victim->last_use) victim = e;
  }
  dyb200_ctx::ParamPack* e = hit ? hit : victim;
  const size_t floats = (size_t)(rows + rows2) * pitch;
  if (!hit) {
    if (e->hi && e->floats < floats) {   // evicted entry is too small: its buffers may still be read by queued kernels
      DYB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      cudaFree(e->hi); cudaFree(e->lo);
      e->hi = e->lo = nullptr;
    }
    if (!e->hi) {
      if (cudaMalloc((void**)&e->hi, floats * sizeof(float)) != cudaSuccess || cudaMalloc((void**)&e->lo, floats * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        if (e->hi) cudaFree(e->hi);
        e->hi = e->lo = nullptr;
        return dyb200_fail(ctx, DYB200_ENOMEM, "parameter cache: cudaMalloc of %zu bytes failed", 2 * floats * sizeof(float));
      }
      e->floats = floats;
    }
    e->src = src; e->src2 = src2; e->rows2 = rows2; e->ld = ld; e->rows = rows; e->K = K; e->pitch = pitch; e->k_is_fast = (int)k_is_fast;
    e->version = ~0ull;
  }
  if (e->version != ctx->param_version) {
    PackJobs batch;
    dyb200_tc_pack_begin(&batch);
    int rc = pack(ctx, src, ld, k_is_fast, rows, K, nullptr, 0, 0, e->hi, e->lo, pitch, &batch);
    if (!rc && rows2) rc = pack(ctx, src2, ld, k_is_fast, rows2, K, nullptr, 0, 0, e->hi + (size_t)rows * pitch, e->lo + (size_t)rows * pitch, pitch, &batch);
    if (!rc) rc = pack_flush_impl(ctx, &batch);
    if (rc) return rc;
    e->version = ctx->param_version;
  }
  e->last_use = ++ctx->param_tick;
  *hi = e->hi; *lo = e->lo;
  return DYB200_OK;
}

}  // namespace

// ---- building blocks shared with the fused LSTM entry points ----------------------------------
int dyb200_tc_pack_flush(dyb200_ctx* ctx, PackJobs* batch) { return pack_flush_impl(ctx, batch); }

int dyb200_tc_pack(dyb200_ctx* ctx, const float* src, uint32_t ld, bool k_is_fast, uint32_t rows, uint32_t K,
                   const float* mask, uint32_t mask_ld, int mask_full, PackedOp* out, PackJobs* batch) {
  const uint32_t pitch = round_up(K, 32);
  void* buf;
  int rc = dyb200_scratch(ctx, (size_t)2 * rows * pitch * sizeof(float) + 256, &buf);
  if (rc) return rc;
  out->hi = (float*)buf;
  out->lo = (float*)(((uintptr_t)(out->hi + (size_t)rows * pitch) + 255) & ~(uintptr_t)255);
  out->rows = rows; out->K = K; out->pitch = pitch;
  return pack(ctx, src, ld, k_is_fast ? 1 : 0, rows, K, mask, mask_ld, mask_full, out->hi, out->lo, pitch, batch);
}

int dyb200_tc_planes(dyb200_ctx* ctx, uint32_t rows, uint32_t K, PackedOp* out) {
  const uint32_t pitch = round_up(K, 32);
  void* buf;
  int rc = dyb200_scratch(ctx, (size_t)2 * rows * pitch * sizeof(float) + 256, &buf);
  if (rc) return rc;
  out->hi = (float*)buf;
  out->lo = (float*)(((uintptr_t)(out->hi + (size_t)rows * pitch) + 255) & ~(uintptr_t)255);
  out->rows = rows; out->K = K; out->pitch = pitch;
  return DYB200_OK;
}

int dyb200_tc_param(dyb200_ctx* ctx, const float* src, uint32_t ld, bool k_is_fast, uint32_t rows, uint32_t K, PackedOp* out) {
  if (!ctx->param_cache_on) return dyb200_tc_pack(ctx, src, ld, k_is_fast, rows, K, nullptr, 0, 0, out, nullptr);
  out->rows = rows; out->K = K; out->pitch = round_up(K, 32);
  return cached_param_pack(ctx, src, ld, k_is_fast ? 1 : 0, rows, K, out->pitch, &out->hi, &out->lo);
}

int dyb200_tc_param_gates(dyb200_ctx* ctx, const float* src, uint32_t ld, uint32_t rows, uint32_t K, PackedOp* out) {
  const uint32_t pitch = round_up(K, 32);
  out->rows = rows; out->K = K; out->pitch = pitch;
  if (ctx->param_cache_on) return cached_param_pack(ctx, src, ld, kLayoutGates, rows, K, pitch, &out->hi, &out->lo);
  void* buf;
  int rc = dyb200_scratch(ctx, (size_t)2 * rows * pitch * sizeof(float) + 256, &buf);
  if (rc) return rc;
  out->hi = (float*)buf;
  out->lo = (float*)(((uintptr_t)(out->hi + (size_t)rows * pitch) + 255) & ~(uintptr_t)255);
  return pack(ctx, src, ld, kLayoutGates, rows, K, nullptr, 0, 0, out->hi, out->lo, pitch, nullptr);
}

inline uint32_t tile_cols(uint32_t N) { return N <= 64 ? 64 : BN; }

// Cost model of one launch (us): waves x (k-blocks per CTA x t_kb + 9 us of pipeline fill and epilogue), waves =
// ceil(tiles x S / SMs); S > 1 adds the second kernel that sums the S partial products into C ((S + 2) M N floats through
// HBM + a launch).  Measured on B200: within 2 us of the per-step LSTM products (dx / dh: 64 or 48 tiles, K = 4096 ->
// S = 2 and 3).
static double split_cost(double sms, uint32_t tiles, uint32_t kb_total, uint32_t S, double t_kb, double mn_bytes) {
  const uint32_t kb_split = (kb_total + S - 1) / S;
  double t = ceil((double)tiles * S / sms) * (kb_split * t_kb + 9.0);
  if (S > 1) t += (S + 2) * mn_bytes / 5.0e6 + 5.0;   // bytes / (5 TB/s) in us
  return t;
}
static uint32_t best_split(double sms, uint32_t tiles, uint32_t kb_total, double t_kb, double mn_bytes, double* cost) {
  uint32_t best = 1;
  double best_t = split_cost(sms, tiles, kb_total, 1, t_kb, mn_bytes);
  for (uint32_t S = 2; S <= 8; ++S) {
    if (kb_total / S < 8) break;   // at least 8 k-blocks per split
    const uint32_t kb_split = (kb_total + S - 1) / S;
    if ((kb_total + kb_split - 1) / kb_split != S) continue;
    const double t = split_cost(sms, tiles, kb_total, S, t_kb, mn_bytes);
    if (t < best_t * 0.97) { best = S; best_t = t; }   // a split must win by 3 %
  }
  if (cost) *cost = best_t;
  return best;
}
// The partly filled last round of a many-tile product can run as a product of its own (see dyb200_tc_gemm_packed) when K is
// long and its tiles form a rectangle: 2 = the last tail / tiles_n row blocks of every column of tiles (the persistent kernel
// keeps its grouped tile order on the row blocks before them), 1 = the last `tail` row blocks of the last column of tiles
// (row-block-fastest order), 0 = neither.
static int tail_can_run_apart(const dyb200_ctx* ctx, uint32_t tiles_m, uint32_t tiles, uint32_t kb_total, uint32_t bn) {
  const uint32_t tail = tiles % (uint32_t)ctx->sm_count, tiles_n = tiles / tiles_m;
  if (!(tiles > (uint32_t)ctx->sm_count && tail > 0 && 2 * tail <= (uint32_t)ctx->sm_count && kb_total >= 64 && bn == BN)) return 0;
  if (tail % tiles_n == 0 && tail / tiles_n < tiles_m) return 2;
  return tail <= tiles_m ? 1 : 0;
}

// Number of K splits of a product: the one the cost model says is fastest.  For a product with more tiles than SMs the
// unsplit form is the persistent kernel (epilogues overlapped, ~3 us left per tile) with its last round split apart.
uint32_t dyb200_tc_splits(const dyb200_ctx* ctx, uint32_t M, uint32_t N, uint32_t kb_total) {
  const uint32_t bn = tile_cols(N);
  const uint32_t tiles_m = (M + BM - 1) / BM, tiles = tiles_m * ((N + bn - 1) / bn);
  const double sms = (double)ctx->sm_count, t_kb = bn == 64 ? 0.40 : 0.66;
  const double mn_bytes = 4.0 * (double)M * (double)N;
  double cost;
  const uint32_t S = best_split(sms, tiles, kb_total, t_kb, mn_bytes, &cost);
  if (S > 1 && tail_can_run_apart(ctx, tiles_m, tiles, kb_total, bn)) {
    const uint32_t tail = tiles % (uint32_t)ctx->sm_count;
    double tail_cost;
    best_split(sms, tail, kb_total, t_kb, mn_bytes * tail / tiles, &tail_cost);
    const double persistent = (tiles / (uint32_t)ctx->sm_count) * (kb_total * t_kb + 3.0) + tail_cost;
    if (persistent < cost) return 1;
  }
  return S;
}

bool dyb200_lstm_bwd_tiling(const dyb200_ctx* ctx, uint32_t I, uint32_t H, uint32_t B, LstmBwdTiling* out) {
  // 128-column tiles from 256 columns up; two column blocks per CTA whenever the batch has an even number of them (128
  // columns: two blocks of 64), so that each CTA of the sequence kernel alternates between two independent chains
  const uint32_t bn = (B >= 256 && B % 128 == 0) ? 128u : 64u;
  if (B == 0 || B % bn != 0 || B / bn > 32 || H % 64 != 0 || I % 4 != 0) return false;
  const uint32_t tiles_m = (I + H + BM - 1) / BM, tiles_n = B / bn, kb = 4 * H / 32;
  const uint32_t ncb = tiles_n % 2 == 0 ? 2u : 1u;
  // as many K splits as keep every CTA of the sequence kernel resident (one per SM), at least 8 k-blocks each
  const uint32_t groups = tiles_m * (tiles_n / ncb);
  uint32_t S = (uint32_t)ctx->sm_count / groups;
  if (S == 0 || tiles_m * tiles_n > 160) return false;
  if (S > 8) S = 8;
  while (S > 1 && kb / S < 8) --S;
  const uint32_t per = (kb + S - 1) / S;
  S = (kb + per - 1) / per;
  out->bn = bn; out->ncb = ncb; out->S = S;
  return true;
}

int dyb200_tc_param2(dyb200_ctx* ctx, const float* src, uint32_t rows, const float* src2, uint32_t rows2, uint32_t ld,
                     bool k_is_fast, uint32_t K, PackedOp* out) {
  const uint32_t pitch = round_up(K, 32);
  out->rows = rows + rows2; out->K = K; out->pitch = pitch;
  if (ctx->param_cache_on) return cached_param_pack(ctx, src, ld, k_is_fast, rows, K, pitch, &out->hi, &out->lo, src2, rows2);
  void* buf;
  int rc = dyb200_scratch(ctx, (size_t)2 * out->rows * pitch * sizeof(float) + 256, &buf);
  if (rc) return rc;
  out->hi = (float*)buf;
  out->lo = (float*)(((uintptr_t)(out->hi + (size_t)out->rows * pitch) + 255) & ~(uintptr_t)255);
  PackJobs batch;
  dyb200_tc_pack_begin(&batch);
  rc = pack(ctx, src, ld, k_is_fast, rows, K, nullptr, 0, 0, out->hi, out->lo, pitch, &batch);
  if (!rc) rc = pack(ctx, src2, ld, k_is_fast, rows2, K, nullptr, 0, 0, out->hi + (size_t)rows * pitch, out->lo + (size_t)rows * pitch, pitch, &batch);
  if (!rc) rc = pack_flush_impl(ctx, &batch);
  return rc;
}

int dyb200_tc_gemm_packed(dyb200_ctx* ctx, uint32_t M, uint32_t N, int npairs, const PackedOp* A, const PackedOp* B,
                          const GemmEpilogue& epi, uint32_t force_splits) {
  EncodeTiledFn enc;
  int rc = get_encoder(ctx, &enc);
  if (rc) return rc;
  // (function attributes are per device: the context remembers what it has set on its own device)
  if (!(ctx->func_attr_done & 1u)) {
    DYB_CUDA(ctx, cudaFuncSetAttribute(k_gemm_tc<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    DYB_CUDA(ctx, cudaFuncSetAttribute(k_gemm_tc<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    ctx->func_attr_done |= 1u;
  }
  const uint32_t bn = tile_cols(N);
  TmapPack tm;
  memset(&tm, 0, sizeof(tm));
  double flops = 0;
  const bool a_mn = A[0].mn_major != 0, b_mn = B[0].mn_major != 0;
  // (an MN-major plane is read in groups of 32 rows: its pitch covers the rows rounded up to 32)
  DYB_CHECK_ARG(ctx, !a_mn || (npairs == 1 && A[0].pitch % 32 == 0 && A[0].pitch >= M && aligned16(A[0].hi) && aligned16(A[0].lo)),
                "tensor GEMM: an MN-major left operand needs a single pair, a pitch that is a multiple of 32 and covers the rows, and 16-byte aligned planes");
  DYB_CHECK_ARG(ctx, !b_mn || (npairs == 1 && B[0].pitch % 32 == 0 && B[0].pitch >= N && aligned16(B[0].hi) && aligned16(B[0].lo)),
                "tensor GEMM: an MN-major right operand needs a single pair, a pitch that is a multiple of 32 and covers the rows, and 16-byte aligned planes");
  tm.a_mn = a_mn ? 1u : 0u;
  tm.b_mn = b_mn ? 1u : 0u;
  for (int p = 0; p < npairs; ++p) {
    DYB_CHECK_ARG(ctx, A[p].rows == M && B[p].rows == N && A[p].K == B[p].K && A[p].pitch % 32 == 0 && B[p].pitch % 32 == 0,
                  "tensor GEMM: packed operand shapes do not match (M %u, N %u)", M, N);
    flops += 2.0 * M * N * A[p].K;
    if (a_mn) {
      if ((rc = make_map_mn(ctx, enc, &tm.t[0], A[0].hi, M, A[0].K, A[0].pitch))) return rc;
      if ((rc = make_map_mn(ctx, enc, &tm.t[1], A[0].lo, M, A[0].K, A[0].pitch))) return rc;
    } else {
      if ((rc = make_map(ctx, enc, &tm.t[4 * p + 0], A[p].hi, M, A[p].K, A[p].pitch))) return rc;
      if ((rc = make_map(ctx, enc, &tm.t[4 * p + 1], A[p].lo, M, A[p].K, A[p].pitch))) return rc;
    }
    if (b_mn) {
      if ((rc = make_map_mn(ctx, enc, &tm.t[2], B[0].hi, N, B[0].K, B[0].pitch, bn))) return rc;
      if ((rc = make_map_mn(ctx, enc, &tm.t[3], B[0].lo, N, B[0].K, B[0].pitch, bn))) return rc;
    } else {
      if ((rc = make_map(ctx, enc, &tm.t[4 * p + 2], B[p].hi, N, B[p].K, B[p].pitch, bn))) return rc;
      if ((rc = make_map(ctx, enc, &tm.t[4 * p + 3], B[p].lo, N, B[p].K, B[p].pitch, bn))) return rc;
    }
  }
  if (npairs == 1) for (int k = 0; k < 4; ++k) tm.t[4 + k] = tm.t[k];
  uint32_t kb0 = round_up(A[0].K, 32) / BK, kb1 = npairs > 1 ? round_up(A[1].K, 32) / BK : 0;
  const uint32_t kb_total = kb0 + kb1;
  dim3 grid((M + BM - 1) / BM, (N + bn - 1) / bn, 1);
  DYB_CHECK_ARG(ctx, epi.mode != EPI_LSTM_CELL || (M % BM == 0 && epi.H * 4 == M && epi.ldc % 4 == 0 && aligned16(epi.C) &&
                                                      aligned16(epi.bias) && aligned16(epi.c_prev) && aligned16(epi.c_out) && aligned16(epi.h_out)),
                "tensor GEMM: the LSTM-cell epilogue needs whole tiles of interleaved gate rows and 16-byte aligned tensors");
  // Split K when the output has too few tiles to occupy the SMs (e.g. dx = W^T dgate: 16-32 tiles, K = 4096).
  uint32_t S = force_splits ? (force_splits < kb_total ? force_splits : kb_total) : dyb200_tc_splits(ctx, M, N, kb_total);
  uint32_t kb_per_split = (kb_total + S - 1) / S;
  S = (kb_total + kb_per_split - 1) / kb_per_split;
  GemmEpilogue kepi = epi;
  float* part = nullptr;
  // K splits as one thread-block cluster per tile (partial tiles meet in distributed shared memory) when every cluster
  // of the launch can be resident at once; dyb200_ctx_cluster_splitk(ctx, 0) keeps the workspace + second-kernel form.
  if (S > 1 && ctx->cluster_splitk) {
    if (!(ctx->func_attr_done & 2u)) {
      DYB_CUDA(ctx, cudaFuncSetAttribute(k_gemm_tc<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
      DYB_CUDA(ctx, cudaFuncSetAttribute(k_gemm_tc<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
      ctx->func_attr_done |= 2u;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.blockDim = dim3(kThreads, 1, 1); cfg.dynamicSmemBytes = SMEM_BYTES; cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    auto fits = [&](uint32_t Sc) -> bool {
      int& mc = ctx->max_clusters[bn == 64 ? 0 : 1][Sc];   // [tile width][cluster size], 0 = not asked yet on this device
      if (mc == 0) {
        cfg.gridDim = dim3(grid.x, grid.y, Sc);
        attr[0].val.clusterDim.z = Sc;
        int n = 0;
        cudaError_t e = bn == 64 ? cudaOccupancyMaxActiveClusters(&n, k_gemm_tc<64, true>, &cfg)
                                 : cudaOccupancyMaxActiveClusters(&n, k_gemm_tc<128, true>, &cfg);
        if (e != cudaSuccess) { (void)cudaGetLastError(); n = -1; }
        mc = n > 0 ? n : -1;
      }
      return mc > 0 && grid.x * grid.y <= (uint32_t)mc;
    };
    // (a smaller cluster size that fits was tried when the model's count does not - batch 64, 16 tiles: 7 instead of 8 -
    // and measured slower than the workspace form of the model's count: 4.73 vs 4.60 ms per step)
    const uint32_t Sc = (S <= 8 && fits(S)) ? S : 0;
    if (Sc) {
      kb_per_split = (kb_total + Sc - 1) / Sc;
      cfg.gridDim = dim3(grid.x, grid.y, Sc);
      attr[0].val.clusterDim.z = Sc;
      GemmProfScope scope(ctx, flops, 1, M, N, kb_total * BK, (uint32_t)epi.mode);
      if (bn == 64) cudaLaunchKernelEx(&cfg, k_gemm_tc<64, true>, tm, M, N, kb0, kb1, kb_per_split, epi, ctx->dev_flags);
      else cudaLaunchKernelEx(&cfg, k_gemm_tc<128, true>, tm, M, N, kb0, kb1, kb_per_split, epi, ctx->dev_flags);
      DYB_LAUNCHED(ctx);
      return DYB200_OK;
    }
  }
  if (S > 1) {
    void* pw;
    rc = dyb200_scratch(ctx, (size_t)S * M * N * sizeof(float), &pw);
    if (rc) return rc;
    part = (float*)pw;
    kepi = GemmEpilogue{EPI_STORE, part, M, nullptr, 0, 0.f, nullptr, 0, 0};   // (no second destination)
    grid.z = S;
  }
  if (S == 1 && grid.x * grid.y > (uint32_t)ctx->sm_count) {
    // A partly filled last round (dR: 632 tiles = 4 rounds of 148 + 40) would keep 108 SMs idle for a whole tile time.
    // When those last tiles form a rectangle (dR: the last 5 row blocks of all 8 columns of tiles) and K is long, the
    // persistent kernel stops before them and they run as a product of their own (the sub-matrices of the same operands),
    // which the cost model splits along K.
    uint32_t tiles_run = grid.x * grid.y;
    const uint32_t tail = tiles_run % (uint32_t)ctx->sm_count;
    const bool plain_epi = (epi.mode == EPI_STORE || epi.mode == EPI_ACCUM || epi.mode == EPI_BIAS) && epi.split_m == 0;
    const int tail_form = plain_epi ? tail_can_run_apart(ctx, grid.x, tiles_run, kb_total, bn) : 0;
    const bool tail_apart = tail_form != 0;
    if (tail_apart) tiles_run -= tail;
    // row blocks the persistent launch covers (all of them, unless the last ones run apart in every column of tiles)
    const uint32_t rows_run = tail_form == 2 ? grid.x - tail / grid.y : grid.x;
    if (!(ctx->func_attr_done & 4u)) {
      DYB_CUDA(ctx, cudaFuncSetAttribute(k_gemm_persist<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_PERSIST_BYTES));
      DYB_CUDA(ctx, cudaFuncSetAttribute(k_gemm_persist<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_PERSIST_BYTES));
      ctx->func_attr_done |= 4u;
    }
    // A long reduction whose tiles fill the last round badly (the deferred weight gradients: 256 tiles of 560 k-blocks on
    // 148 SMs = two rounds, the second 73 % full) is cut into Sp K splits as further work items of the same persistent
    // launch: 1024 items of 140 k-blocks make seven nearly full rounds.  The partial products go to a workspace and
    // k_splitk_reduce adds them in split order and applies the epilogue.  Same cost form as dyb200_tc_splits, with the 3 us
    // that a persistent CTA spends between items.
    uint32_t Sp = 1;
    if (!tail_apart && epi.mode != EPI_LSTM_CELL && epi.mode != EPI_GATES) {
      const double sms = (double)ctx->sm_count, t_kb = bn == 64 ? 0.40 : 0.66, mn_bytes = 4.0 * (double)M * (double)N;
      auto est = [&](uint32_t q) {
        const double rounds = ceil((double)tiles_run * q / sms);
        return rounds * ((double)((kb_total + q - 1) / q) * t_kb + 3.0) + (q > 1 ? (q + 2) * mn_bytes / 5.0e6 + 8.0 : 0.0);
      };
      double best = est(1);
      for (uint32_t q = 2; q <= 4; ++q)
        if (kb_total / q >= 64 && est(q) < 0.95 * best && est(q) < 0.95 * est(1)) { best = est(q); Sp = q; }
    }
    GemmEpilogue pepi = epi;
    float* ppart = nullptr;
    if (Sp > 1) {
      void* pw;
      if ((rc = dyb200_scratch(ctx, (size_t)Sp * M * N * sizeof(float), &pw))) return rc;
      ppart = (float*)pw;
      pepi = GemmEpilogue{EPI_STORE, ppart, M, nullptr, 0, 0.f, nullptr, 0, 0};
    }
    {
      GemmProfScope scope(ctx, flops * ((double)tiles_run / (grid.x * grid.y)), 1, M, N, kb_total * BK, (uint32_t)epi.mode);
      // grouped tile order when the A operand has many row blocks (unless the last round runs apart as part of the last
      // column of tiles, which relies on the row-block-fastest order)
      const uint32_t gm = (tail_form != 1 && rows_run > 16) ? 16u : 0u;
      if (bn == 64) dyb_launch(k_gemm_persist<64>, dim3(ctx->sm_count), kThreads, SMEM_PERSIST_BYTES, ctx, tm, M, N, kb0, kb1, rows_run, tiles_run, gm, Sp, pepi, ctx->dev_flags);
      else dyb_launch(k_gemm_persist<128>, dim3(ctx->sm_count), kThreads, SMEM_PERSIST_BYTES, ctx, tm, M, N, kb0, kb1, rows_run, tiles_run, gm, Sp, pepi, ctx->dev_flags);
      DYB_LAUNCHED(ctx);
      if (Sp > 1 && (rc = dyb200_splitk_reduce(ctx, ppart, Sp, M, N, epi))) return rc;
    }
    if (!tail_apart) return DYB200_OK;
    // the last `tail` row blocks of the last column of tiles, or the last tail / tiles_n row blocks of every column
    const uint32_t m_off = (tail_form == 2 ? rows_run : grid.x - tail) * BM, n_off = tail_form == 2 ? 0u : (grid.y - 1) * bn;
    PackedOp A2[2], B2[2];
    for (int p = 0; p < npairs; ++p) {
      A2[p] = A[p]; A2[p].rows = M - m_off;   // (MN-major planes: the rows are the fast index)
      A2[p].hi += a_mn ? (size_t)m_off : (size_t)m_off * A[p].pitch; A2[p].lo += a_mn ? (size_t)m_off : (size_t)m_off * A[p].pitch;
      B2[p] = B[p]; B2[p].rows = N - n_off;
      B2[p].hi += b_mn ? (size_t)n_off : (size_t)n_off * B[p].pitch; B2[p].lo += b_mn ? (size_t)n_off : (size_t)n_off * B[p].pitch;
    }
    GemmEpilogue e2 = epi;
    e2.C += m_off + (size_t)epi.ldc * n_off;
    if (epi.mode == EPI_BIAS) e2.bias += m_off;
    return dyb200_tc_gemm_packed(ctx, M - m_off, N - n_off, npairs, A2, B2, e2);
  }
  {
    // times the MMA kernel (and the split-K reduction); the packing launches show up in the step time
    GemmProfScope scope(ctx, flops, 1, M, N, kb_total * BK, (uint32_t)epi.mode);
    if (bn == 64) dyb_launch(k_gemm_tc<64, false>, grid, kThreads, SMEM_BYTES, ctx, tm, M, N, kb0, kb1, kb_per_split, kepi, ctx->dev_flags);
    else dyb_launch(k_gemm_tc<128, false>, grid, kThreads, SMEM_BYTES, ctx, tm, M, N, kb0, kb1, kb_per_split, kepi, ctx->dev_flags);
    DYB_LAUNCHED(ctx);
    if (S > 1 && epi.mode == EPI_LSTM_CELL) {
      dyb_launch(k_splitk_reduce_cell, stream_grid(ctx, (size_t)M / 16 * N + 1, 256), 256, 0, ctx, part, S, M, N, epi);
      DYB_LAUNCHED(ctx);
    } else if (S > 1) {
      int vec = M % 4 == 0 && epi.ldc % 4 == 0 && aligned16(epi.C) && epi.mode != EPI_GATES &&
                (epi.mode != EPI_BIAS || aligned16(epi.bias)) &&
                (epi.mode != EPI_ACCUM_MASK || (aligned16(epi.maskC) && (!epi.maskc_full || epi.maskc_ld % 4 == 0)));
      if (epi.split_m)
        vec = vec && epi.split_m % 4 == 0 && epi.ldc2 % 4 == 0 && aligned16(epi.C2) &&
              (epi.mode != EPI_ACCUM_MASK || (aligned16(epi.maskC2) && (!epi.maskc2_full || epi.maskc2_ld % 4 == 0)));
      dyb_launch(k_splitk_reduce, stream_grid(ctx, (size_t)M * N / 4 + 1, 256), 256, 0, ctx, part, S, M, N, epi, vec);
      DYB_LAUNCHED(ctx);
    }
  }
  return DYB200_OK;
}

// Second stage of a K split for callers outside this file: C = epilogue(sum over s of part[s]), the S partial products
// (M x N each, leading dimension M) added in ascending order.
int dyb200_splitk_reduce(dyb200_ctx* ctx, const float* part, uint32_t S, uint32_t M, uint32_t N, const GemmEpilogue& epi) {
  int vec = M % 4 == 0 && epi.ldc % 4 == 0 && aligned16(epi.C) && epi.mode != EPI_GATES && (epi.mode != EPI_BIAS || aligned16(epi.bias)) &&
            (epi.mode != EPI_ACCUM_MASK || (aligned16(epi.maskC) && (!epi.maskc_full || epi.maskc_ld % 4 == 0)));
  if (epi.split_m)
    vec = vec && epi.split_m % 4 == 0 && epi.ldc2 % 4 == 0 && aligned16(epi.C2) &&
          (epi.mode != EPI_ACCUM_MASK || (aligned16(epi.maskC2) && (!epi.maskc2_full || epi.maskc2_ld % 4 == 0)));
  dyb_launch(k_splitk_reduce, stream_grid(ctx, (size_t)M * N / 4 + 1, 256), 256, 0, ctx, part, S, M, N, epi, vec);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

bool dyb200_tc_eligible(uint32_t M, uint32_t N, double flops) {
  // Small products stay on the CUDA-core kernel: packing + a 128x128 tile would mostly move padding.  A product with few
  // rows but many columns or a long reduction (the tag layer of a tagger: 32 or 45 rows times 100 000 tokens) is still far
  // better off here - most of a tile's rows are padding, but the work is bound by reading the long operand once.
  // (Between 2 and 8 MFLOP the CUDA-core kernel is slow when its grid is one or two CTAs - 190 us for the 128 x 21 x 1024
  // products of a tagger batch's last time steps - but it is plain fp32: a lower limit here was measured to cost accuracy
  // margin in small-batch recurrences (1.5e-4 of a row's scale after 100 steps of 3xTF32 products), so the limit stays.)
  return !(flops < 8.0e6 || M < 16 || (M + BM - 1) / BM > 65535u || (N + BN - 1) / BN > 65535u);
}

int dyb200_gemm_tc(dyb200_ctx* ctx, uint32_t M, uint32_t N, int npairs, const GemmPair* pairs, const GemmEpilogue& epi,
                   int* handled) {
  *handled = 0;
  if (M == 0 || N == 0 || npairs < 1 || npairs > 2) return DYB200_OK;
  double flops = 0;
  for (int p = 0; p < npairs; ++p) flops += 2.0 * M * N * pairs[p].K;
  if (!dyb200_tc_eligible(M, N, flops)) return DYB200_OK;
  for (int p = 0; p < npairs; ++p) if (pairs[p].K == 0) return DYB200_OK;
  *handled = 1;
  PackedOp A[2], B[2];
  PackJobs batch;   // all operands that need packing go out in one launch
  dyb200_tc_pack_begin(&batch);
  for (int p = 0; p < npairs; ++p) {
    const GemmPair& g = pairs[p];
    // A: rows = m. op(A)(m,k) = transA ? A[k + lda*m] : A[m + lda*k]  -> k is fast iff transA.  An operand whose rows are
    // the fast index is split as it lies (K rows of M values) and read MN-major (single products only): no transposing
    // pass, and a parameter then has ONE set of planes for this product and for the one that uses it transposed.
    const bool a_mn = npairs == 1 && g.transA == 0, b_mn = npairs == 1 && g.transB != 0;
    int rc;
    if (a_mn) {
      rc = g.a_is_param ? dyb200_tc_param(ctx, g.A, g.lda, true, g.K, M, &A[p])
                        : dyb200_tc_pack(ctx, g.A, g.lda, true, g.K, M, nullptr, 0, 0, &A[p], &batch);
      A[p].rows = M; A[p].K = g.K; A[p].mn_major = 1;
    } else {
      rc = g.a_is_param ? dyb200_tc_param(ctx, g.A, g.lda, g.transA != 0, M, g.K, &A[p])
                        : dyb200_tc_pack(ctx, g.A, g.lda, g.transA != 0, M, g.K, nullptr, 0, 0, &A[p], &batch);
    }
    if (rc) return rc;
    // B: rows = n. op(B)(k,n) = transB ? B[n + ldb*k] : B[k + ldb*n]  -> k is fast iff !transB
    if (b_mn) {
      rc = dyb200_tc_pack(ctx, g.B, g.ldb, true, g.K, N, g.maskB, g.mask_ld, g.mask_full, &B[p], &batch);
      B[p].rows = N; B[p].K = g.K; B[p].mn_major = 1;
    } else {
      rc = dyb200_tc_pack(ctx, g.B, g.ldb, g.transB == 0, N, g.K, g.maskB, g.mask_ld, g.mask_full, &B[p], &batch);
    }
    if (rc) return rc;
  }
  int rcf = dyb200_tc_pack_flush(ctx, &batch);
  if (rcf) return rcf;
  return dyb200_tc_gemm_packed(ctx, M, N, npairs, A, B, epi);
}

// ---- deferred parameter-gradient products ---------------------------------------------------------
// dW = sum_t A_t * B_t^T (A_t: M x k_t, B_t: N x k_t, both column-major) arises once per time step for
// a parameter shared by all steps (dWx, dWh of an LSTM layer, dR of the output projection).  Instead of
// T small products with K = batch, the packed K-major planes of every step are appended along K and ONE
// product with K = sum k_t runs at the end: the tensor pipe sees a long reduction and C is read and
// written once.  One A operand can serve two B operands (dWx and dWh share the gate gradient).
// All planes are MN-major for that product: one row per COLUMN of the accumulator - Mp = M rounded up to 32 floats in A,
// Np[j] in B[j] - element (m, col) at plane[col * Mp + m].  For an LSTM layer these are the layouts the recurrence reads
// K-major: A = the gate-gradient planes, right operand of dx / dh = [Wx; Wh]^T dgates in the backward pass; B[0] = x .*
// mask_x and B[1] = h_tm1 .* mask_h, right operands of the gate product in the forward pass.  So every set of planes is
// written once, by whoever produces the values (a packing launch, the LSTM epilogue, the cell pass), serves both products,
// and no transposed copy exists.
struct dyb200_wgrad {
  uint32_t M, Mp, N[2], Np[2], Kcap;
  uint32_t k;    // columns of A filled so far (the product at flush time runs over [0, k))
  uint32_t kb;   // columns of the B operands filled so far
  PackedOp A, B[2];
  // Pre-split sequence inputs (dyb200_wgrad_pack_inputs): x_cols = columns of B[0] that hold a whole sequence's x .* mask_x
  // (0: none); rows [c, c + batch) of B[1] are the h input of the step that starts at column c, written by the LSTM
  // epilogue of the step before; h_col = the column whose B[1] rows the last forward call wrote; step = columns per step
  // of that sequence (0: varying).
  uint32_t x_cols, h_col, step;
};
// natural pack of the k columns [col, col + k) of operand j (b is N[j] x k column-major; the mask is indexed like b)
static int pack_b_rows(dyb200_ctx* ctx, dyb200_wgrad* w, int j, uint32_t col, uint32_t k, const float* b, uint32_t ldb, const float* mask,
                       int mask_full, PackJobs* batch) {
  return pack(ctx, b, ldb, 1, k, w->N[j], mask, ldb, mask_full, w->B[j].hi + (size_t)col * w->Np[j], w->B[j].lo + (size_t)col * w->Np[j],
              w->Np[j], batch);
}

// Same as dyb200_wgrad_push, but the packing work is queued in `batch` (the caller launches it).
int dyb200_wgrad_push_batched(dyb200_wgrad* w, uint32_t k, const float* a, uint32_t lda, const float* b0, uint32_t ldb0,
                              const float* mask0, int mask0_full, const float* b1, uint32_t ldb1, const float* mask1,
                              int mask1_full, dyb200_ctx* ctx, PackJobs* batch) {
  DYB_CHECK_ARG(ctx, w && a && b0 && (w->N[1] == 0 || b1), "wgrad_push: null argument");
  DYB_CHECK_ARG(ctx, w->k + k <= w->Kcap, "wgrad_push: %u + %u columns exceed the capacity %u", w->k, k, w->Kcap);
  if (k == 0) return DYB200_OK;
  // (a is M x k column-major: the k rows of the MN-major planes, each M contiguous values)
  int rc = pack(ctx, a, lda, true, k, w->M, nullptr, 0, 0, w->A.hi + (size_t)w->k * w->Mp, w->A.lo + (size_t)w->k * w->Mp, w->Mp, batch);
  if (rc) return rc;
  rc = pack_b_rows(ctx, w, 0, w->k, k, b0, ldb0, mask0, mask0_full, batch);
  if (rc) return rc;
  if (w->N[1]) {
    rc = pack_b_rows(ctx, w, 1, w->k, k, b1, ldb1, mask1, mask1_full, batch);
    if (rc) return rc;
  }
  w->k += k;
  w->kb = w->k;
  return DYB200_OK;
}

// For a producer that writes the A planes of the next k columns itself: where they go (k rows of `pitch` floats: row =
// column of the accumulator, M values each), and the B operands queued as in dyb200_wgrad_push_batched.  The accumulator
// advances by k.
int dyb200_wgrad_reserve(dyb200_wgrad* w, uint32_t k, float** a_hi, float** a_lo, uint32_t* pitch, const float* b0, uint32_t ldb0,
                         const float* mask0, int mask0_full, const float* b1, uint32_t ldb1, const float* mask1, int mask1_full,
                         dyb200_ctx* ctx, PackJobs* batch) {
  DYB_CHECK_ARG(ctx, w && b0 && (w->N[1] == 0 || b1), "wgrad_reserve: null argument");
  DYB_CHECK_ARG(ctx, w->k + k <= w->Kcap, "wgrad_reserve: %u + %u columns exceed the capacity %u", w->k, k, w->Kcap);
  *a_hi = w->A.hi + (size_t)w->k * w->Mp; *a_lo = w->A.lo + (size_t)w->k * w->Mp; *pitch = w->Mp;
  int rc = pack_b_rows(ctx, w, 0, w->k, k, b0, ldb0, mask0, mask0_full, batch);
  if (rc) return rc;
  if (w->N[1]) {
    rc = pack_b_rows(ctx, w, 1, w->k, k, b1, ldb1, mask1, mask1_full, batch);
    if (rc) return rc;
  }
  w->k += k;
  w->kb = w->k;
  return DYB200_OK;
}
// Explicit column positions, for callers that fill the B operands (the layer inputs) during the forward pass and the A
// operand (the gate gradient) during the backward pass: step t of a sequence uses columns [t * k, (t + 1) * k) both times.
int dyb200_wgrad_push_b_at(dyb200_wgrad* w, uint32_t col, uint32_t k, const float* b0, uint32_t ldb0, const float* mask0, int mask0_full,
                           const float* b1, uint32_t ldb1, const float* mask1, int mask1_full, dyb200_ctx* ctx, PackJobs* batch) {
  // (b0 == nullptr: the first operand's columns are already in place, see dyb200_wgrad_pack_inputs)
  DYB_CHECK_ARG(ctx, w && (w->N[1] == 0 || b1), "wgrad_push_b_at: null argument");
  DYB_CHECK_ARG(ctx, (uint64_t)col + k <= w->Kcap, "wgrad_push_b_at: columns [%u, %u) exceed the capacity %u", col, col + k, w->Kcap);
  int rc = b0 ? pack_b_rows(ctx, w, 0, col, k, b0, ldb0, mask0, mask0_full, batch) : DYB200_OK;
  if (rc) return rc;
  if (w->N[1]) {
    rc = pack_b_rows(ctx, w, 1, col, k, b1, ldb1, mask1, mask1_full, batch);
    if (rc) return rc;
  }
  if (col + k > w->kb) w->kb = col + k;
  return DYB200_OK;
}
int dyb200_wgrad_reserve_a_at(dyb200_wgrad* w, uint32_t col, uint32_t k, float** a_hi, float** a_lo, uint32_t* pitch, dyb200_ctx* ctx) {
  DYB_CHECK_ARG(ctx, w && (uint64_t)col + k <= w->Kcap, "wgrad_reserve_a_at: columns [%u, %u) exceed the capacity", col, col + k);
  *a_hi = w->A.hi + (size_t)col * w->Mp; *a_lo = w->A.lo + (size_t)col * w->Mp; *pitch = w->Mp;
  if (col + k > w->k) w->k = col + k;
  return DYB200_OK;
}
int dyb200_wgrad_pack_a_at(dyb200_wgrad* w, uint32_t col, uint32_t k, const float* a, uint32_t lda, dyb200_ctx* ctx, PackJobs* batch) {
  DYB_CHECK_ARG(ctx, w && a && (uint64_t)col + k <= w->Kcap, "wgrad_pack_a_at: columns [%u, %u) exceed the capacity", col, col + k);
  int rc = pack(ctx, a, lda, 1, k, w->M, nullptr, 0, 0, w->A.hi + (size_t)col * w->Mp, w->A.lo + (size_t)col * w->Mp, w->Mp, batch);
  if (rc) return rc;
  if (col + k > w->k) w->k = col + k;
  return DYB200_OK;
}
bool dyb200_wgrad_x_planes(const dyb200_wgrad* w, uint32_t col, uint32_t k, PackedOp* out) {
  if (!w || (w->step && k != w->step) || (uint64_t)col + k > w->x_cols) return false;
  *out = w->B[0];
  out->rows = k; out->K = w->N[0]; out->mn_major = 0;
  out->hi += (size_t)col * w->Np[0]; out->lo += (size_t)col * w->Np[0];
  return true;
}
bool dyb200_wgrad_h_planes(const dyb200_wgrad* w, uint32_t col, uint32_t k, PackedOp* out) {
  if (!w || w->N[1] == 0 || (w->step && k != w->step) || w->h_col != col || (uint64_t)col + k > w->x_cols) return false;
  *out = w->B[1];
  out->rows = k; out->K = w->N[1]; out->mn_major = 0;
  out->hi += (size_t)col * w->Np[1]; out->lo += (size_t)col * w->Np[1];
  return true;
}
bool dyb200_wgrad_next_h(dyb200_wgrad* w, uint32_t col, uint32_t k, GemmEpilogue* epi) {
  // (all k columns of h_t are written at the next step's position; with steps of varying width the next step may use fewer)
  if (!w || w->N[1] == 0 || w->x_cols == 0 || (w->step && k != w->step) || (uint64_t)col + 2 * (uint64_t)k > w->x_cols) return false;
  const uint32_t next = col + k;
  epi->hn_hi = w->B[1].hi + (size_t)next * w->Np[1]; epi->hn_lo = w->B[1].lo + (size_t)next * w->Np[1]; epi->hn_pitch = w->Np[1];
  w->h_col = next;
  if (next + k > w->kb) w->kb = next + k;
  return true;
}
// ---- sequence kernels (lstm_seq.cu): the operand planes the accumulator holds for a whole sequence ----
bool dyb200_wgrad_seq_planes(const dyb200_wgrad* w, uint32_t steps, uint32_t step, SeqPlanes* out) {
  if (!w || w->N[1] == 0 || w->x_cols == 0 || w->step != step || w->x_cols != (uint64_t)steps * step) return false;
  out->X = w->B[0]; out->X.rows = w->x_cols; out->X.K = w->N[0]; out->X.mn_major = 0;
  out->Hs = w->B[1]; out->Hs.rows = w->x_cols; out->Hs.K = w->N[1]; out->Hs.mn_major = 0;
  return true;
}
// h of the first step (h0 .* mask_h): operand planes of columns [0, step).  The same values
// dyb200_vanilla_lstm_fwd_fused_at splits at deferred_col = 0.
int dyb200_wgrad_seq_h0(dyb200_wgrad* w, const float* h0, const float* mh, int mh_full, dyb200_ctx* ctx, PackJobs* batch) {
  return pack_b_rows(ctx, w, 1, 0, w->step, h0, w->N[1], mh, mh_full, batch);
}
void dyb200_wgrad_seq_done(dyb200_wgrad* w) {
  w->h_col = w->x_cols - w->step;   // the planes of the last step's h input are the most recent ones
  if (w->x_cols > w->kb) w->kb = w->x_cols;
}
int dyb200_tc_make_tmap(dyb200_ctx* ctx, void* map, float* plane, uint32_t rows, uint32_t K, uint32_t pitch, uint32_t box_rows) {
  EncodeTiledFn enc;
  int rc = get_encoder(ctx, &enc);
  if (rc) return rc;
  return make_map(ctx, enc, (CUtensorMap*)map, plane, rows, K, pitch, box_rows);
}
uint32_t dyb200_tc_tile_cols(uint32_t N) { return tile_cols(N); }
uint32_t dyb200_wgrad_rows(const dyb200_wgrad* w) { return w->M; }
uint32_t dyb200_wgrad_fill(const dyb200_wgrad* w) { return w->k; }

extern "C" {

int dyb200_wgrad_create(dyb200_ctx* ctx, uint32_t M, uint32_t N0, uint32_t N1, uint32_t Kcap, dyb200_wgrad** out) {
  DYB_CHECK_ARG(ctx, out && M > 0 && N0 > 0 && Kcap > 0, "wgrad_create: bad shape");
  dyb200_wgrad* w = (dyb200_wgrad*)calloc(1, sizeof(dyb200_wgrad));
  if (!w) return dyb200_fail(ctx, DYB200_ENOMEM, "wgrad_create: host allocation failed");
  w->M = M; w->Mp = round_up(M, 32); w->N[0] = N0; w->N[1] = N1; w->Np[0] = round_up(N0, 32); w->Np[1] = round_up(N1, 32);
  w->Kcap = round_up(Kcap, 32); w->k = 0; w->kb = 0;
  w->x_cols = 0; w->h_col = 0xffffffffu; w->step = 0;
  auto alloc = [&](PackedOp* p, uint32_t rows) -> bool {
    p->rows = rows; p->K = 0; p->pitch = w->Kcap;
    size_t bytes = (size_t)rows * w->Kcap * sizeof(float);
    if (cudaMalloc((void**)&p->hi, bytes) != cudaSuccess) { cudaGetLastError(); p->hi = nullptr; return false; }
    if (cudaMalloc((void**)&p->lo, bytes) != cudaSuccess) { cudaGetLastError(); p->lo = nullptr; return false; }
    return true;
  };
  // (Kcap rows of Mp / Np floats, the same bytes as Mp / Np rows of Kcap; zeroed once so that the padding beyond M / N stays
  // finite)
  bool ok = alloc(&w->A, w->Mp) && alloc(&w->B[0], w->Np[0]) && (N1 == 0 || alloc(&w->B[1], w->Np[1]));
  if (ok) {
    w->A.rows = M; w->A.pitch = w->Mp; w->A.mn_major = 1;
    for (int j = 0; j < 2; ++j) { w->B[j].rows = w->N[j]; w->B[j].pitch = w->Np[j]; w->B[j].mn_major = 1; }
    PackedOp* ps[3] = {&w->A, &w->B[0], &w->B[1]};
    for (int q = 0; q < 3 && ok; ++q) {
      if (!ps[q]->hi) continue;
      const size_t bytes = (size_t)ps[q]->pitch * w->Kcap * sizeof(float);
      ok = cudaMemset(ps[q]->hi, 0, bytes) == cudaSuccess && cudaMemset(ps[q]->lo, 0, bytes) == cudaSuccess;
    }
    if (!ok) cudaGetLastError();
  }
  if (!ok) {
    for (PackedOp* p : {&w->A, &w->B[0], &w->B[1]}) { if (p->hi) cudaFree(p->hi); if (p->lo) cudaFree(p->lo); }
    free(w);
    return dyb200_fail(ctx, DYB200_ENOMEM, "wgrad_create: cudaMalloc failed for M %u, N %u + %u, K %u", M, N0, N1, Kcap);
  }
  *out = w;
  return DYB200_OK;
}

int dyb200_wgrad_destroy(dyb200_wgrad* w) {
  if (!w) return DYB200_OK;
  for (PackedOp* p : {&w->A, &w->B[0], &w->B[1]}) { if (p->hi) cudaFree(p->hi); if (p->lo) cudaFree(p->lo); }
  free(w);
  return DYB200_OK;
}

// Appends one step: a = A_t (M x k, leading dimension lda), b0 / b1 = B_t operands (N x k) with optional
// multiplicative masks indexed like b (mask[r + (full ? ld * c : 0)]).
int dyb200_wgrad_push(dyb200_wgrad* w, uint32_t k, const float* a, uint32_t lda, const float* b0, uint32_t ldb0,
                      const float* mask0, int mask0_full, const float* b1, uint32_t ldb1, const float* mask1,
                      int mask1_full, dyb200_ctx* ctx) {
  PackJobs batch;
  dyb200_tc_pack_begin(&batch);
  int rc = dyb200_wgrad_push_batched(w, k, a, lda, b0, ldb0, mask0, mask0_full, b1, ldb1, mask1, mask1_full, ctx, &batch);
  if (rc) return rc;
  return dyb200_tc_pack_flush(ctx, &batch);
}

// C0 += A * B0^T (and C1 += A * B1^T) over everything pushed since the last flush; empties the accumulator.
int dyb200_wgrad_pack_inputs(dyb200_wgrad* w, const dyb200_tensor* x_all, const dyb200_tensor* mask_x, uint32_t step, dyb200_ctx* ctx) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  DYB_CHECK_ARG(ctx, w && x_all && x_all->v, "wgrad_pack_inputs: null argument");
  DYB_CHECK_ARG(ctx, step > 0 || !mask_x, "wgrad_pack_inputs: steps of varying width (step = 0) take no mask");
  const uint32_t I = t_rows(x_all), n = x_all->bd;
  DYB_CHECK_ARG(ctx, t_cols(x_all) == 1 && I == w->N[0] && w->N[1] > 0 && n <= w->Kcap && (step == 0 || n % step == 0),
                "wgrad_pack_inputs: x is %u x %u, the accumulator expects %u rows, at most %u columns, whole steps of %u", I, n, w->N[0], w->Kcap, step);
  DYB_CHECK_ARG(ctx, !mask_x || (t_rows(mask_x) == I && (mask_x->bd == step || mask_x->bd == 1)), "wgrad_pack_inputs: mask shape mismatch");
  const float* mk = mask_x ? mask_x->v : nullptr;
  const int full = mask_x ? mask_x->bd == step : 0;
  PackJobs batch;
  dyb200_tc_pack_begin(&batch);
  // row = column of the sequence, reduction index of the forward product = input feature
  int rc = pack(ctx, x_all->v, I, 1, n, I, mk, I, full, w->B[0].hi, w->B[0].lo, w->Np[0], &batch, step ? step : n);
  if (!rc) rc = pack_flush_impl(ctx, &batch);
  if (rc) return rc;
  w->x_cols = n; w->step = step; w->h_col = 0xffffffffu;
  if (n > w->kb) w->kb = n;
  return DYB200_OK;
}

int dyb200_wgrad_flush(dyb200_wgrad* w, float* C0, uint32_t ldc0, float* C1, uint32_t ldc1, dyb200_ctx* ctx) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  DYB_CHECK_ARG(ctx, w && C0 && (w->N[1] == 0 || C1), "wgrad_flush: null argument");
  // (pre-split inputs belong to one sequence: the next one has to call dyb200_wgrad_pack_inputs again)
  const uint32_t kb_seen = w->kb;
  w->x_cols = 0; w->h_col = 0xffffffffu;
  if (w->k == 0) { w->kb = 0; return DYB200_OK; }
  DYB_CHECK_ARG(ctx, kb_seen >= w->k, "wgrad_flush: the B operands cover %u columns, the A operand %u", kb_seen, w->k);
  PackedOp A = w->A;
  A.K = w->k;
  for (int j = 0; j < 2; ++j) {
    if (w->N[j] == 0) continue;
    PackedOp B = w->B[j];   // (MN-major: rows = N[j], one plane row per column)
    B.K = w->k;
    GemmEpilogue e{EPI_ACCUM, j == 0 ? C0 : C1, j == 0 ? ldc0 : ldc1, nullptr, 0, 0.f, nullptr, 0, 0};
    int rc = dyb200_tc_gemm_packed(ctx, w->M, w->N[j], 1, &A, &B, e);
    if (rc) return rc;
  }
  w->k = 0;
  w->kb = 0;
  return DYB200_OK;
}

}  // extern "C"
