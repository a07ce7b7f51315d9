// One LSTM layer over ALL time steps of a sequence in one kernel (forward): the call pattern of
// CompactVanillaLSTMBuilder::add_input_impl (dynet/lstm.cc:1044-1080) driven through RNNBuilder::add_input
// (dynet/rnn.h:120) for a batch of equally long sequences, i.e. T times
//     gates_t = VanillaLSTMGates(x_t, h_{t-1}, Wx, Wh, b [, masks]);  c_t = VanillaLSTMC(c_{t-1}, gates_t);
//     h_t = VanillaLSTMH(c_t, gates_t).
// The per-step form (dyb200_vanilla_lstm_fwd_fused_at) launches one 3xTF32 product per step.  Here the CTAs of that
// product stay resident for the whole sequence: CTA (mt, nt[, split]) owns the same 128 interleaved gate rows (32 hidden
// units) x BNT batch columns in every step.  What that buys per step: no launch gap, no TMEM allocation / barrier set-up /
// tensor-map fetch, and the Wx x_{t+1} share of a step's k-blocks (which does not depend on h_t) runs while the epilogue of
// step t is still writing and handing over.  The weights are not kept in shared memory; their split planes stay in L2.
//
// Hand-over of h_t: the epilogue writes h_t .* mask_h as TF32 hi / lo operand planes (rows = batch columns) and then
// adds 1 to a counter of its column block; the TMA warp of every CTA of that column block waits for the count of the
// previous step before its first Wh h k-block.  The wait is bounded like every other wait of these kernels: on expiry
// the CTA sets DYB200_FLAG_WAIT_TIMEOUT, skips its stores, keeps taking part in the hand-shakes so that nothing else
// stalls, frees its TMEM and returns.
//
// Values are bit for bit those of the per-step calls: the same k-blocks in the same accumulation chains (cut every
// kChunkKB k-blocks), the same K split (k_split) reduced in split order through distributed shared memory, the same epilogue.
#include "seq_dev.cuh"

namespace {

struct SeqFwd {
  uint32_t T, B, H;                 // time steps, batch columns per step, hidden units (M = 4H gate rows)
  uint32_t kb0, kb1;                // k-blocks of Wx x and of Wh h
  float* gates; float* cs; float* hs;   // outputs of step t at + t * 4H * B / + t * H * B
  const float* c0;                  // cell state before the first step
  const float* bias; float forget_bias;
  // operand planes of h .* mask_h: row = column of the sequence (K-major right operand of the gate products; the layer's
  // weight-gradient product reads the same planes MN-major)
  float *hn_hi, *hn_lo; uint32_t hn_pitch;
  const float* hmask; uint32_t hmask_ld; int hmask_full;
  uint32_t* ready;                  // one arrival counter per column block, zero at launch
  uint32_t* flags;
};

// grid = (4H / 128, B / BNT, S); with S > 1 the S CTAs of a tile are one thread-block cluster (1 x 1 x S).  S (1, 2, 4 or 8) is
// a template parameter so that the column exchange indexes registers statically.
template <int BNT, uint32_t S>
__global__ void __launch_bounds__(kThreads, 1) k_lstm_seq_fwd(const __grid_constant__ TmapPack tm, const SeqFwd a) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // 64-column tiles need 48 KiB per stage, so the ring holds four of them: at 0.4 us per k-block three stages do not cover
  // the latency of a tile fetch
  constexpr int kStages = BNT == 64 ? 4 : 3;
  constexpr int kStageBytes = 2 * TILE_BYTES + 2 * BNT * BK * 4;
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], acc_full[kSeqBufs], acc_empty[kSeqBufs], park_full, park_free;
  __shared__ uint32_t tmem_base_slot;
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* park = reinterpret_cast<float*>(ring + (size_t)kStages * kStageBytes);   // 64 columns x BM rows
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int TILE_B_BYTES = BNT * BK * 4;
  constexpr int STAGE_TX = 2 * TILE_BYTES + 2 * TILE_B_BYTES;
  const uint32_t rank = blockIdx.z;
  const uint32_t m0 = blockIdx.x * BM, n0 = blockIdx.y * BNT;
  const KSplit ks = k_split(a.kb0, a.kb1, rank, S);
  const uint32_t total = ks.n0 + ks.n1;          // k-blocks of this CTA per time step
  const uint32_t M = 4 * a.H, N = a.B;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (uint32_t q = 0; q < kSeqBufs; ++q) { mbar_init(&acc_full[q], 1); mbar_init(&acc_empty[q], kEpiWarps); }
    mbar_init(&park_full, 4 * S); mbar_init(&park_free, S);   // arrivals: the 4 sending warps of every CTA / one per CTA
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (threadIdx.x == 32 * 2) {
#pragma unroll
    for (int q = 0; q < 8; ++q) asm volatile("prefetch.tensormap [%0];" ::"l"(&tm.t[q]) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kSeqBufs * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  if (S > 1) cluster_sync_all();   // every CTA's barriers exist before anyone arrives on them remotely
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      // TMA producer.  Step t reads Wx / Wh rows [m0, m0 + 128) and the operand planes of columns [t B + n0, + BNT).
      uint32_t s = 0, ph = 0;
      bool fail = false;
      const uint32_t per_step = gridDim.x * S;   // arrivals per column block and step: every CTA that writes a piece of h_t
      for (uint32_t t = 0; t < a.T && !fail; ++t) {
        const int brow = (int)(t * a.B + n0);
        for (uint32_t it = 0; it < total;) {
          if (it == ks.n0 && t > 0) {
            // The Wh h share of this step needs the planes of h_{t-1}, complete for this column block.  The weight tiles
            // of its first k-blocks do not: they are requested before the wait (a stage's barrier completes when both its
            // weight and its activation tiles have arrived), so only the small activation tiles are still to come afterwards.
            const uint32_t pre = min((uint32_t)kStages, ks.n1);
            uint32_t s2 = s, ph2 = ph;
            for (uint32_t j = 0; j < pre && !fail; ++j) {
              if (!mbar_wait(&empty_bar[s2], ph2 ^ 1)) { fail = true; break; }
              unsigned char* st = ring + (size_t)s2 * kStageBytes;
              mbar_expect_tx(&full_bar[s2], STAGE_TX);
              tma_load_2d(st, &tm.t[4], &full_bar[s2], (int)((ks.b1 + j) * BK), (int)m0);
              tma_load_2d(st + TILE_BYTES, &tm.t[5], &full_bar[s2], (int)((ks.b1 + j) * BK), (int)m0);
              if (++s2 == kStages) { s2 = 0; ph2 ^= 1; }
            }
            if (fail) break;
            if (!wait_counter(a.ready + blockIdx.y, t * per_step)) { fail = true; break; }
            asm volatile("fence.proxy.async.global;" ::: "memory");   // generic-proxy stores of other CTAs -> this CTA's TMA reads
            for (uint32_t j = 0; j < pre; ++j) {
              unsigned char* st = ring + (size_t)s * kStageBytes;
              tma_load_2d(st + 2 * TILE_BYTES, &tm.t[6], &full_bar[s], (int)((ks.b1 + j) * BK), brow);
              tma_load_2d(st + 2 * TILE_BYTES + TILE_B_BYTES, &tm.t[7], &full_bar[s], (int)((ks.b1 + j) * BK), brow);
              if (++s == kStages) { s = 0; ph ^= 1; }
            }
            it += pre;
            continue;
          }
          if (!mbar_wait(&empty_bar[s], ph ^ 1)) { fail = true; break; }
          const uint32_t pair = it < ks.n0 ? 0 : 1, kblk = pair ? ks.b1 + (it - ks.n0) : ks.b0 + it;
          unsigned char* st = ring + (size_t)s * kStageBytes;
          mbar_expect_tx(&full_bar[s], STAGE_TX);
          tma_load_2d(st, &tm.t[4 * pair + 0], &full_bar[s], (int)(kblk * BK), (int)m0);
          tma_load_2d(st + TILE_BYTES, &tm.t[4 * pair + 1], &full_bar[s], (int)(kblk * BK), (int)m0);
          tma_load_2d(st + 2 * TILE_BYTES, &tm.t[4 * pair + 2], &full_bar[s], (int)(kblk * BK), brow);
          tma_load_2d(st + 2 * TILE_BYTES + TILE_B_BYTES, &tm.t[4 * pair + 3], &full_bar[s], (int)(kblk * BK), brow);
          if (++s == kStages) { s = 0; ph ^= 1; }
          ++it;
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
      // stage, phase and chunk counters run on across time steps; an accumulation chain never crosses a step
      uint32_t s = 0, ph = 0, chunk = 0, buf = 0;
      bool fail = false;
      for (uint32_t t = 0; t < a.T && !fail; ++t) {
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
    // epilogue warps 2..9: TMEM lanes 32 (warp % 4) .. +31; warps 2-5 hold columns 0-63 of the tile, warps 6-9 columns 64-127
    const uint32_t quarter = warp & 3, half = (warp - 2) >> 2;
    const uint32_t te = threadIdx.x - 64;
    const bool has_cols = 64 * half < BNT;
    const uint32_t nchunks = (total + kChunkKB - 1) / kChunkKB;
    // In the cooperative pass over a finished 64-column half this thread owns hidden units [u, u + 4) (rows 32 q + l of the
    // tile are gate q of unit 32 mt + l) for the columns te / 8 and te / 8 + 32 of that half.
    const uint32_t l = 4 * (te & 7), u = blockIdx.x * 32 + l;
    // The 64 columns of a half are finished by the S CTAs of the cluster, w columns each (S is a power of two here): rank r
    // takes columns [r w, r w + w).  Every CTA sends its partial sums of those columns straight into rank r's exchange
    // buffer (slot = sender's rank), so the owner adds S slots from its own shared memory - no remote loads, whose round
    // trips would sit on the step's critical path.  Without a K split (S = 1) the buffer is simply the parked half tile.
    constexpr uint32_t w = 64 / S;
    const uint32_t c_lo = rank * w, c_hi = c_lo + w;
    uint32_t peer[8];   // this CTA's exchange buffer as seen ... and the peers': shared::cluster addresses
#pragma unroll
    for (uint32_t r = 0; r < 8; ++r) {
      peer[r] = smem_u32(park);
      if (S > 1 && r < S) asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer[r]) : "r"(smem_u32(park)), "r"(r));
    }
    float4 bias[4];   // the same for every step
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      bias[q] = ld4(a.bias + (size_t)q * a.H + u);
      if (q == 1) { bias[q].x += a.forget_bias; bias[q].y += a.forget_bias; bias[q].z += a.forget_bias; bias[q].w += a.forget_bias; }
    }
    uint32_t cg = 0, pf_phase = 0, pr_phase = 0;
    bool ok = true;   // the same for all 256 epilogue threads after every bar_and below
    const size_t HB = (size_t)a.H * a.B;
#pragma unroll 1
    for (uint32_t t = 0; t < a.T; ++t) {
      float* const gates_t = a.gates + (size_t)t * 4 * HB;
      const float* const c_prev = t ? a.cs + (size_t)(t - 1) * HB : a.c0;
      float* const c_out = a.cs + (size_t)t * HB;
      float* const h_out = a.hs + (size_t)t * HB;
      const bool emit = t + 1 < a.T;   // h_t is the next step's input
      // h_t .* mask_h as operand planes of step t + 1: rows (t + 1) B .. of the planes
      float* const hn_hi = a.hn_hi + (size_t)(t + 1) * a.B * a.hn_pitch;
      float* const hn_lo = a.hn_lo + (size_t)(t + 1) * a.B * a.hn_pitch;
      // previous cell states and mask values of the columns this thread finishes (c_prev was written by this same thread one
      // step earlier); fetched now, while the products of the step run
      float4 cp[BNT / 64][2], hm[BNT / 64][2];
#pragma unroll
      for (int hh = 0; hh < BNT / 64; ++hh)
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const uint32_t c = (te >> 3) + 32 * k, n = n0 + 64 * hh + c;
          const bool mine = n < N && c >= c_lo && c < c_hi;
          cp[hh][k] = mine ? ld4(c_prev + u + (size_t)a.H * n) : make_float4(0.f, 0.f, 0.f, 0.f);
          hm[hh][k] = (mine && a.hmask) ? ld4(a.hmask + u + (a.hmask_full ? (size_t)a.hmask_ld * n : 0)) : make_float4(1.f, 1.f, 1.f, 1.f);
        }
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
#pragma unroll
      for (int hh = 0; hh < BNT / 64; ++hh) {
        // Every CTA's exchange buffer is free once its owner has read the previous pass: the owners say so on park_free
        // (S > 1), or this CTA's own threads have left the previous pass (the barrier at its end).
        if (S > 1 && ok && !mbar_wait_cluster(&park_free, pr_phase ^ 1)) ok = false;
        if (half == (uint32_t)hh) {
          // column q of this half goes to rank q / w, slot = this rank, as column q % w; 32 consecutive rows per warp store
          const uint32_t row = quarter * 32 + lane;
#pragma unroll
          for (int q = 0; q < 64; ++q) {
            const uint32_t dst = peer[(uint32_t)q / w] + 4u * (((rank * w + (uint32_t)q % w) * BM) + row);
            if (S > 1) asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst), "f"(sum[q]) : "memory");
            else park[(size_t)q * BM + row] = sum[q];
          }
        }
        if (S > 1) {
          // each sending warp reports on its own: its lanes' stores are ordered before the arrivals by the warp barrier,
          // so a receiver can start as soon as the 4 S sending warps of the cluster are through
          if (half == (uint32_t)hh) {
            __syncwarp();
            if (lane < S) mbar_arrive_remote(&park_full, lane);   // (release at cluster scope)
          }
          const bool got = mbar_wait_cluster(&park_full, pf_phase);
          ok = bar_and(1, 256, ok && got) != 0;
          pf_phase ^= 1; pr_phase ^= 1;
        } else {
          ok = bar_and(1, 256, ok) != 0;
        }
        // ---- the LSTM epilogue on this CTA's columns of the half: the arithmetic of epilogue_pass (EPI_LSTM_CELL), the S
        // partial sums added in split order, c / h / the operand planes of h.  The planes of h, which the next step waits for,
        // go out first and are published before the other stores are issued.
        const uint32_t nh = n0 + 64 * hh;
        const bool last_pass = hh == BNT / 64 - 1;
        float4 g[2][4], cn[2], hv[2], phi[2], plo[2];
        bool live[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const uint32_t c = (te >> 3) + 32 * k, n = nh + c;
          live[k] = ok && n < N && c >= c_lo && c < c_hi;
          if (!live[k]) continue;
          const float* col = park + (size_t)(c - c_lo) * BM + l;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float4 acc = ld4(col + 32 * q);
#pragma unroll
            for (uint32_t r = 1; r < 8; ++r)
              if (r < S) { const float4 pv = ld4(col + (size_t)r * w * BM + 32 * q); acc.x += pv.x; acc.y += pv.y; acc.z += pv.z; acc.w += pv.w; }
            const float4 x = make_float4(acc.x + bias[q].x, acc.y + bias[q].y, acc.z + bias[q].z, acc.w + bias[q].w);
            g[k][q] = q == 3 ? make_float4(gate_tanh(x.x), gate_tanh(x.y), gate_tanh(x.z), gate_tanh(x.w))
                             : make_float4(gate_sigmoid(x.x), gate_sigmoid(x.y), gate_sigmoid(x.z), gate_sigmoid(x.w));
          }
          const float4 cv = cp[hh][k];
          cn[k] = make_float4(lstm_cell_c(g[k][0].x, g[k][3].x, g[k][1].x, cv.x), lstm_cell_c(g[k][0].y, g[k][3].y, g[k][1].y, cv.y),
                              lstm_cell_c(g[k][0].z, g[k][3].z, g[k][1].z, cv.z), lstm_cell_c(g[k][0].w, g[k][3].w, g[k][1].w, cv.w));
          hv[k] = make_float4(lstm_cell_h(g[k][2].x, cn[k].x), lstm_cell_h(g[k][2].y, cn[k].y), lstm_cell_h(g[k][2].z, cn[k].z), lstm_cell_h(g[k][2].w, cn[k].w));
          if (emit) {
            // h .* mask_h as the next step's operand planes (the values of epi_emit_h)
            const float4 mk = hm[hh][k];
            const float4 hmk = a.hmask ? make_float4(hv[k].x * mk.x, hv[k].y * mk.y, hv[k].z * mk.z, hv[k].w * mk.w) : hv[k];
            split_tf32(hmk.x, phi[k].x, plo[k].x); split_tf32(hmk.y, phi[k].y, plo[k].y);
            split_tf32(hmk.z, phi[k].z, plo[k].z); split_tf32(hmk.w, phi[k].w, plo[k].w);
            st4(hn_hi + (size_t)n * a.hn_pitch + u, phi[k]);
            st4(hn_lo + (size_t)n * a.hn_pitch + u, plo[k]);
          }
        }
        // all reads of the exchange buffer are done (the next pass may overwrite it) and, in the last pass, every thread has
        // issued its stores of the operand planes
        bar_sync(1, 256);
        if (S > 1 && te < S) mbar_arrive_remote(&park_free, te);
        if (last_pass && emit && te == 0) {
          // One thread publishes: its release orders all stores it has observed, through the barrier, before the counter
          // update (cumulativity), for the generic and for the async proxy (the readers are TMA loads).
          asm volatile("fence.proxy.async.global;" ::: "memory");
          signal_counter(a.ready + blockIdx.y);
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          if (!live[k]) continue;
          const uint32_t n = nh + (te >> 3) + 32 * k;
#pragma unroll
          for (int q = 0; q < 4; ++q) st4(gates_t + (size_t)q * a.H + u + (size_t)M * n, g[k][q]);
          const size_t ei = u + (size_t)a.H * n;
          st4(c_out + ei, cn[k]);
          st4(h_out + ei, hv[k]);
        }
      }
    }
    if (!ok && lane == 0) atomicOr(a.flags, DYB200_FLAG_WAIT_TIMEOUT);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (S > 1) cluster_sync_all();   // no CTA leaves while another may still arrive on its barriers
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kSeqBufs * BN) : "memory");
  }
}

}  // namespace

// ---- host side ---------------------------------------------------------------------------------------------------------
namespace {

// How many clusters of S CTAs of the sequence kernel fit on the GPU at once (remembered per context = per device).
template <int BNT, uint32_t S>
int seq_clusters_that_fit(dyb200_ctx* ctx) {
  int& mc = ctx->seq_max_clusters[BNT == 64 ? 0 : 1][S];
  if (mc == 0) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(1, 1, S); cfg.blockDim = dim3(kThreads, 1, 1); cfg.dynamicSmemBytes = SMEM_SEQ_BYTES; cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = S;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, k_lstm_seq_fwd<BNT, S>, &cfg) != cudaSuccess) { (void)cudaGetLastError(); n = -1; }
    mc = n > 0 ? n : -1;
  }
  return mc;
}

template <int BNT, uint32_t S>
int launch_seq_fwd(dyb200_ctx* ctx, const TmapPack& tm, const SeqFwd& a, dim3 grid, double flops, uint32_t K) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid; cfg.blockDim = dim3(kThreads, 1, 1); cfg.dynamicSmemBytes = SMEM_SEQ_BYTES; cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (grid.z > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = grid.z;
    ++na;
  }
  // All CTAs wait on one another, so they have to be resident together.  The grid never exceeds what the GPU holds at
  // once (checked by the caller); the cooperative attribute additionally makes the driver schedule them as one gang.  A
  // driver that refuses the attribute for this launch shape gets a plain launch (the waits are bounded either way).
  if (ctx->seq_coop >= 0) {
    attr[na].id = cudaLaunchAttributeCooperative;
    attr[na].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = na + 1;
    GemmProfScope scope(ctx, flops, 1, 4 * a.H, a.B * a.T, K, EPI_LSTM_CELL);
    cudaError_t e = cudaLaunchKernelEx(&cfg, k_lstm_seq_fwd<BNT, S>, tm, a);
    if (e == cudaSuccess) { ctx->seq_coop = 1; ctx->launches++; return DYB200_OK; }
    (void)cudaGetLastError();
    if (ctx->seq_coop == 1) return dyb200_fail(ctx, DYB200_ECUDA, "sequence kernel launch failed: %s", cudaGetErrorString(e));
    ctx->seq_coop = -1;
  }
  cfg.attrs = attr; cfg.numAttrs = na;
  GemmProfScope scope(ctx, flops, 1, 4 * a.H, a.B * a.T, K, EPI_LSTM_CELL);
  cudaLaunchKernelEx(&cfg, k_lstm_seq_fwd<BNT, S>, tm, a);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

// the (tile width, K splits) instantiations behind one switch
enum SeqOp { SEQ_SET_SMEM, SEQ_FIT, SEQ_LAUNCH };
template <int BNT, uint32_t S>
int seq_fwd_do(SeqOp op, dyb200_ctx* ctx, const TmapPack* tm, const SeqFwd* a, dim3 grid, double flops, uint32_t K) {
  if (op == SEQ_SET_SMEM) {
    // (the shared-memory limit of the kernel has to be raised before its occupancy is asked for)
    const uint32_t bit = (BNT == 64 ? 16u : 256u) << (S == 1 ? 0 : S == 2 ? 1 : S == 4 ? 2 : 3);
    if (!(ctx->func_attr_done & bit)) {
      DYB_CUDA(ctx, cudaFuncSetAttribute(k_lstm_seq_fwd<BNT, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_SEQ_BYTES));
      ctx->func_attr_done |= bit;
    }
    return DYB200_OK;
  }
  if (op == SEQ_FIT) return seq_clusters_that_fit<BNT, S>(ctx);
  return launch_seq_fwd<BNT, S>(ctx, *tm, *a, grid, flops, K);
}
int seq_fwd_dispatch(SeqOp op, uint32_t bn, uint32_t S, dyb200_ctx* ctx, const TmapPack* tm = nullptr, const SeqFwd* a = nullptr,
                     dim3 grid = dim3(), double flops = 0, uint32_t K = 0) {
  if (bn == 64) {
    switch (S) {
      case 1: return seq_fwd_do<64, 1>(op, ctx, tm, a, grid, flops, K);
      case 2: return seq_fwd_do<64, 2>(op, ctx, tm, a, grid, flops, K);
      case 4: return seq_fwd_do<64, 4>(op, ctx, tm, a, grid, flops, K);
      default: return seq_fwd_do<64, 8>(op, ctx, tm, a, grid, flops, K);
    }
  }
  switch (S) {
    case 1: return seq_fwd_do<128, 1>(op, ctx, tm, a, grid, flops, K);
    case 2: return seq_fwd_do<128, 2>(op, ctx, tm, a, grid, flops, K);
    case 4: return seq_fwd_do<128, 4>(op, ctx, tm, a, grid, flops, K);
    default: return seq_fwd_do<128, 8>(op, ctx, tm, a, grid, flops, K);
  }
}

}  // namespace

extern "C" {

int dyb200_vanilla_lstm_seq_fwd(const dyb200_tensor* x_all, const dyb200_tensor* h0, const dyb200_tensor* c0,
                                const dyb200_tensor* Wx, const dyb200_tensor* Wh, const dyb200_tensor* b,
                                const dyb200_tensor* mask_x, const dyb200_tensor* mask_h, const dyb200_lstm_gates_attrs* attrs,
                                dyb200_tensor* gates_all, dyb200_tensor* c_all, dyb200_tensor* h_all, dyb200_wgrad* deferred,
                                uint32_t steps, dyb200_ctx* ctx) {
  DYB_CHECK_ARG(ctx, x_all && h0 && c0 && Wx && Wh && b && attrs && gates_all && c_all && h_all && steps > 0, "lstm_seq_fwd: null argument");
  DYB_CHECK_ARG(ctx, (attrs->dropout != 0) == (mask_x != nullptr && mask_h != nullptr), "lstm_seq_fwd: masks must be given exactly when dropout is set");
  DYB_CHECK_ARG(ctx, x_all->nd == 1 && x_all->bd % steps == 0, "lstm_seq_fwd: x_all must be Dim({I}, steps * batch)");
  const uint32_t T = steps, B = x_all->bd / T, I = t_dim(x_all, 0), H = t_dim(h0, 0), G = 4 * H;
  const size_t HB = (size_t)H * B;
  DYB_CHECK_ARG(ctx, h0->nd == 1 && h0->bd == B && c0->bd == B && t_dim(c0, 0) == H, "lstm_seq_fwd: h0 / c0 must be Dim({H}, batch)");
  DYB_CHECK_ARG(ctx, t_size(gates_all) == 4 * HB * T && t_size(c_all) == HB * T && t_size(h_all) == HB * T, "lstm_seq_fwd: outputs must hold all %u steps", T);
  if (HB == 0) return DYB200_OK;
  int rc;
  if (deferred && (rc = dyb200_wgrad_pack_inputs(deferred, x_all, mask_x, B, ctx))) return rc;
  const float* mx = attrs->dropout ? mask_x->v : nullptr;
  const float* mh = attrs->dropout ? mask_h->v : nullptr;
  const int mh_full = mh ? mask_h->bd == B : 0;
  (void)mx;

  // ---- one kernel for the whole sequence, when its CTAs can all be resident ----
  const uint32_t bn = dyb200_tc_tile_cols(B);
  const uint32_t kb0 = (I + 31) / 32, kb1 = (H + 31) / 32, kb_total = kb0 + kb1;
  bool persistent = ctx->seq_kernels && deferred && T >= 2 && attrs->weightnoise_std == 0.f && H % 32 == 0 && I % 4 == 0 && B % bn == 0 &&
                    dyb200_tc_eligible(G, B, 2.0 * G * B * (I + H)) && Wx->nd == 2 && Wx->d[0] == G && Wx->d[1] == I && Wh->nd == 2 &&
                    Wh->d[0] == G && Wh->d[1] == H && t_size(b) == G && aligned16(gates_all->v) && aligned16(b->v) && aligned16(c0->v) &&
                    aligned16(c_all->v) && aligned16(h_all->v) && (!mh || aligned16(mh)) &&
                    (!attrs->dropout || ((mask_h->bd == B || mask_h->bd == 1) && t_dim(mask_h, 0) == H));
  uint32_t S = 1;
  SeqPlanes pl;
  if (persistent) {
    S = dyb200_tc_splits(ctx, G, B, kb_total);
    const uint32_t per = (kb_total + S - 1) / S;
    S = (kb_total + per - 1) / per;
    const uint32_t tiles = (G / BM) * (B / bn);
    if (S > 8 || (S & (S - 1)) != 0 || (S > 1 && !ctx->cluster_splitk)) persistent = false;   // (the column exchange wants a power of two)
    else {
      if ((rc = seq_fwd_dispatch(SEQ_SET_SMEM, bn, S, ctx))) return rc;
      if (S > 1) {
        const int fit = seq_fwd_dispatch(SEQ_FIT, bn, S, ctx);
        persistent = fit > 0 && tiles <= (uint32_t)fit;
      } else {
        persistent = tiles <= (uint32_t)ctx->sm_count;   // one CTA per SM (225 KB of shared memory each)
      }
    }
    if (B / bn > 32) persistent = false;                // one hand-over counter per column block
    if (persistent) persistent = dyb200_wgrad_seq_planes(deferred, T, B, &pl);
  }
  if (persistent) {
    { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
    DYB_CHECK_ARG(ctx, dyb200_wgrad_rows(deferred) == G, "lstm_seq_fwd: the deferred accumulator has %u rows, the layer %u", dyb200_wgrad_rows(deferred), G);
    PackedOp A[2];
    if ((rc = dyb200_tc_param_gates(ctx, Wx->v, G, G, I, &A[0]))) return rc;
    if ((rc = dyb200_tc_param_gates(ctx, Wh->v, G, G, H, &A[1]))) return rc;
    PackJobs batch;
    dyb200_tc_pack_begin(&batch);
    if ((rc = dyb200_wgrad_seq_h0(deferred, h0->v, mh, mh_full, ctx, &batch))) return rc;
    if ((rc = dyb200_tc_pack_flush(ctx, &batch))) return rc;
    TmapPack tm;
    memset(&tm, 0, sizeof(tm));
    if ((rc = dyb200_tc_make_tmap(ctx, &tm.t[0], A[0].hi, G, I, A[0].pitch, BM))) return rc;
    if ((rc = dyb200_tc_make_tmap(ctx, &tm.t[1], A[0].lo, G, I, A[0].pitch, BM))) return rc;
    if ((rc = dyb200_tc_make_tmap(ctx, &tm.t[2], pl.X.hi, T * B, I, pl.X.pitch, bn))) return rc;
    if ((rc = dyb200_tc_make_tmap(ctx, &tm.t[3], pl.X.lo, T * B, I, pl.X.pitch, bn))) return rc;
    if ((rc = dyb200_tc_make_tmap(ctx, &tm.t[4], A[1].hi, G, H, A[1].pitch, BM))) return rc;
    if ((rc = dyb200_tc_make_tmap(ctx, &tm.t[5], A[1].lo, G, H, A[1].pitch, BM))) return rc;
    if ((rc = dyb200_tc_make_tmap(ctx, &tm.t[6], pl.Hs.hi, T * B, H, pl.Hs.pitch, bn))) return rc;
    if ((rc = dyb200_tc_make_tmap(ctx, &tm.t[7], pl.Hs.lo, T * B, H, pl.Hs.pitch, bn))) return rc;
    SeqFwd a;
    memset(&a, 0, sizeof(a));
    a.T = T; a.B = B; a.H = H; a.kb0 = kb0; a.kb1 = kb1;
    a.gates = gates_all->v; a.cs = c_all->v; a.hs = h_all->v; a.c0 = c0->v; a.bias = b->v; a.forget_bias = attrs->forget_gate_bias;
    a.hn_hi = pl.Hs.hi; a.hn_lo = pl.Hs.lo; a.hn_pitch = pl.Hs.pitch;
    a.hmask = mh; a.hmask_ld = H; a.hmask_full = mh_full;
    a.ready = ctx->dev_flags + DYB200_DEV_SEQ0;
    a.flags = ctx->dev_flags;
    DYB_CUDA(ctx, cudaMemsetAsync(a.ready, 0, 32 * sizeof(uint32_t), ctx->stream));
    const dim3 grid(G / BM, B / bn, S);
    const double flops = 2.0 * G * (double)B * (I + H) * T;
    rc = seq_fwd_dispatch(SEQ_LAUNCH, bn, S, ctx, &tm, &a, grid, flops, I + H);
    if (rc) return rc;
    dyb200_wgrad_seq_done(deferred);
    return DYB200_OK;
  }

  // ---- the same sequence as one call per time step ----
  for (uint32_t t = 0; t < T; ++t) {
    dyb200_tensor x = *x_all, hp = *h0, cp = *c0, g = *gates_all, c = *c_all, h = *h_all;
    x.bd = B; x.v = x_all->v + (size_t)t * I * B;
    g.bd = B; g.v = gates_all->v + (size_t)t * 4 * HB;
    c.bd = B; c.v = c_all->v + (size_t)t * HB;
    h.bd = B; h.v = h_all->v + (size_t)t * HB;
    if (t > 0) { hp.v = h_all->v + (size_t)(t - 1) * HB; cp.v = c_all->v + (size_t)(t - 1) * HB; }
    if ((rc = dyb200_vanilla_lstm_fwd_fused_at(&x, &hp, &cp, Wx, Wh, b, mask_x, mask_h, attrs, &g, &c, &h, deferred, t * B, ctx))) return rc;
  }
  return DYB200_OK;
}

}  // extern "C"
