// Autobatch data movers: ragged gather (parallel_memcpy) and ragged scatter-add
// (parallel_accumulate).  The pointer/length tables live in device memory, exactly as
// BatchedExecutionEngine uploads them (dynet/exec.cc:346-356, :398-408).
//
// Copy: one warp per slice when the slices are short (the autobatch case: 128-1024 floats, where a CTA per slice would
// leave most of its lanes without work), one CTA per slice otherwise; 128-bit loads/stores when both ends are 16-byte
// aligned, up to four vectors per lane in flight.
// Accumulate: when all targets are distinct (checked on the device with an address table) every slice is added by one warp
// (short slices) or CTA, in any order.  Otherwise slices are grouped by target pointer (in-CTA sort, <= 4096 slices per pass,
// all passes sorted in one launch) and one warp or CTA per distinct target adds that target's sources in ascending slice
// order, so slices that share a target are summed deterministically and without atomics.
#include "common.cuh"
#include "sortseg.cuh"

namespace {

constexpr int kThreads = 128;

__global__ void __launch_bounds__(kThreads) k_ragged_copy(int num_seqs, float* const* __restrict__ src,
                                                         float* const* __restrict__ trg, const size_t* __restrict__ len) {
  dyb_grid_dep_sync();
  for (int s = blockIdx.x; s < num_seqs; s += gridDim.x) {
    const float* a = src[s];
    float* b = trg[s];
    const size_t n = len[s];
    if (aligned16(a) && aligned16(b)) {
      const size_t n4 = n / 4;
      for (size_t i = threadIdx.x; i < n4; i += kThreads) st4(b + 4 * i, ld4_stream(a + 4 * i));
      for (size_t i = 4 * n4 + threadIdx.x; i < n; i += kThreads) b[i] = a[i];
    } else {
      for (size_t i = threadIdx.x; i < n; i += kThreads) b[i] = a[i];
    }
  }
}

// Short slices: warp w of the grid moves slices w, w + warps, ...  A lane owns the float4 pieces lane, lane + 32, ...
constexpr int kWarpSliceMax = 4096;   // floats: up to this length a slice is one warp's work
__global__ void __launch_bounds__(256) k_ragged_copy_warp(int num_seqs, float* const* __restrict__ src,
                                                         float* const* __restrict__ trg, const size_t* __restrict__ len) {
  dyb_grid_dep_sync();
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * 8;
  for (int s = blockIdx.x * 8 + (threadIdx.x >> 5); s < num_seqs; s += warps) {
    const float* a = src[s];
    float* b = trg[s];
    const size_t n = len[s];
    if (aligned16(a) && aligned16(b)) {
      const size_t n4 = n / 4;
      size_t i = lane;
      for (; i + 96 < n4; i += 128) {   // four vectors in flight
        const float4 v0 = ld4_stream(a + 4 * i), v1 = ld4_stream(a + 4 * (i + 32)), v2 = ld4_stream(a + 4 * (i + 64)), v3 = ld4_stream(a + 4 * (i + 96));
        st4(b + 4 * i, v0); st4(b + 4 * (i + 32), v1); st4(b + 4 * (i + 64), v2); st4(b + 4 * (i + 96), v3);
      }
      for (; i < n4; i += 32) st4(b + 4 * i, ld4_stream(a + 4 * i));
      for (size_t j = 4 * n4 + lane; j < n; j += 32) b[j] = a[j];
    } else {
      for (size_t j = lane; j < n; j += 32) b[j] = a[j];
    }
  }
}

// ---- are the targets distinct? ------------------------------------------------------------------------------------------
// In the executor's accumulate_tensors the targets are almost always distinct (one gradient slot per node argument); then
// no ordering is needed at all and every slice can be added by whichever warp gets to it.  Each slice inserts its target
// address into an open-addressing table (zeroed before the launch); meeting its own address again raises *dup, and the
// sorted path below runs instead.
__global__ void __launch_bounds__(256) k_ragged_probe(float* const* __restrict__ trg, uint32_t n, unsigned long long* __restrict__ table,
                                                     uint32_t mask, uint32_t* __restrict__ dup) {
  dyb_grid_dep_sync();
  for (uint32_t s = blockIdx.x * 256 + threadIdx.x; s < n; s += gridDim.x * 256) {
    const unsigned long long key = (unsigned long long)(uintptr_t)trg[s];
    uint32_t h = (uint32_t)(((key >> 2) * 0x9E3779B97F4A7C15ull) >> 32) & mask;
    for (uint32_t it = 0; it <= mask; ++it) {
      const unsigned long long old = atomicCAS(&table[h], 0ull, key);
      if (old == 0ull) break;
      if (old == key) { atomicOr(dup, 1u); break; }
      h = (h + 1) & mask;
    }
  }
}

// key = (target address / 4) << 18 | slice index (slice index < 2^18 within a pass).  CTA p sorts pass p (slices
// [p kSortMax, ...)); nothing to do when the targets are distinct.
__global__ void __launch_bounds__(kSortThreads) k_sort_targets(float* const* __restrict__ trg, uint32_t n_total,
                                                              uint32_t* __restrict__ slice_sorted,
                                                              uint32_t* __restrict__ group_sorted,
                                                              uint32_t* __restrict__ seg_start, uint32_t* __restrict__ nseg,
                                                              const uint32_t* __restrict__ dup) {
  dyb_grid_dep_sync();
  if (*dup == 0) return;
  __shared__ unsigned long long keys[kSortMax];
  __shared__ uint32_t scan[kSortThreads];
  const uint32_t base = blockIdx.x * kSortMax, n = min((uint32_t)kSortMax, n_total - base);
  uint32_t npow = 1;
  while (npow < n) npow <<= 1;
  for (uint32_t k = threadIdx.x; k < npow; k += kSortThreads) {
    unsigned long long key = ~0ull;
    if (k < n) key = (((unsigned long long)(uintptr_t)trg[base + k] >> 2) << 18) | k;
    keys[k] = key;
  }
  __syncthreads();
  // (per pass: n entries of slice_sorted / group_sorted, n + 1 of seg_start)
  sort_and_segment(keys, scan, n, npow, 18, slice_sorted + base, group_sorted + base, seg_start + base + blockIdx.x, nseg + blockIdx.x);
}

// Distinct targets: slice s is one warp's (or one CTA's) work, in any order.
template <bool WARP>
__global__ void __launch_bounds__(WARP ? 256 : kThreads) k_ragged_accumulate_direct(int num_seqs, float* const* __restrict__ src,
                                                                                   float* const* __restrict__ trg,
                                                                                   const size_t* __restrict__ len,
                                                                                   const uint32_t* __restrict__ dup) {
  dyb_grid_dep_sync();
  if (*dup != 0) return;
  const int group = WARP ? blockIdx.x * 8 + (threadIdx.x >> 5) : blockIdx.x, groups = WARP ? gridDim.x * 8 : gridDim.x;
  const uint32_t me = WARP ? (threadIdx.x & 31) : threadIdx.x, width = WARP ? 32 : kThreads;
  for (int s = group; s < num_seqs; s += groups) {
    const float* a = src[s];
    float* t = trg[s];
    const size_t n = len[s];
    if (aligned16(a) && aligned16(t)) {
      const size_t n4 = n / 4;
      size_t i = me;
      for (; i + width < n4; i += 2 * width) {   // two vectors per lane in flight
        const float4 o0 = ld4(t + 4 * i), o1 = ld4(t + 4 * (i + width)), v0 = ld4_stream(a + 4 * i), v1 = ld4_stream(a + 4 * (i + width));
        st4(t + 4 * i, make_float4(o0.x + v0.x, o0.y + v0.y, o0.z + v0.z, o0.w + v0.w));
        st4(t + 4 * (i + width), make_float4(o1.x + v1.x, o1.y + v1.y, o1.z + v1.z, o1.w + v1.w));
      }
      for (; i < n4; i += width) {
        const float4 o = ld4(t + 4 * i), v = ld4_stream(a + 4 * i);
        st4(t + 4 * i, make_float4(o.x + v.x, o.y + v.y, o.z + v.z, o.w + v.w));
      }
      for (size_t j = 4 * n4 + me; j < n; j += width) t[j] += a[j];
    } else {
      for (size_t j = me; j < n; j += width) t[j] += a[j];
    }
  }
}

// Shared targets, all sort passes in one launch.  A thread group (a CTA of kThreads threads, or a warp of a 256-thread
// CTA when WARP) takes segment u of pass blockIdx.y; it OWNS the segment's target if no earlier pass holds that target
// (binary searches in the earlier passes' sorted segment lists), and then adds the target's slices of this pass and of
// every later pass that holds it, in pass order and ascending slice order inside a pass - the order of the one-slice-at-a-time
// loop, whichever pass a slice falls into.  A target is written by exactly one group: no barrier between passes, no atomics.
struct RaggedPasses {
  float* const* src; float* const* trg; const size_t* len;
  const uint32_t* slice_sorted; const uint32_t* seg_start; const uint32_t* nseg;   // per pass p: at + p kSortMax, + p kSortMax + p, + p
  uint32_t n, npass;
};
// the segment of pass q whose target is t, or -1
__device__ __forceinline__ int find_target(const RaggedPasses& a, uint32_t q, const float* t) {
  const uint32_t base = q * kSortMax;
  const uint32_t* ss = a.slice_sorted + base;
  const uint32_t* st = a.seg_start + base + q;
  uint32_t lo = 0, hi = a.nseg[q];
  while (lo < hi) {
    const uint32_t mid = (lo + hi) >> 1;
    const float* tm = a.trg[base + ss[st[mid]]];
    if (tm < t) lo = mid + 1; else hi = mid;
  }
  return (lo < a.nseg[q] && a.trg[base + ss[st[lo]]] == t) ? (int)lo : -1;
}
template <bool WARP>
__global__ void __launch_bounds__(WARP ? 256 : kThreads) k_ragged_accumulate(const RaggedPasses a, const uint32_t* __restrict__ dup) {
  dyb_grid_dep_sync();
  if (*dup == 0) return;   // (distinct targets: k_ragged_accumulate_direct has done the work)
  const uint32_t p = blockIdx.y;
  const uint32_t U = a.nseg[p];
  const uint32_t group = WARP ? blockIdx.x * 8 + (threadIdx.x >> 5) : blockIdx.x, groups = WARP ? gridDim.x * 8 : gridDim.x;
  const uint32_t me = WARP ? (threadIdx.x & 31) : threadIdx.x, width = WARP ? 32 : kThreads;
  for (uint32_t u = group; u < U; u += groups) {
    const uint32_t base = p * kSortMax;
    float* t = a.trg[base + a.slice_sorted[base + a.seg_start[base + p + u]]];
    bool owner = true;
    for (uint32_t q = 0; q < p && owner; ++q) owner = find_target(a, q, t) < 0;
    if (!owner) continue;
    // the widest slice and the common alignment over all passes that hold the target
    size_t nmax = 0;
    bool al = aligned16(t);
    int seg_of[32];   // (at most 32 passes are looked at per round; longer lists go round by round below)
    for (uint32_t q0 = p; q0 < a.npass; q0 += 32) {
      const uint32_t q1 = min(a.npass, q0 + 32);
      nmax = 0;
      for (uint32_t q = q0; q < q1; ++q) {
        const int uq = q == p ? (int)u : find_target(a, q, t);
        seg_of[q - q0] = uq;
        if (uq < 0) continue;
        const uint32_t bq = q * kSortMax, k0 = a.seg_start[bq + q + uq], k1 = a.seg_start[bq + q + uq + 1];
        for (uint32_t k = k0; k < k1; ++k) {
          const uint32_t sidx = bq + a.slice_sorted[bq + k];
          nmax = max(nmax, a.len[sidx]);
          al = al && aligned16(a.src[sidx]) && (a.len[sidx] % 4 == 0);
        }
      }
      if (al) {
        for (size_t i = me; i < nmax / 4; i += width) {
          float4 acc = ld4(t + 4 * i);
          for (uint32_t q = q0; q < q1; ++q) {
            const int uq = seg_of[q - q0];
            if (uq < 0) continue;
            const uint32_t bq = q * kSortMax, k0 = a.seg_start[bq + q + uq], k1 = a.seg_start[bq + q + uq + 1];
            for (uint32_t k = k0; k < k1; ++k) {
              const uint32_t sidx = bq + a.slice_sorted[bq + k];
              if (4 * i < a.len[sidx]) {
                const float4 v = ld4_stream(a.src[sidx] + 4 * i);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
              }
            }
          }
          st4(t + 4 * i, acc);
        }
      } else {
        for (size_t i = me; i < nmax; i += width) {
          float acc = t[i];
          for (uint32_t q = q0; q < q1; ++q) {
            const int uq = seg_of[q - q0];
            if (uq < 0) continue;
            const uint32_t bq = q * kSortMax, k0 = a.seg_start[bq + q + uq], k1 = a.seg_start[bq + q + uq + 1];
            for (uint32_t k = k0; k < k1; ++k) {
              const uint32_t sidx = bq + a.slice_sorted[bq + k];
              if (i < a.len[sidx]) acc += a.src[sidx][i];
            }
          }
          t[i] = acc;
        }
      }
      if (WARP) __syncwarp(); else __syncthreads();   // (a later round re-reads what this one wrote)
    }
  }
}

}  // namespace

extern "C" {

int dyb200_parallel_memcpy(int num_seqs, int max_len, float** src, float** trg, size_t* len, dyb200_ctx* ctx) {
  DYB_CHECK_ARG(ctx, num_seqs >= 0, "parallel_memcpy: negative slice count");
  if (num_seqs == 0) return DYB200_OK;
  DYB_CHECK_ARG(ctx, src && trg && len, "parallel_memcpy: null table");
  // max_len (the longest slice, as the reference passes it, dynet/exec.cc:357) picks the work split
  if (max_len > 0 && max_len <= kWarpSliceMax)
    dyb_launch(k_ragged_copy_warp, stream_grid(ctx, (size_t)num_seqs, 8, 8), 256, 0, ctx, num_seqs, src, trg, len);
  else
    dyb_launch(k_ragged_copy, stream_grid(ctx, (size_t)num_seqs, 1, 16), kThreads, 0, ctx, num_seqs, src, trg, len);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_parallel_accumulate(int num_seqs, int max_len, float** src, float** trg, size_t* len, dyb200_ctx* ctx) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  DYB_CHECK_ARG(ctx, num_seqs >= 0, "parallel_accumulate: negative slice count");
  if (num_seqs == 0) return DYB200_OK;
  DYB_CHECK_ARG(ctx, src && trg && len, "parallel_accumulate: null table");
  const uint32_t n = (uint32_t)num_seqs, npass = (n + kSortMax - 1) / kSortMax;
  uint32_t cap = 1024;
  while (cap < 2 * n) cap <<= 1;
  // scratch: the address table + the flag (zeroed), then the sort tables of all passes
  const size_t table_bytes = (size_t)cap * sizeof(unsigned long long) + 256;
  void* scratch;
  int rc = dyb200_scratch(ctx, table_bytes + ((size_t)3 * n + 2 * npass + 8) * sizeof(uint32_t), &scratch);
  if (rc) return rc;
  unsigned long long* table = (unsigned long long*)scratch;
  uint32_t* dup = (uint32_t*)(table + cap);
  uint32_t* slice_sorted = (uint32_t*)((char*)scratch + table_bytes);
  uint32_t* group_sorted = slice_sorted + n;
  uint32_t* seg_start = group_sorted + n;          // n + npass entries: pass p starts at p kSortMax + p
  uint32_t* nseg = seg_start + n + npass;
  DYB_CUDA(ctx, cudaMemsetAsync(scratch, 0, table_bytes, ctx->stream));
  const bool warp = max_len > 0 && max_len <= kWarpSliceMax;
  dyb_launch(k_ragged_probe, stream_grid(ctx, n, 256), 256, 0, ctx, trg, n, table, cap - 1, dup);
  DYB_LAUNCHED(ctx);
  // distinct targets (the usual case): one pass, no order needed
  if (warp) dyb_launch(k_ragged_accumulate_direct<true>, stream_grid(ctx, n, 8, 8), 256, 0, ctx, num_seqs, src, trg, len, dup);
  else dyb_launch(k_ragged_accumulate_direct<false>, stream_grid(ctx, n, 1, 16), kThreads, 0, ctx, num_seqs, src, trg, len, dup);
  DYB_LAUNCHED(ctx);
  // shared targets: grouped by target, added in ascending slice order (these launches return at once otherwise)
  dyb_launch(k_sort_targets, npass, kSortThreads, 0, ctx, trg, n, slice_sorted, group_sorted, seg_start, nseg, dup);
  DYB_LAUNCHED(ctx);
  // one launch for all passes: blockIdx.y = pass
  RaggedPasses ra{src, trg, len, slice_sorted, seg_start, nseg, n, npass};
  const uint32_t np = n < (uint32_t)kSortMax ? n : (uint32_t)kSortMax;
  if (warp) dyb_launch(k_ragged_accumulate<true>, dim3(stream_grid(ctx, np, 8, 8), npass), 256, 0, ctx, ra, (const uint32_t*)dup);
  else dyb_launch(k_ragged_accumulate<false>, dim3(stream_grid(ctx, np, 1, 16), npass), kThreads, 0, ctx, ra, (const uint32_t*)dup);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

}  // extern "C"
