// LookupNode forward (embedding row gather) and LookupParameterStorage::accumulate_grads
// (deterministic scatter-add).
//
// Gather: one warp per looked-up row; the row is staged through shared memory by the
// bulk-copy (TMA) engine -- cp.async.bulk global->shared completing on an mbarrier, then
// cp.async.bulk shared->global -- with two buffers per warp so the next row's load overlaps
// the current row's store.  No multicast is used anywhere.  Rows that are not 16-byte
// multiples fall back to plain loads.
//
// Scatter-add: (id, position) pairs are sorted by id inside one CTA (bitonic, <= 4096 pairs
// per pass).  The sorted list is cut into chunks of 32 positions; one warp per (chunk, 128-float
// column slice) adds the rows of each id in ascending position -- the order of the reference's CPU
// loop (dynet/model.cc:735-741) -- straight into the table row when the id's run lies inside the
// chunk, or into a per-chunk partial when a frequent id (Zipf head) spans chunks; a second pass
// adds those partials in chunk order.  No atomics, a fixed summation tree, balanced work.
#include <stdlib.h>

#include "common.cuh"
#include "sortseg.cuh"

namespace {

constexpr int kGatherWarps = 8;
constexpr int kGatherRowBytesMax = 4096;  // per buffer; 2 buffers per warp
constexpr uint32_t kWaitLimit = 1u << 22; // bounded mbarrier wait (iterations)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Returns false if the wait ran out (the caller sets the error flag and stops).
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
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Wait until at most `N` bulk stores of this thread still READ their shared source.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- gather, bulk-copy staged -----------------------------------------------------------
__global__ void __launch_bounds__(kGatherWarps * 32) k_gather_bulk(const float* __restrict__ table,
                                                                  const uint32_t* __restrict__ ids, uint32_t n,
                                                                  uint32_t E, uint32_t vocab, float scale,
                                                                  float* __restrict__ out, uint32_t* flags) {
  dyb_grid_dep_sync();
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t bars[kGatherWarps][2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row_bytes = E * 4u;
  unsigned char* buf0 = smem + (size_t)warp * 2 * row_bytes;
  unsigned char* buf[2] = {buf0, buf0 + row_bytes};
  if (lane == 0) { mbar_init(&bars[warp][0], 1); mbar_init(&bars[warp][1], 1); }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  const uint32_t nwarps = gridDim.x * kGatherWarps;
  uint32_t first = blockIdx.x * kGatherWarps + warp;
  uint32_t phase[2] = {0, 0};
  bool ok = true;
  // prologue: issue the first load
  auto issue = [&](uint32_t b, int s) {
    if (lane == 0) {
      uint32_t id = ids[b];
      if (id >= vocab) { atomicOr(flags, DYB200_FLAG_BAD_INDEX); id = vocab - 1; }
      mbar_expect_tx(&bars[warp][s], row_bytes);
      bulk_g2s(buf[s], table + (size_t)id * E, row_bytes, &bars[warp][s]);
    }
  };
  int s = 0;
  if (first < n) issue(first, 0);
  for (uint32_t b = first; b < n && ok; b += nwarps, s ^= 1) {
    uint32_t nb = b + nwarps;
    if (nb < n) {
      // buffer s^1 was the source of the store issued one iteration ago
      if (lane == 0) bulk_wait_read<0>();
      __syncwarp();
      issue(nb, s ^ 1);
    }
    ok = mbar_wait(&bars[warp][s], phase[s]);
    phase[s] ^= 1;
    if (!ok) { if (lane == 0) atomicOr(flags, DYB200_FLAG_WAIT_TIMEOUT); break; }
    float* dst = out + (size_t)b * E;
    if (scale == 1.0f) {
      if (lane == 0) bulk_s2g(dst, buf[s], row_bytes);
    } else {
      const float4* src4 = reinterpret_cast<const float4*>(buf[s]);
      for (uint32_t i = lane; i < E / 4; i += 32) {
        float4 v = src4[i];
        st4_stream(dst + 4 * i, make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale));
      }
      __syncwarp();
    }
  }
  if (lane == 0) bulk_wait_all();  // shared memory must outlive the stores that read it
}

// ---- gather, plain loads (rows that are not 16-byte multiples, or very long rows) ---------
__global__ void __launch_bounds__(256) k_gather_plain(const float* __restrict__ table, const uint32_t* __restrict__ ids,
                                                     uint32_t n, uint32_t E, uint32_t vocab, float scale,
                                                     float* __restrict__ out, uint32_t* flags, int vec) {
  dyb_grid_dep_sync();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t nwarps = gridDim.x * 8;
  for (uint32_t b = blockIdx.x * 8 + warp; b < n; b += nwarps) {
    uint32_t id = ids[b];
    if (id >= vocab) { if (lane == 0) atomicOr(flags, DYB200_FLAG_BAD_INDEX); id = vocab - 1; }
    const float* src = table + (size_t)id * E;
    float* dst = out + (size_t)b * E;
    if (vec) {
      for (uint32_t i = lane; i < E / 4; i += 32) {
        float4 v = ld4(src + 4 * i);
        st4_stream(dst + 4 * i, make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale));
      }
    } else {
      for (uint32_t i = lane; i < E; i += 32) dst[i] = src[i] * scale;
    }
  }
}

// ---- scatter-add: sort + segment + reduce ---------------------------------------------------
// key = id << 32 | position: sorting groups equal ids and keeps positions ascending inside a group.
__global__ void __launch_bounds__(kSortThreads) k_sort_segments(const uint32_t* __restrict__ ids, uint32_t n,
                                                               uint32_t base, uint32_t vocab,
                                                               uint32_t* __restrict__ pos_sorted,
                                                               uint32_t* __restrict__ id_sorted,
                                                               uint32_t* __restrict__ seg_start,
                                                               uint32_t* __restrict__ nseg, uint32_t* flags) {
  dyb_grid_dep_sync();
  __shared__ unsigned long long keys[kSortMax];
  __shared__ uint32_t scan[kSortThreads];
  uint32_t npow = 1;
  while (npow < n) npow <<= 1;
  for (uint32_t k = threadIdx.x; k < npow; k += kSortThreads) {
    unsigned long long key = ~0ull;  // padding sorts last
    if (k < n) {
      uint32_t id = ids[base + k];
      if (id >= vocab) { atomicOr(flags, DYB200_FLAG_BAD_INDEX); id = vocab - 1; }
      key = ((unsigned long long)id << 32) | (base + k);
    }
    keys[k] = key;
  }
  __syncthreads();
  sort_and_segment(keys, scan, n, npow, 32, pos_sorted, id_sorted, seg_start, nseg);
}

// One warp per (segment, slice of 128 floats): row = table row; row += g[pos] for the segment's
// positions in ascending order; write the row back.  Loads of up to 4 source rows are issued
// ahead of the dependent adds.
__global__ void __launch_bounds__(256) k_segment_add(const float* __restrict__ g, float* __restrict__ all_grads,
                                                    uint32_t E, const uint32_t* __restrict__ pos_sorted,
                                                    const uint32_t* __restrict__ id_sorted,
                                                    const uint32_t* __restrict__ seg_start,
                                                    const uint32_t* __restrict__ nseg, uint32_t slices, int vec) {
  dyb_grid_dep_sync();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t U = *nseg;
  const size_t work = (size_t)U * slices;
  for (size_t w = (size_t)blockIdx.x * 8 + warp; w < work; w += (size_t)gridDim.x * 8) {
    const uint32_t u = (uint32_t)(w / slices), sl = (uint32_t)(w % slices);
    const uint32_t k0 = seg_start[u], k1 = seg_start[u + 1];
    float* row = all_grads + (size_t)id_sorted[u] * E;
    if (vec) {
      const uint32_t col = sl * 128 + lane * 4;
      if (col >= E) continue;
      float4 acc = ld4(row + col);
      uint32_t k = k0;
      for (; k + 4 <= k1; k += 4) {
        float4 v0 = ld4_stream(g + (size_t)pos_sorted[k] * E + col), v1 = ld4_stream(g + (size_t)pos_sorted[k + 1] * E + col);
        float4 v2 = ld4_stream(g + (size_t)pos_sorted[k + 2] * E + col), v3 = ld4_stream(g + (size_t)pos_sorted[k + 3] * E + col);
        acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
        acc.x += v1.x; acc.y += v1.y; acc.z += v1.z; acc.w += v1.w;
        acc.x += v2.x; acc.y += v2.y; acc.z += v2.z; acc.w += v2.w;
        acc.x += v3.x; acc.y += v3.y; acc.z += v3.z; acc.w += v3.w;
      }
      for (; k < k1; ++k) {
        float4 v = ld4_stream(g + (size_t)pos_sorted[k] * E + col);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      st4(row + col, acc);
    } else {
      for (uint32_t col = sl * 128 + lane; col < min(E, (sl + 1) * 128); col += 32) {
        float acc = row[col];
        for (uint32_t k = k0; k < k1; ++k) acc += g[(size_t)pos_sorted[k] * E + col];
        row[col] = acc;
      }
    }
  }
}


// ---- scatter-add, chunked (load-balanced) variant ------------------------------------------------
constexpr uint32_t kChunk = 32;

// CTA p sorts the ids of pass p (positions [p kSortMax, ...)): the passes of a long id list are sorted side by side in one launch.
__global__ void __launch_bounds__(kSortThreads) k_sort_ids(const uint32_t* __restrict__ ids, uint32_t n_total,
                                                          uint32_t vocab, uint32_t* __restrict__ pos_sorted,
                                                          uint32_t* __restrict__ id_at, uint32_t* flags) {
  dyb_grid_dep_sync();
  __shared__ unsigned long long keys[kSortMax];
  const uint32_t base = blockIdx.x * kSortMax;
  const uint32_t n = min((uint32_t)kSortMax, n_total - base);
  uint32_t npow = 1;
  while (npow < n) npow <<= 1;
  for (uint32_t k = threadIdx.x; k < npow; k += kSortThreads) {
    unsigned long long key = ~0ull;
    if (k < n) {
      uint32_t id = ids[base + k];
      if (id >= vocab) { atomicOr(flags, DYB200_FLAG_BAD_INDEX); id = vocab - 1; }
      key = ((unsigned long long)id << 32) | (base + k);
    }
    keys[k] = key;
  }
  __syncthreads();
  bitonic_sort_keys(keys, npow);
  for (uint32_t k = threadIdx.x; k < n; k += kSortThreads) {
    pos_sorted[base + k] = (uint32_t)keys[k];
    id_at[base + k] = (uint32_t)(keys[k] >> 32);
  }
}

// Merges the sorted runs of k_sort_ids (run p = positions [p kSortMax, ...), sorted by (id, position)) into one sorted list:
// one thread per element, whose place is the number of smaller keys in every run.  Positions grow with the run number, so
// among equal ids the earlier run comes first: runs before the element's own count their ids <= id, later runs their ids < id.
__global__ void __launch_bounds__(256) k_merge_runs(const uint32_t* __restrict__ pos_run, const uint32_t* __restrict__ id_run,
                                                   uint32_t n, uint32_t* __restrict__ pos_out, uint32_t* __restrict__ id_out) {
  dyb_grid_dep_sync();
  const uint32_t e = blockIdx.x * 256 + threadIdx.x;
  if (e >= n) return;
  const uint32_t p = e / kSortMax, id = id_run[e];
  const uint32_t npass = (n + kSortMax - 1) / kSortMax;
  uint32_t rank = e - p * kSortMax;
  for (uint32_t q = 0; q < npass; ++q) {
    if (q == p) continue;
    const uint32_t* run = id_run + (size_t)q * kSortMax;
    uint32_t lo = 0, hi = min((uint32_t)kSortMax, n - q * kSortMax);
    const uint32_t bound = q < p ? id + 1 : id;   // count ids < bound  (id + 1 does not wrap: ids are below the vocabulary size)
    while (lo < hi) {
      const uint32_t mid = (lo + hi) >> 1;
      if (run[mid] < bound) lo = mid + 1; else hi = mid;
    }
    rank += lo;
  }
  pos_out[rank] = pos_run[e];
  id_out[rank] = id;
}

__device__ __forceinline__ void add4(float4& a, const float4& b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }

// Pass A: one warp per (chunk, slice).  A run that starts in the chunk begins from the table row
// (so a run that also ends here reproduces the sequential CPU sum exactly); a run that started in an
// earlier chunk begins from zero and goes to head[chunk]; a run that continues goes to tail[chunk].
__global__ void __launch_bounds__(256) k_chunk_add(const float* __restrict__ g, float* __restrict__ all_grads, uint32_t E,
                                                  const uint32_t* __restrict__ pos_sorted, const uint32_t* __restrict__ id_at,
                                                  uint32_t n, uint32_t slices, float* __restrict__ head, float* __restrict__ tail) {
  dyb_grid_dep_sync();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t nchunks = (n + kChunk - 1) / kChunk;
  const size_t work = (size_t)nchunks * slices;
  for (size_t w = (size_t)blockIdx.x * 8 + warp; w < work; w += (size_t)gridDim.x * 8) {
    const uint32_t c = (uint32_t)(w / slices), sl = (uint32_t)(w % slices);
    const uint32_t k0 = c * kChunk, k1 = min(n, k0 + kChunk);
    const uint32_t col = sl * 128 + lane * 4;
    const bool live = col < E;   // lanes past the row end still take part in the shuffles
    const uint32_t my_id = k0 + lane < k1 ? id_at[k0 + lane] : 0xffffffffu;
    const uint32_t my_pos = k0 + lane < k1 ? pos_sorted[k0 + lane] : 0;
    uint32_t cur = __shfl_sync(0xffffffffu, my_id, 0);
    bool started_before = k0 > 0 && id_at[k0 - 1] == cur;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 acc = (started_before || !live) ? zero4 : ld4(all_grads + (size_t)cur * E + col);
    float* hslot = head + ((size_t)c * slices + sl) * 128 + lane * 4;
    float* tslot = tail + ((size_t)c * slices + sl) * 128 + lane * 4;
    for (uint32_t j0 = 0; j0 < k1 - k0; j0 += 8) {
      // the gradient rows of the next 8 positions are requested together; the adds stay in order
      float4 rows[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint32_t pos = __shfl_sync(0xffffffffu, my_pos, (j0 + u) & 31);
        rows[u] = (live && j0 + u < k1 - k0) ? ld4_stream(g + (size_t)pos * E + col) : zero4;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint32_t id = __shfl_sync(0xffffffffu, my_id, (j0 + u) & 31);
        if (j0 + u < k1 - k0) {
          if (id != cur) {   // the run of `cur` ends inside this chunk
            if (live) {
              if (started_before) st4(hslot, acc);
              else st4(all_grads + (size_t)cur * E + col, acc);
            }
            cur = id;
            started_before = false;
            acc = live ? ld4(all_grads + (size_t)cur * E + col) : zero4;
          }
          add4(acc, rows[u]);
        }
      }
    }
    const bool continues = k1 < n && id_at[k1] == cur;
    if (live) {
      if (started_before) st4(hslot, acc);                           // middle or last piece
      else if (continues) st4(tslot, acc);                           // first piece (holds the row)
      else st4(all_grads + (size_t)cur * E + col, acc);              // whole run
    }
  }
}
// Pass B: the chunk in which a multi-chunk run starts adds the later pieces in chunk order and writes the row.
__global__ void __launch_bounds__(256) k_chunk_combine(float* __restrict__ all_grads, uint32_t E, const uint32_t* __restrict__ id_at,
                                                      uint32_t n, uint32_t slices, const float* __restrict__ head,
                                                      const float* __restrict__ tail) {
  dyb_grid_dep_sync();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t nchunks = (n + kChunk - 1) / kChunk;
  const size_t work = (size_t)nchunks * slices;
  for (size_t w = (size_t)blockIdx.x * 8 + warp; w < work; w += (size_t)gridDim.x * 8) {
    const uint32_t c = (uint32_t)(w / slices), sl = (uint32_t)(w % slices);
    const uint32_t k0 = c * kChunk, k1 = min(n, k0 + kChunk);
    const uint32_t col = sl * 128 + lane * 4;
    if (col >= E || k1 >= n) continue;
    const uint32_t id = id_at[k1 - 1];
    if (id_at[k1] != id) continue;                         // last run of the chunk does not continue
    if (id_at[k0] == id && k0 > 0 && id_at[k0 - 1] == id) continue;   // it started earlier: not the owner
    float4 acc = ld4(tail + ((size_t)c * slices + sl) * 128 + lane * 4);
    // A frequent id runs over hundreds of chunks (the most frequent word of a 107 k-token batch: ~500).  The last chunk of
    // the run is found by a binary search over the chunk heads (ids are sorted), then sixteen pieces are requested at a
    // time; the adds stay in chunk order.
    uint32_t lo = c + 1, hi = nchunks;   // first chunk in [lo, hi) whose head is another id
    while (lo < hi) {
      const uint32_t mid = (lo + hi) >> 1;
      if (id_at[mid * kChunk] == id) lo = mid + 1; else hi = mid;
    }
    const uint32_t c_end = lo;
    for (uint32_t c2 = c + 1; c2 < c_end; c2 += 16) {
      float4 piece[16];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        if (c2 + u < c_end) piece[u] = ld4(head + ((size_t)(c2 + u) * slices + sl) * 128 + lane * 4);
#pragma unroll
      for (int u = 0; u < 16; ++u)
        if (c2 + u < c_end) add4(acc, piece[u]);
    }
    st4(all_grads + (size_t)id * E + col, acc);
  }
}

}  // namespace

// Load-balanced path (rows that are multiples of 4 floats).  Up to kMergeMaxIds ids the sorted runs of the passes are merged
// into one sorted list and added in ONE pair of launches; scratch then holds pos / id of the runs and of the merged list and
// two partial buffers of nchunks * slices * 128 floats for all n ids.  Longer lists go pass after pass (scratch: the runs and
// the partial buffers of one pass).
constexpr uint32_t kMergeMaxIds = 1u << 18;
static size_t chunked_scratch_bytes(uint32_t n, uint32_t E) {
  const bool merged = n > (uint32_t)kSortMax && n <= kMergeMaxIds;
  const uint32_t np = (n < (uint32_t)kSortMax || merged) ? n : (uint32_t)kSortMax;
  uint32_t nchunks = (np + kChunk - 1) / kChunk, slices = (E + 127) / 128;
  return ((size_t)(merged ? 4 : 2) * n * sizeof(uint32_t) + 512) + (size_t)2 * nchunks * slices * 128 * sizeof(float) + 512;
}
static int scatter_run_chunked(dyb200_ctx* ctx, unsigned n, const unsigned* ids_dev, const float* g, float* all_grads,
                               unsigned E, unsigned vocab, void* scratch) {
  const uint32_t slices = (E + 127) / 128;
  const uint32_t npass = (n + kSortMax - 1) / kSortMax;
  const bool merged = npass > 1 && n <= kMergeMaxIds;
  uint32_t* pos_all = (uint32_t*)scratch;
  uint32_t* id_all = pos_all + n;
  uint32_t* pos_m = id_all + n;                      // (merged only)
  uint32_t* id_m = pos_m + n;
  const uint32_t np_max = (n < (uint32_t)kSortMax || merged) ? n : (uint32_t)kSortMax;
  float* head = (float*)(((uintptr_t)(id_all + (merged ? 3 : 1) * (size_t)n) + 255) & ~(uintptr_t)255);
  float* tail = head + (size_t)((np_max + kChunk - 1) / kChunk) * slices * 128;
  // every pass's ids are sorted in the same launch (one CTA each)
  dyb_launch(k_sort_ids, npass, kSortThreads, 0, ctx, ids_dev, n, vocab, pos_all, id_all, ctx->dev_flags);
  DYB_LAUNCHED(ctx);
  if (merged) {
    dyb_launch(k_merge_runs, (n + 255) / 256, 256, 0, ctx, (const uint32_t*)pos_all, (const uint32_t*)id_all, n, pos_m, id_m);
    DYB_LAUNCHED(ctx);
    const size_t work = (size_t)((n + kChunk - 1) / kChunk) * slices;
    dyb_launch(k_chunk_add, stream_grid(ctx, work, 8), 256, 0, ctx, g, all_grads, E, pos_m, id_m, n, slices, head, tail);
    DYB_LAUNCHED(ctx);
    dyb_launch(k_chunk_combine, stream_grid(ctx, work, 8), 256, 0, ctx, all_grads, E, id_m, n, slices, head, tail);
    DYB_LAUNCHED(ctx);
    return DYB200_OK;
  }
  // the adds run pass after pass, so that a table row that several passes touch receives their sums in pass order
  for (uint32_t base = 0; base < n; base += kSortMax) {
    uint32_t np = n - base < (uint32_t)kSortMax ? n - base : (uint32_t)kSortMax;
    uint32_t nchunks = (np + kChunk - 1) / kChunk;
    uint32_t* pos_sorted = pos_all + base;
    uint32_t* id_at = id_all + base;
    size_t work = (size_t)nchunks * slices;
    dyb_launch(k_chunk_add, stream_grid(ctx, work, 8), 256, 0, ctx, g, all_grads, E, pos_sorted, id_at, np, slices, head, tail);
    DYB_LAUNCHED(ctx);
    dyb_launch(k_chunk_combine, stream_grid(ctx, work, 8), 256, 0, ctx, all_grads, E, id_at, np, slices, head, tail);
    DYB_LAUNCHED(ctx);
  }
  return DYB200_OK;
}

// Runs the sort + segmented-add passes using `scratch`, which must hold at least
// dyb200_lookup_scatter_scratch_bytes(min(n, kSortMax)) bytes.
size_t dyb200_lookup_scatter_scratch_bytes(uint32_t n_pass) { return ((size_t)3 * n_pass + 8) * sizeof(uint32_t); }

int dyb200_lookup_scatter_run(dyb200_ctx* ctx, unsigned n, const unsigned* ids_dev, const float* g, float* all_grads,
                              unsigned E, unsigned vocab, void* scratch) {
  const int vec = (E % 4 == 0) && aligned16(g) && aligned16(all_grads);
  const uint32_t slices = (E + 127) / 128;
  for (uint32_t base = 0; base < n; base += kSortMax) {
    uint32_t np = n - base < (uint32_t)kSortMax ? n - base : (uint32_t)kSortMax;
    uint32_t* pos_sorted = (uint32_t*)scratch;
    uint32_t* id_sorted = pos_sorted + np;
    uint32_t* seg_start = id_sorted + np;       // np + 1 entries
    uint32_t* nseg = seg_start + np + 1;
    dyb_launch(k_sort_segments, 1, kSortThreads, 0, ctx, ids_dev, np, base, vocab, pos_sorted, id_sorted, seg_start, nseg, ctx->dev_flags);
    DYB_LAUNCHED(ctx);
    size_t work = (size_t)np * slices;  // upper bound: every position its own segment
    dyb_launch(k_segment_add, stream_grid(ctx, work, 8), 256, 0, ctx, g, all_grads, E, pos_sorted, id_sorted, seg_start, nseg, slices, vec);
    DYB_LAUNCHED(ctx);
  }
  return DYB200_OK;
}

// ---- scatter-add for callers that cannot allocate ---------------------------------------------
// Some hosts of this library may not call cudaMalloc at all: a training loop whose device memory
// is one pool carved up at start-up (DyNet's own model: four fixed pools per device and
// EIGEN_NO_MALLOC in the CUDA build), or code running inside a region where an allocation would
// be an error.  For them the sort/segment tables of the scatter-add live in this fixed array
// instead of the context's growable arena.  It is part of the library image: every GPU that loads
// the library holds these 49,408 bytes until the process exits.
constexpr unsigned kNoAllocMaxIds = DYB200_NOALLOC_MAX_IDS;   // one sort pass
constexpr size_t kNoAllocBytes = ((((size_t)3 * kNoAllocMaxIds + 8) * sizeof(uint32_t)) + 255) & ~(size_t)255;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];
// The array's name is only a host-side handle; kernels need its device address, looked up once
// per device with that device current.
constexpr int kMaxDevices = 64;
static void* g_noalloc_addr[kMaxDevices] = {};

extern "C" {

int dyb200_lookup_accumulate_grads_noalloc(unsigned n, const unsigned* ids_host, const unsigned* ids_dev,
                                           const float* g, float* all_grads, unsigned dim_size, unsigned vocab,
                                           dyb200_ctx* ctx) {
  DYB_CHECK_ARG(ctx, ids_dev != nullptr && g != nullptr && all_grads != nullptr, "accumulate_grads_noalloc: null pointer");
  DYB_CHECK_ARG(ctx, n <= kNoAllocMaxIds,
                "accumulate_grads_noalloc: %u ids exceed the fixed scratch (DYB200_NOALLOC_MAX_IDS = %u per call); "
                "split the call or use dyb200_lookup_accumulate_grads", n, kNoAllocMaxIds);
  if (ids_host)
    for (unsigned b = 0; b < n; ++b)
      DYB_CHECK_ARG(ctx, ids_host[b] < vocab, "Out-of-bounds attempt to access index %u for LookupParameter of size %u", ids_host[b], vocab);
  DYB_CHECK_ARG(ctx, ctx->device >= 0 && ctx->device < kMaxDevices, "accumulate_grads_noalloc: device id %d not supported", ctx->device);
  if (n == 0 || dim_size == 0) return DYB200_OK;
  // The array exists once per device and its address belongs to the device that is current when it is looked up; the
  // kernels below run on the context's stream.  Both must be the same device, on every call: with another device current
  // the launches would go there carrying a pointer into this device's copy.  The caller's current device is not changed.
  int cur = -1;
  DYB_CUDA(ctx, cudaGetDevice(&cur));
  DYB_CHECK_ARG(ctx, cur == ctx->device, "accumulate_grads_noalloc: the current device is %d, the context belongs to device %d "
                "(make it current with cudaSetDevice before the call)", cur, ctx->device);
  if (g_noalloc_addr[ctx->device] == nullptr) {   // first call on this device: one-time set-up
    // (looking the symbol up may initialise the module on this device, which is not allowed while a capture is open)
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    DYB_CUDA(ctx, cudaStreamIsCapturing(ctx->stream, &cap));
    if (cap != cudaStreamCaptureStatusNone)
      return dyb200_fail(ctx, DYB200_ERUNTIME, "accumulate_grads_noalloc: the first call on a device does a one-time set-up and "
                                              "must come before any stream capture");
    void* addr = nullptr;
    DYB_CUDA(ctx, cudaGetSymbolAddress(&addr, g_noalloc_scratch));
    g_noalloc_addr[ctx->device] = addr;
  }
  // Every table entry the kernels read is written by the sort kernel of the same call, so nothing
  // left over from an earlier call needs clearing.
  return dyb200_lookup_scatter_run(ctx, n, ids_dev, g, all_grads, dim_size, vocab, g_noalloc_addr[ctx->device]);
}

int dyb200_lookup_fwd(DYB200_FWD_ARGS) {
  DYB_CHECK_ARG(ctx, nxs == 0 && xs == nullptr, "Failed dimension check in LookupNode::forward (no inputs expected)");
  DYB_CHECK_ARG(ctx, attrs != nullptr && aux_mem != nullptr, "LookupNode: attrs and aux_mem (bd uint32) required");
  const dyb200_lookup_attrs* a = (const dyb200_lookup_attrs*)attrs;
  const uint32_t n = a->n, E = (uint32_t)t_batch_size(fx);
  DYB_CHECK_ARG(ctx, fx->bd == n, "In LookupNode, in index vector size (%u) doesn't match batch size in expressions (%u)", n, fx->bd);
  if (n == 0 || E == 0) return DYB200_OK;
  uint32_t* ids_dev = (uint32_t*)aux_mem;
  if (a->ids_host) {
    for (uint32_t b = 0; b < n; ++b)
      DYB_CHECK_ARG(ctx, a->ids_host[b] < a->vocab, "Out-of-bounds attempt to access index %u for LookupParameter of size %u", a->ids_host[b], a->vocab);
    DYB_CUDA(ctx, cudaMemcpyAsync(ids_dev, a->ids_host, n * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream));
  }  // else: aux_mem already holds the ids on the device; the kernel clamps and flags a bad id
  const bool al = aligned16(a->all_values) && aligned16(fx->v) && E % 4 == 0;
  if (al && E * 4u <= (uint32_t)kGatherRowBytesMax) {
    size_t smem = (size_t)kGatherWarps * 2 * E * 4;
    if (!(ctx->func_attr_done & 8u)) {   // (per device: remembered by the context)
      DYB_CUDA(ctx, cudaFuncSetAttribute(k_gather_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, kGatherWarps * 2 * kGatherRowBytesMax));
      ctx->func_attr_done |= 8u;
    }
    unsigned grid = stream_grid(ctx, n, kGatherWarps, 3);
    dyb_launch(k_gather_bulk, grid, kGatherWarps * 32, smem, ctx, a->all_values, ids_dev, n, E, a->vocab, a->weight_decay_scale, fx->v, ctx->dev_flags);
  } else {
    dyb_launch(k_gather_plain, stream_grid(ctx, n, 8), 256, 0, ctx, a->all_values, ids_dev, n, E, a->vocab, a->weight_decay_scale, fx->v, ctx->dev_flags, al ? 1 : 0);
  }
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_lookup_accumulate_grads(unsigned n, const unsigned* ids_host, const unsigned* ids_dev, const float* g,
                                   float* all_grads, unsigned dim_size, unsigned vocab, dyb200_ctx* ctx) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  DYB_CHECK_ARG(ctx, ids_dev != nullptr && g != nullptr && all_grads != nullptr, "accumulate_grads: null pointer");
  if (ids_host)
    for (unsigned b = 0; b < n; ++b)
      DYB_CHECK_ARG(ctx, ids_host[b] < vocab, "Out-of-bounds attempt to access index %u for LookupParameter of size %u", ids_host[b], vocab);
  if (n == 0 || dim_size == 0) return DYB200_OK;
  uint32_t np = n < (unsigned)kSortMax ? n : (unsigned)kSortMax;
  void* scratch;
  if (dim_size % 4 == 0 && aligned16(g) && aligned16(all_grads)) {
    int rc = dyb200_scratch(ctx, chunked_scratch_bytes(n, dim_size), &scratch);
    if (rc) return rc;
    return scatter_run_chunked(ctx, n, ids_dev, g, all_grads, dim_size, vocab, scratch);
  }
  int rc = dyb200_scratch(ctx, dyb200_lookup_scatter_scratch_bytes(np), &scratch);
  if (rc) return rc;
  return dyb200_lookup_scatter_run(ctx, n, ids_dev, g, all_grads, dim_size, vocab, scratch);
}

}  // extern "C"
