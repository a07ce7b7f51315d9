// Autobatch data movers: ragged gather (parallel_memcpy) and ragged scatter-add
// (parallel_accumulate).  The pointer/length tables live in device memory, exactly as
// BatchedExecutionEngine uploads them (dynet/exec.cc:346-356, :398-408).
//
// Copy: one CTA per slice, 128-bit loads/stores when both ends are 16-byte aligned.
// Accumulate: slices are grouped by target pointer (in-CTA sort, <= 4096 slices per pass); one
// CTA per distinct target adds that target's sources in ascending slice order, so slices that
// share a target are summed deterministically and without atomics.
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

// key = (target address / 4) << 18 | slice index (slice index < 2^18 within a pass)
__global__ void __launch_bounds__(kSortThreads) k_sort_targets(float* const* __restrict__ trg, uint32_t n, uint32_t base,
                                                              uint32_t* __restrict__ slice_sorted,
                                                              uint32_t* __restrict__ group_sorted,
                                                              uint32_t* __restrict__ seg_start, uint32_t* __restrict__ nseg) {
  dyb_grid_dep_sync();
  __shared__ unsigned long long keys[kSortMax];
  __shared__ uint32_t scan[kSortThreads];
  uint32_t npow = 1;
  while (npow < n) npow <<= 1;
  for (uint32_t k = threadIdx.x; k < npow; k += kSortThreads) {
    unsigned long long key = ~0ull;
    if (k < n) key = (((unsigned long long)(uintptr_t)trg[base + k] >> 2) << 18) | k;
    keys[k] = key;
  }
  __syncthreads();
  sort_and_segment(keys, scan, n, npow, 18, slice_sorted, group_sorted, seg_start, nseg);
}

__global__ void __launch_bounds__(kThreads) k_ragged_accumulate(float* const* __restrict__ src, float* const* __restrict__ trg,
                                                               const size_t* __restrict__ len, uint32_t base,
                                                               const uint32_t* __restrict__ slice_sorted,
                                                               const uint32_t* __restrict__ seg_start,
                                                               const uint32_t* __restrict__ nseg) {
  dyb_grid_dep_sync();
  const uint32_t U = *nseg;
  for (uint32_t u = blockIdx.x; u < U; u += gridDim.x) {
    const uint32_t k0 = seg_start[u], k1 = seg_start[u + 1];
    float* t = trg[base + slice_sorted[k0]];
    size_t nmax = 0;
    bool al = aligned16(t);
    for (uint32_t k = k0; k < k1; ++k) {
      uint32_t s = base + slice_sorted[k];
      nmax = max(nmax, len[s]);
      al = al && aligned16(src[s]) && (len[s] % 4 == 0);
    }
    if (al) {
      for (size_t i = threadIdx.x; i < nmax / 4; i += kThreads) {
        float4 acc = ld4(t + 4 * i);
        for (uint32_t k = k0; k < k1; ++k) {
          uint32_t s = base + slice_sorted[k];
          if (4 * i < len[s]) {
            float4 v = ld4_stream(src[s] + 4 * i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
        }
        st4(t + 4 * i, acc);
      }
    } else {
      for (size_t i = threadIdx.x; i < nmax; i += kThreads) {
        float acc = t[i];
        for (uint32_t k = k0; k < k1; ++k) {
          uint32_t s = base + slice_sorted[k];
          if (i < len[s]) acc += src[s][i];
        }
        t[i] = acc;
      }
    }
  }
}

}  // namespace

extern "C" {

int dyb200_parallel_memcpy(int num_seqs, int max_len, float** src, float** trg, size_t* len, dyb200_ctx* ctx) {
  (void)max_len;
  DYB_CHECK_ARG(ctx, num_seqs >= 0, "parallel_memcpy: negative slice count");
  if (num_seqs == 0) return DYB200_OK;
  DYB_CHECK_ARG(ctx, src && trg && len, "parallel_memcpy: null table");
  dyb_launch(k_ragged_copy, stream_grid(ctx, (size_t)num_seqs, 1, 16), kThreads, 0, ctx, num_seqs, src, trg, len);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_parallel_accumulate(int num_seqs, int max_len, float** src, float** trg, size_t* len, dyb200_ctx* ctx) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)max_len;
  DYB_CHECK_ARG(ctx, num_seqs >= 0, "parallel_accumulate: negative slice count");
  if (num_seqs == 0) return DYB200_OK;
  DYB_CHECK_ARG(ctx, src && trg && len, "parallel_accumulate: null table");
  uint32_t np = (uint32_t)num_seqs < (uint32_t)kSortMax ? (uint32_t)num_seqs : (uint32_t)kSortMax;
  void* scratch;
  int rc = dyb200_scratch(ctx, ((size_t)3 * np + 8) * sizeof(uint32_t), &scratch);
  if (rc) return rc;
  for (uint32_t base = 0; base < (uint32_t)num_seqs; base += kSortMax) {
    uint32_t n = (uint32_t)num_seqs - base < (uint32_t)kSortMax ? (uint32_t)num_seqs - base : (uint32_t)kSortMax;
    uint32_t* slice_sorted = (uint32_t*)scratch;
    uint32_t* group_sorted = slice_sorted + n;
    uint32_t* seg_start = group_sorted + n;
    uint32_t* nseg = seg_start + n + 1;
    dyb_launch(k_sort_targets, 1, kSortThreads, 0, ctx, trg, n, base, slice_sorted, group_sorted, seg_start, nseg);
    DYB_LAUNCHED(ctx);
    dyb_launch(k_ragged_accumulate, stream_grid(ctx, n, 1, 16), kThreads, 0, ctx, src, trg, len, base, slice_sorted, seg_start, nseg);
    DYB_LAUNCHED(ctx);
  }
  return DYB200_OK;
}

}  // extern "C"
