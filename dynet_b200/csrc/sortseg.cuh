// In-CTA bitonic sort of up to 4096 64-bit keys followed by segmentation into runs of equal
// "group" (key >> shift).  Used by the embedding scatter-add (group = id) and by the ragged
// accumulate (group = target pointer).  Deterministic: keys are unique, so the sorted order
// is fully defined by the input.
#pragma once
#include "common.cuh"

constexpr int kSortMax = 4096;
constexpr int kSortThreads = 1024;

// keys[0..npow) hold the n keys followed by ~0 padding; must be called by all kSortThreads
// threads.  Outputs: payload_sorted[k] = low `shift` bits of the k-th key (truncated to 32 bits),
// group_sorted[u] = low 32 bits of the group of segment u, seg_start[0..U] (seg_start[U] = n), *nseg = U.
__device__ __forceinline__ void bitonic_sort_keys(unsigned long long* keys, uint32_t npow) {
  for (uint32_t size = 2; size <= npow; size <<= 1) {
    for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
      for (uint32_t t = threadIdx.x; t < npow / 2; t += kSortThreads) {
        uint32_t lo = 2 * t - (t & (stride - 1));
        uint32_t hi = lo + stride;
        bool up = (lo & size) == 0;
        unsigned long long a = keys[lo], b = keys[hi];
        if ((a > b) == up) { keys[lo] = b; keys[hi] = a; }
      }
      __syncthreads();
    }
  }
}

__device__ __forceinline__ void sort_and_segment(unsigned long long* keys, uint32_t* scan, uint32_t n, uint32_t npow,
                                                 int shift, uint32_t* __restrict__ payload_sorted,
                                                 uint32_t* __restrict__ group_sorted, uint32_t* __restrict__ seg_start,
                                                 uint32_t* __restrict__ nseg) {
  for (uint32_t size = 2; size <= npow; size <<= 1) {
    for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
      for (uint32_t t = threadIdx.x; t < npow / 2; t += kSortThreads) {
        uint32_t lo = 2 * t - (t & (stride - 1));
        uint32_t hi = lo + stride;
        bool up = (lo & size) == 0;
        unsigned long long a = keys[lo], b = keys[hi];
        if ((a > b) == up) { keys[lo] = b; keys[hi] = a; }
      }
      __syncthreads();
    }
  }
  const unsigned long long pmask = shift >= 64 ? ~0ull : ((1ull << shift) - 1ull);
  // segment heads: each thread owns a contiguous run of `per` sorted entries
  const uint32_t per = (n + kSortThreads - 1) / kSortThreads;
  const uint32_t k0 = min(n, threadIdx.x * per), k1 = min(n, k0 + per);
  uint32_t cnt = 0;
  for (uint32_t k = k0; k < k1; ++k) cnt += (k == 0 || (keys[k] >> shift) != (keys[k - 1] >> shift));
  scan[threadIdx.x] = cnt;
  __syncthreads();
  for (uint32_t off = 1; off < kSortThreads; off <<= 1) {  // inclusive Hillis-Steele scan
    uint32_t v = threadIdx.x >= off ? scan[threadIdx.x - off] : 0;
    __syncthreads();
    scan[threadIdx.x] += v;
    __syncthreads();
  }
  uint32_t seg = scan[threadIdx.x] - cnt;
  for (uint32_t k = k0; k < k1; ++k) {
    unsigned long long grp = keys[k] >> shift;
    payload_sorted[k] = (uint32_t)(keys[k] & pmask);
    if (k == 0 || grp != (keys[k - 1] >> shift)) { seg_start[seg] = k; group_sorted[seg] = (uint32_t)grp; ++seg; }
  }
  if (threadIdx.x == kSortThreads - 1) { *nseg = scan[threadIdx.x]; seg_start[scan[threadIdx.x]] = n; }
}
