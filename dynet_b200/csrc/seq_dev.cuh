// Device helpers of the sequence-persistent LSTM kernels (lstm_seq.cu, lstm_seq_bwd.cu): bounded polling of hand-over
// counters in global memory, cluster-scope mbarrier operations, named-barrier reductions.
#pragma once
#include "tc_dev.cuh"

namespace {

constexpr uint32_t kPollLimit = 1u << 22;      // polls of a global counter before a CTA gives up (~ seconds)
constexpr uint32_t kSeqBufs = 4;               // TMEM accumulators (4 x 128 columns)
constexpr int SMEM_SEQ_BYTES = SMEM_BYTES + BM * 64 * 4;   // operand ring (3 x 64 KiB or 4 x 48 KiB) + a 64-column exchange buffer


__device__ __forceinline__ bool wait_counter(const uint32_t* p, uint32_t target) {
  for (uint32_t i = 0; i < kPollLimit; ++i) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    if (v >= target) return true;
  }
  return false;
}
__device__ __forceinline__ uint32_t peek_counter(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void signal_counter(uint32_t* p) {
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
// mbarrier wait that also orders after arrivals from other CTAs of the cluster
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t done = 0;
  for (uint32_t it = 0; it < kWaitLimit; ++it) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// arrive on the same barrier of CTA `rank` of this cluster
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t rank) {
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(bar)), "r"(rank));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(ra) : "memory");
}
__device__ __forceinline__ uint32_t bar_and(uint32_t id, uint32_t count, bool pred) {
  uint32_t r;
  asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.cta.red.and.pred p, %2, %3, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(r) : "r"((uint32_t)pred), "r"(id), "r"(count) : "memory");
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

}  // namespace
