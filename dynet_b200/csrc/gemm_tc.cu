// 3xTF32 tensor-pipe GEMM (tcgen05 + TMEM + TMA).  Placeholder until the kernel lands:
// reports "not handled" so the dispatcher uses the CUDA-core path.
#include "gemm.cuh"

int dyb200_gemm_tc(dyb200_ctx*, uint32_t, uint32_t, int, const GemmPair*, const GemmEpilogue&, int* handled) {
  *handled = 0;
  return DYB200_ERUNTIME;
}
