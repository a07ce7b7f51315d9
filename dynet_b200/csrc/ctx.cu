// Context, status reporting and the library-owned scratch arena.
#include <stdarg.h>
#include <stdlib.h>

#include "common.cuh"

int dyb200_fail(dyb200_ctx* ctx, int code, const char* fmt, ...) {
  if (ctx) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
    va_end(ap);
  }
  return code;
}

// Called at the start of every public entry point that (directly or through helpers) needs
// temporaries.  Releases the previous call's blocks; when the previous call overflowed the main
// block, waits for the stream, frees the overflow blocks and re-sizes the main block to the
// high-water mark, so the steady state never allocates.
int dyb200_scratch_begin(dyb200_ctx* ctx) {
  if (ctx->n_overflow > 0 || ctx->scratch_peak > ctx->scratch_bytes) {
    DYB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (int k = 0; k < ctx->n_overflow; ++k) cudaFree(ctx->overflow[k]);
    ctx->n_overflow = 0;
    if (ctx->scratch_peak > ctx->scratch_bytes) {
      if (ctx->scratch) DYB_CUDA(ctx, cudaFree(ctx->scratch));
      ctx->scratch = nullptr;
      ctx->scratch_bytes = 0;
      size_t want = ctx->scratch_peak + (ctx->scratch_peak >> 2) + (1u << 20);
      cudaError_t e = cudaMalloc(&ctx->scratch, want);
      if (e != cudaSuccess) {
        cudaGetLastError();
        return dyb200_fail(ctx, DYB200_ENOMEM, "scratch arena: cudaMalloc(%zu) failed: %s", want, cudaGetErrorString(e));
      }
      ctx->scratch_bytes = want;
    }
  }
  ctx->scratch_off = 0;
  return DYB200_OK;
}

int dyb200_scratch(dyb200_ctx* ctx, size_t bytes, void** out) {
  size_t off = (ctx->scratch_off + 255) & ~(size_t)255;
  if (bytes == 0) bytes = 256;
  if (off + bytes <= ctx->scratch_bytes) {
    *out = (char*)ctx->scratch + off;
  } else {
    if (ctx->n_overflow >= 64) return dyb200_fail(ctx, DYB200_ENOMEM, "scratch arena: too many overflow blocks in one call");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return dyb200_fail(ctx, DYB200_ENOMEM, "scratch arena: cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    }
    ctx->overflow[ctx->n_overflow++] = p;
    *out = p;
  }
  ctx->scratch_off = off + bytes;
  if (ctx->scratch_off > ctx->scratch_peak) ctx->scratch_peak = ctx->scratch_off;
  return DYB200_OK;
}

extern "C" {

const char* dyb200_version(void) { return "dyb200 1 sm_100a"; }

int dyb200_ctx_create(int device, void* stream, dyb200_ctx** out) {
  if (!out) return DYB200_EINVAL;
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0 || device < 0 || device >= count) {
    cudaGetLastError();
    return DYB200_ECUDA;  // no usable CUDA device: there is no CPU fallback
  }
  if (cudaSetDevice(device) != cudaSuccess) return DYB200_ECUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return DYB200_ECUDA;
  if (prop.major != 10) return DYB200_ERUNTIME;  // kernels are built for sm_100a only
  dyb200_ctx* c = (dyb200_ctx*)calloc(1, sizeof(dyb200_ctx));
  if (!c) return DYB200_ENOMEM;
  c->device = device;
  c->stream = (cudaStream_t)stream;
  c->sm_count = prop.multiProcessorCount;
  c->cluster_splitk = 1;
  c->seq_kernels = 1;
  if (cudaMalloc((void**)&c->dev_flags, DYB200_DEV_WORDS * 4) != cudaSuccess || cudaMemset(c->dev_flags, 0, DYB200_DEV_WORDS * 4) != cudaSuccess) {
    free(c);
    return DYB200_ENOMEM;
  }
  *out = c;
  return DYB200_OK;
}

int dyb200_ctx_destroy(dyb200_ctx* ctx) {
  if (!ctx) return DYB200_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  for (int k = 0; k < ctx->n_overflow; ++k) cudaFree(ctx->overflow[k]);
  for (auto& e : ctx->param_pack) { if (e.hi) cudaFree(e.hi); if (e.lo) cudaFree(e.lo); }
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->dev_flags) cudaFree(ctx->dev_flags);
  free(ctx);
  return DYB200_OK;
}

int dyb200_ctx_dependent_launch(dyb200_ctx* ctx, int enable) {
  if (!ctx) return DYB200_EINVAL;
  ctx->pdl = enable ? 1 : 0;
  return DYB200_OK;
}

int dyb200_ctx_cluster_splitk(dyb200_ctx* ctx, int enable) {
  if (!ctx) return DYB200_EINVAL;
  ctx->cluster_splitk = enable ? 1 : 0;
  return DYB200_OK;
}

int dyb200_ctx_sequence_kernels(dyb200_ctx* ctx, int enable) {
  if (!ctx) return DYB200_EINVAL;
  ctx->seq_kernels = enable ? 1 : 0;
  // enable == 2: launch them without the cooperative attribute (for tools that cannot replay cooperative launches; the
  // grid still never exceeds what the GPU holds at once, and every wait in the kernels is bounded)
  ctx->seq_coop = enable == 2 ? -1 : 0;
  return DYB200_OK;
}

int dyb200_ctx_param_cache(dyb200_ctx* ctx, int enable) {
  ctx->param_cache_on = enable ? 1 : 0;
  ctx->param_version++;
  return DYB200_OK;
}

int dyb200_ctx_params_changed(dyb200_ctx* ctx) {
  ctx->param_version++;
  return DYB200_OK;
}

int dyb200_ctx_profile_begin(dyb200_ctx* ctx, int capacity) {
  DYB_CHECK_ARG(ctx, capacity > 0 && capacity <= (1 << 20), "profile_begin: capacity out of range");
  if (ctx->prof_ev) return dyb200_fail(ctx, DYB200_ERUNTIME, "profile_begin: already profiling");
  ctx->prof_ev = (cudaEvent_t*)calloc(2 * (size_t)capacity, sizeof(cudaEvent_t));
  ctx->prof_flops = (double*)calloc(capacity, sizeof(double));
  ctx->prof_path = (int*)calloc(capacity, sizeof(int));
  ctx->prof_shape = (uint32_t*)calloc(4 * (size_t)capacity, sizeof(uint32_t));
  if (!ctx->prof_ev || !ctx->prof_flops || !ctx->prof_path || !ctx->prof_shape) return dyb200_fail(ctx, DYB200_ENOMEM, "profile_begin: host allocation failed");
  for (int k = 0; k < 2 * capacity; ++k) DYB_CUDA(ctx, cudaEventCreate(&ctx->prof_ev[k]));
  ctx->prof_cap = capacity;
  ctx->prof_n = 0;
  return DYB200_OK;
}

int dyb200_ctx_profile_launch(dyb200_ctx* ctx, int k, uint32_t shape_out[4], int* path_out, float* ms_out, double* flops_out) {
  if (!ctx->prof_ev) return dyb200_fail(ctx, DYB200_ERUNTIME, "profile_launch: profiling is not on");
  DYB_CHECK_ARG(ctx, k >= 0 && k < ctx->prof_n, "profile_launch: index %d out of range (%d launches recorded)", k, ctx->prof_n);
  DYB_CUDA(ctx, cudaEventSynchronize(ctx->prof_ev[2 * k + 1]));
  float t = 0.f;
  DYB_CUDA(ctx, cudaEventElapsedTime(&t, ctx->prof_ev[2 * k], ctx->prof_ev[2 * k + 1]));
  if (shape_out) for (int q = 0; q < 4; ++q) shape_out[q] = ctx->prof_shape[4 * k + q];
  if (path_out) *path_out = ctx->prof_path[k];
  if (ms_out) *ms_out = t;
  if (flops_out) *flops_out = ctx->prof_flops[k];
  return DYB200_OK;
}

int dyb200_ctx_profile_count(const dyb200_ctx* ctx) { return ctx && ctx->prof_ev ? ctx->prof_n : 0; }

int dyb200_ctx_profile_end(dyb200_ctx* ctx, double* ms_out, uint64_t* launches_out, double* flops_out) {
  if (!ctx->prof_ev) return dyb200_fail(ctx, DYB200_ERUNTIME, "profile_end: profiling is not on");
  DYB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  double ms[2] = {0, 0}, fl[2] = {0, 0};
  uint64_t cnt[2] = {0, 0};
  for (int k = 0; k < ctx->prof_n; ++k) {
    float t = 0.f;
    DYB_CUDA(ctx, cudaEventElapsedTime(&t, ctx->prof_ev[2 * k], ctx->prof_ev[2 * k + 1]));
    int p = ctx->prof_path[k] ? 1 : 0;
    ms[p] += t; fl[p] += ctx->prof_flops[k]; cnt[p]++;
  }
  for (int k = 0; k < 2 * ctx->prof_cap; ++k) cudaEventDestroy(ctx->prof_ev[k]);
  free(ctx->prof_ev); free(ctx->prof_flops); free(ctx->prof_path); free(ctx->prof_shape);
  ctx->prof_ev = nullptr; ctx->prof_flops = nullptr; ctx->prof_path = nullptr; ctx->prof_shape = nullptr;
  ctx->prof_cap = ctx->prof_n = 0;
  for (int p = 0; p < 2; ++p) {
    if (ms_out) ms_out[p] = ms[p];
    if (launches_out) launches_out[p] = cnt[p];
    if (flops_out) flops_out[p] = fl[p];
  }
  return DYB200_OK;
}

const char* dyb200_last_error(const dyb200_ctx* ctx) { return ctx ? ctx->err : "null context"; }

uint64_t dyb200_ctx_launch_count(const dyb200_ctx* ctx) { return ctx ? ctx->launches : 0; }

int dyb200_ctx_check_device_errors(dyb200_ctx* ctx, uint32_t* flags_out) {
  uint32_t f = 0;
  DYB_CUDA(ctx, cudaMemcpyAsync(&f, ctx->dev_flags, sizeof(f), cudaMemcpyDeviceToHost, ctx->stream));
  DYB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (f) DYB_CUDA(ctx, cudaMemsetAsync(ctx->dev_flags, 0, sizeof(f), ctx->stream));
  if (flags_out) *flags_out = f;
  if (f) return dyb200_fail(ctx, DYB200_ECUDA, "device error flags 0x%x (1=bad index, 2=wait timeout)", f);
  return DYB200_OK;
}

}  // extern "C"
