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

// Returns a pointer to at least `bytes` of device scratch, 256-byte aligned.  The
// arena only grows; growing synchronises the stream first so that no kernel in
// flight still reads the old block.
int dyb200_scratch(dyb200_ctx* ctx, size_t bytes, void** out) {
  if (bytes > ctx->scratch_bytes) {
    size_t want = bytes + (bytes >> 2) + (1u << 20);
    DYB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch) DYB_CUDA(ctx, cudaFree(ctx->scratch));
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    cudaError_t e = cudaMalloc(&ctx->scratch, want);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return dyb200_fail(ctx, DYB200_ENOMEM, "scratch arena: cudaMalloc(%zu) failed: %s", want,
                         cudaGetErrorString(e));
    }
    ctx->scratch_bytes = want;
  }
  *out = ctx->scratch;
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
  if (cudaMalloc((void**)&c->dev_flags, 256) != cudaSuccess || cudaMemset(c->dev_flags, 0, 256) != cudaSuccess) {
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
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->dev_flags) cudaFree(ctx->dev_flags);
  free(ctx);
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
