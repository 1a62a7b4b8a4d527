// C2: the CUDA half of the device-memory FFI that the reference declares but never ships
// (crates/kv/src/gpu_memory.rs:479-501: cuda_malloc_aligned, cuda_free, pinned host memory,
// async H2D/D2H copies, stream sync, memory info, device properties).  Plain C ABI over the CUDA
// runtime; return value is 0 or the negated cudaError_t.  One cudaMemcpyAsync per copy.
#include "../include/unillm_b200.h"
#include <cuda_runtime.h>
#include <string.h>

static inline int rc(cudaError_t e) { return e == cudaSuccess ? 0 : -(int)e; }

extern "C" int ub_cuda_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}
extern "C" int ub_cuda_set_device(int dev) { return rc(cudaSetDevice(dev)); }

extern "C" int ub_cuda_malloc_aligned(void** ptr, unsigned long long bytes, unsigned long long align) {
  // cudaMalloc returns addresses aligned to at least 256 bytes; larger alignments are met by
  // over-allocating is not needed for the pool (it asks for 256).
  if (align > 256) return -(int)cudaErrorInvalidValue;
  return rc(cudaMalloc(ptr, (size_t)bytes));
}
extern "C" int ub_cuda_free(void* ptr) { return rc(cudaFree(ptr)); }
extern "C" int ub_cuda_malloc_host(void** ptr, unsigned long long bytes) { return rc(cudaMallocHost(ptr, (size_t)bytes)); }
extern "C" int ub_cuda_free_host(void* ptr) { return rc(cudaFreeHost(ptr)); }
extern "C" int ub_cuda_memcpy_h2d_async(void* dst, const void* src, unsigned long long bytes, void* stream) {
  return rc(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
}
extern "C" int ub_cuda_memcpy_d2h_async(void* dst, const void* src, unsigned long long bytes, void* stream) {
  return rc(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
}
extern "C" int ub_cuda_memcpy_d2d_async(void* dst, const void* src, unsigned long long bytes, void* stream) {
  return rc(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
}
extern "C" int ub_cuda_stream_create(void** stream) {
  cudaStream_t s;
  cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  *stream = (void*)s;
  return rc(e);
}
extern "C" int ub_cuda_stream_destroy(void* stream) { return rc(cudaStreamDestroy((cudaStream_t)stream)); }
extern "C" int ub_cuda_stream_synchronize(void* stream) { return rc(cudaStreamSynchronize((cudaStream_t)stream)); }
extern "C" int ub_cuda_device_synchronize(void) { return rc(cudaDeviceSynchronize()); }
extern "C" int ub_cuda_mem_info(unsigned long long* free_b, unsigned long long* total_b) {
  size_t f = 0, t = 0;
  cudaError_t e = cudaMemGetInfo(&f, &t);
  *free_b = f;
  *total_b = t;
  return rc(e);
}
extern "C" int ub_cuda_device_props(int dev, UbDeviceProps* out) {
  cudaDeviceProp p;
  cudaError_t e = cudaGetDeviceProperties(&p, dev);
  if (e != cudaSuccess) return rc(e);
  memset(out, 0, sizeof(*out));
  strncpy(out->name, p.name, sizeof(out->name) - 1);
  out->total_mem = p.totalGlobalMem;
  out->sm_count = p.multiProcessorCount;
  out->cc_major = p.major;
  out->cc_minor = p.minor;
  out->max_smem_per_block = (int)p.sharedMemPerBlockOptin;
  out->l2_bytes = p.l2CacheSize;
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, dev) == cudaSuccess) out->clock_khz = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, dev) == cudaSuccess) out->mem_clock_khz = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrGlobalMemoryBusWidth, dev) == cudaSuccess) out->mem_bus_bits = v;
  return 0;
}
extern "C" const char* ub_cuda_error_string(int code) {
  return cudaGetErrorString((cudaError_t)(code < 0 ? -code : code));
}
