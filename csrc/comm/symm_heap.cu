// C1: symmetric heap over the CUDA virtual-memory API, with an NVSwitch multicast view.
//
// Every rank of a node allocates one physical block (cuMemCreate, shareable as a POSIX file descriptor), maps it
// locally, hands the descriptor to its peers (the Python side passes it over a Unix socket) and maps every peer's
// block into its own address space: plain loads and stores on those addresses travel over NVLink.  On top of that,
// when the devices support it, ONE multicast object spans the ranks' blocks (cuMulticastCreate / AddDevice /
// BindMem): an address inside its mapping names the same offset on every rank at once, so
//   multimem.st           stores one value to all ranks' copies (the switch replicates it),
//   multimem.ld_reduce    loads the sum of all ranks' copies (the switch reduces it),
// which is what the all-gather producer and the reduce-scatter consumer of the tensor-parallel pipeline use.
//
// Order of calls on every rank (the barriers are the caller's, over its process group):
//   ub_symm_alloc -> [exchange fds] -> ub_symm_map_peer per peer
//   rank 0: ub_symm_mc_create -> [send its fd to all] -> others: ub_symm_mc_import
//   all: ub_symm_mc_add_device -> [barrier] -> ub_symm_mc_bind -> [barrier] -> ub_symm_mc_map
//   ... use ...   [barrier] -> ub_symm_mc_release (unmap, unbind) -> [barrier] -> ub_symm_unmap / ub_symm_free
// A rank must not leave while its memory is still bound to a multicast object that peers use: release in that order.
//
// The reference declares a device-memory FFI it never ships (crates/kv/src/gpu_memory.rs:479-501) and has no
// peer or multicast memory at all.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include "../include/unillm_b200.h"

namespace {

template <typename F>
F drv(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
  return reinterpret_cast<F>(p);
}

#define DRV(fn) static auto p_##fn = drv<decltype(&fn)>(#fn)

thread_local char g_err[256] = "";
int fail(const char* what, CUresult r) {
  snprintf(g_err, sizeof(g_err), "%s failed with CUresult %d", what, (int)r);
  return -1000 - (int)r;
}

CUmemAllocationProp alloc_prop(int dev) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int map_rw(CUmemGenericAllocationHandle h, size_t bytes, size_t align, int dev, CUdeviceptr* out) {
  DRV(cuMemAddressReserve);
  DRV(cuMemMap);
  DRV(cuMemSetAccess);
  DRV(cuMemAddressFree);
  if (!p_cuMemAddressReserve || !p_cuMemMap || !p_cuMemSetAccess) return fail("driver entry points", CUDA_ERROR_NOT_FOUND);
  CUdeviceptr va = 0;
  CUresult r = p_cuMemAddressReserve(&va, bytes, align, 0, 0);
  if (r != CUDA_SUCCESS) return fail("cuMemAddressReserve", r);
  r = p_cuMemMap(va, bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    p_cuMemAddressFree(va, bytes);
    return fail("cuMemMap", r);
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = p_cuMemSetAccess(va, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) return fail("cuMemSetAccess", r);
  *out = va;
  return 0;
}

}  // namespace

extern "C" {

const char* ub_symm_error(void) { return g_err; }

/* *vmm = 1 when the device can export allocations as POSIX file descriptors; *multicast = 1 when it supports
   NVSwitch multicast objects. */
int ub_symm_supported(int dev, int* vmm, int* multicast) {
  DRV(cuDeviceGetAttribute);
  if (!p_cuDeviceGetAttribute) return fail("driver entry points", CUDA_ERROR_NOT_FOUND);
  int a = 0, b = 0;
  p_cuDeviceGetAttribute(&a, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
  p_cuDeviceGetAttribute(&b, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
  if (vmm) *vmm = a;
  if (multicast) *multicast = b;
  return 0;
}

/* Rounds `bytes` up to what both the allocation and (when `world` > 0) a multicast object over `world` devices
   accept. */
int ub_symm_round_size(unsigned long long bytes, int dev, int world, unsigned long long* out) {
  DRV(cuMemGetAllocationGranularity);
  DRV(cuMulticastGetGranularity);
  if (!p_cuMemGetAllocationGranularity) return fail("driver entry points", CUDA_ERROR_NOT_FOUND);
  CUmemAllocationProp prop = alloc_prop(dev);
  size_t g = 0;
  CUresult r = p_cuMemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) return fail("cuMemGetAllocationGranularity", r);
  if (world > 0 && p_cuMulticastGetGranularity) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = (unsigned)world;
    mp.size = bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (p_cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > g) g = mg;
  }
  if (g == 0) g = 2u << 20;
  *out = (bytes + g - 1) / g * g;
  return 0;
}

/* Physical block of `bytes` (already rounded) on `dev`, mapped read-write; returns its handle, a shareable file
   descriptor (the caller closes it once every peer has it) and the local address. */
int ub_symm_alloc(unsigned long long bytes, int dev, unsigned long long* handle, int* fd, void** va) {
  DRV(cuMemCreate);
  DRV(cuMemExportToShareableHandle);
  DRV(cuMemRelease);
  if (!p_cuMemCreate || !p_cuMemExportToShareableHandle) return fail("driver entry points", CUDA_ERROR_NOT_FOUND);
  if (cudaSetDevice(dev) != cudaSuccess || cudaFree(0) != cudaSuccess) return fail("cudaSetDevice", CUDA_ERROR_INVALID_DEVICE);
  CUmemAllocationProp prop = alloc_prop(dev);
  CUmemGenericAllocationHandle h = 0;
  CUresult r = p_cuMemCreate(&h, bytes, &prop, 0);
  if (r != CUDA_SUCCESS) return fail("cuMemCreate", r);
  int f = -1;
  r = p_cuMemExportToShareableHandle(&f, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    p_cuMemRelease(h);
    return fail("cuMemExportToShareableHandle", r);
  }
  CUdeviceptr p = 0;
  int rc = map_rw(h, bytes, 0, dev, &p);
  if (rc != 0) {
    close(f);
    p_cuMemRelease(h);
    return rc;
  }
  *handle = (unsigned long long)h;
  *fd = f;
  *va = reinterpret_cast<void*>(p);
  return 0;
}

/* Maps a peer's block (its file descriptor, received from that process) read-write on `dev`. */
int ub_symm_map_peer(int fd, unsigned long long bytes, int dev, unsigned long long* handle, void** va) {
  DRV(cuMemImportFromShareableHandle);
  DRV(cuMemRelease);
  if (!p_cuMemImportFromShareableHandle) return fail("driver entry points", CUDA_ERROR_NOT_FOUND);
  CUmemGenericAllocationHandle h = 0;
  CUresult r = p_cuMemImportFromShareableHandle(&h, reinterpret_cast<void*>((uintptr_t)fd), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return fail("cuMemImportFromShareableHandle", r);
  CUdeviceptr p = 0;
  int rc = map_rw(h, bytes, 0, dev, &p);
  if (rc != 0) {
    p_cuMemRelease(h);
    return rc;
  }
  *handle = (unsigned long long)h;
  *va = reinterpret_cast<void*>(p);
  return 0;
}

int ub_symm_unmap(void* va, unsigned long long bytes, unsigned long long handle) {
  DRV(cuMemUnmap);
  DRV(cuMemAddressFree);
  DRV(cuMemRelease);
  if (!p_cuMemUnmap) return fail("driver entry points", CUDA_ERROR_NOT_FOUND);
  CUresult r = CUDA_SUCCESS;
  if (va != nullptr) {
    r = p_cuMemUnmap((CUdeviceptr)va, bytes);
    if (r == CUDA_SUCCESS) r = p_cuMemAddressFree((CUdeviceptr)va, bytes);
  }
  if (handle != 0) {
    CUresult r2 = p_cuMemRelease((CUmemGenericAllocationHandle)handle);
    if (r == CUDA_SUCCESS) r = r2;
  }
  return r == CUDA_SUCCESS ? 0 : fail("cuMemUnmap / cuMemRelease", r);
}

/* Rank 0: a multicast object for `world` devices and `bytes` (rounded); returns its handle and a shareable fd. */
int ub_symm_mc_create(unsigned long long bytes, int world, unsigned long long* mc, int* fd) {
  DRV(cuMulticastCreate);
  DRV(cuMemExportToShareableHandle);
  DRV(cuMemRelease);
  if (!p_cuMulticastCreate) return fail("driver entry points (multicast)", CUDA_ERROR_NOT_FOUND);
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = (unsigned)world;
  mp.size = bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h = 0;
  CUresult r = p_cuMulticastCreate(&h, &mp);
  if (r != CUDA_SUCCESS) return fail("cuMulticastCreate", r);
  int f = -1;
  r = p_cuMemExportToShareableHandle(&f, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    p_cuMemRelease(h);
    return fail("cuMemExportToShareableHandle (multicast)", r);
  }
  *mc = (unsigned long long)h;
  *fd = f;
  return 0;
}

int ub_symm_mc_import(int fd, unsigned long long* mc) {
  DRV(cuMemImportFromShareableHandle);
  if (!p_cuMemImportFromShareableHandle) return fail("driver entry points", CUDA_ERROR_NOT_FOUND);
  CUmemGenericAllocationHandle h = 0;
  CUresult r = p_cuMemImportFromShareableHandle(&h, reinterpret_cast<void*>((uintptr_t)fd), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return fail("cuMemImportFromShareableHandle (multicast)", r);
  *mc = (unsigned long long)h;
  return 0;
}

int ub_symm_mc_add_device(unsigned long long mc, int dev) {
  DRV(cuMulticastAddDevice);
  if (!p_cuMulticastAddDevice) return fail("driver entry points (multicast)", CUDA_ERROR_NOT_FOUND);
  CUresult r = p_cuMulticastAddDevice((CUmemGenericAllocationHandle)mc, (CUdevice)dev);
  return r == CUDA_SUCCESS ? 0 : fail("cuMulticastAddDevice", r);
}

/* Binds this rank's physical block at offset 0 of the multicast object (blocks until every device was added). */
int ub_symm_mc_bind(unsigned long long mc, unsigned long long local_handle, unsigned long long bytes) {
  DRV(cuMulticastBindMem);
  if (!p_cuMulticastBindMem) return fail("driver entry points (multicast)", CUDA_ERROR_NOT_FOUND);
  CUresult r = p_cuMulticastBindMem((CUmemGenericAllocationHandle)mc, 0, (CUmemGenericAllocationHandle)local_handle, 0, bytes, 0);
  return r == CUDA_SUCCESS ? 0 : fail("cuMulticastBindMem", r);
}

int ub_symm_mc_map(unsigned long long mc, unsigned long long bytes, int dev, void** va) {
  CUdeviceptr p = 0;
  int rc = map_rw((CUmemGenericAllocationHandle)mc, bytes, 0, dev, &p);
  if (rc != 0) return rc;
  *va = reinterpret_cast<void*>(p);
  return 0;
}

/* Unmaps the multicast view and unbinds this rank's memory from the object.  Call on every rank, with a barrier
   before (nobody uses the view any more) and after (before any rank frees its block). */
int ub_symm_mc_release(unsigned long long mc, void* mc_va, unsigned long long bytes, int dev) {
  DRV(cuMemUnmap);
  DRV(cuMemAddressFree);
  DRV(cuMulticastUnbind);
  DRV(cuMemRelease);
  CUresult r = CUDA_SUCCESS;
  if (mc_va != nullptr && p_cuMemUnmap) {
    r = p_cuMemUnmap((CUdeviceptr)mc_va, bytes);
    if (r == CUDA_SUCCESS && p_cuMemAddressFree) r = p_cuMemAddressFree((CUdeviceptr)mc_va, bytes);
  }
  if (mc != 0) {
    if (p_cuMulticastUnbind) {
      CUresult r2 = p_cuMulticastUnbind((CUmemGenericAllocationHandle)mc, (CUdevice)dev, 0, bytes);
      if (r == CUDA_SUCCESS) r = r2;
    }
    if (p_cuMemRelease) {
      CUresult r3 = p_cuMemRelease((CUmemGenericAllocationHandle)mc);
      if (r == CUDA_SUCCESS) r = r3;
    }
  }
  return r == CUDA_SUCCESS ? 0 : fail("multicast release", r);
}

}  // extern "C"

// ----------------------------------------------------------------------------------------------
// Probes: NVLink copy bandwidth with plain peer stores / loads, and the two multimem primitives.
// Each is one kernel timed by the caller with CUDA events; `n16` counts 16-byte elements.
// ----------------------------------------------------------------------------------------------
namespace ub {

__global__ void __launch_bounds__(256) peer_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) dst[i] = src[i];
}

// every 16 bytes of `src` (local) go to all ranks' copies through the multicast address `mc_dst`
__global__ void __launch_bounds__(256) multimem_st_kernel(const uint4* __restrict__ src, uint4* mc_dst, long long n16) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const uint4 v = src[i];
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_dst + i), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
  }
}

// dst (local) = sum over all ranks' copies of the bf16 pairs behind the multicast address `mc_src`
__global__ void __launch_bounds__(256) multimem_ld_reduce_kernel(const uint4* mc_src, uint4* __restrict__ dst, long long n16) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc_src + i)
                 : "memory");
    dst[i] = v;
  }
}

}  // namespace ub

extern "C" {

/* kind 0: dst[i] = src[i] (either side may be a peer mapping); 1: multimem.st of src to the multicast address dst;
   2: dst = multimem.ld_reduce (bf16x2 add, fp32 accumulation) of the multicast address src. */
int ub_symm_probe(int kind, const void* src, void* dst, long long bytes, int ctas, void* stream_v) {
  if (bytes <= 0 || bytes % 16 != 0) return -2;
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -3;
  if (ctas <= 0) ctas = 148 * 4;
  cudaStream_t st = (cudaStream_t)stream_v;
  const long long n16 = bytes / 16;
  switch (kind) {
    case 0: ub::peer_copy_kernel<<<ctas, 256, 0, st>>>((const uint4*)src, (uint4*)dst, n16); break;
    case 1: ub::multimem_st_kernel<<<ctas, 256, 0, st>>>((const uint4*)src, (uint4*)dst, n16); break;
    case 2: ub::multimem_ld_reduce_kernel<<<ctas, 256, 0, st>>>((const uint4*)src, (uint4*)dst, n16); break;
    default: return -4;
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

}  // extern "C"
