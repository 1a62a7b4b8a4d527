// Probe of the rate at which one SM can fill its shared memory from L2, for the three kinds of copy a GEMM producer
// could use for a 16 KB operand tile (128 rows x 64 bf16):
//   mode 0  one linear bulk copy (cp.async.bulk) of 16 KB that is contiguous in global memory
//   mode 1  one 2-D tensor copy {64, 128} with the 128-byte swizzle from a row-major matrix (row pitch = K * 2 bytes):
//           what the GEMM kernels issue today
//   mode 2  the same tensor copy from tiles that are stored contiguously (row pitch 128 bytes)
// One thread per CTA keeps six copies (96 KB) in flight; every CTA of a full-device grid walks its own tiles of an
// L2-resident buffer.  Every wait is bounded; a timed-out wait is reported in err[0].  Measured on B200 inside this
// library: 31 - 34 B per clock and SM for all three modes, i.e. the address pattern and the kind of copy do not matter
// at this depth; what does is the number of bytes in flight over the L2 round trip of about 3 000 cycles under load (a
// stand-alone build of mode 0 with 32 KB copies, 192 KB in flight, reached 70 B per clock).  The plain GEMMs pull
// 34.5 B per clock and SM whether they hold five or six stages, so they meet a chip-wide limit (about 9 TB/s for
// their mix of L2 and HBM traffic) rather than this depth limit.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"
#include "../include/unillm_b200.h"

namespace ub {
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld_elems, int box_rows,
                      int box_cols);

namespace fillprobe {

constexpr int STAGES = 6;
constexpr int TILE = 16384;

__device__ __forceinline__ bool wait_bounded(uint64_t* bar, uint32_t parity, int* err) {
  for (int i = 0; i < 30000; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  set_err(err, ERR_MBAR_TIMEOUT, 900);
  return false;
}

__global__ void __launch_bounds__(64) fill_probe_kernel(const __grid_constant__ CUtensorMap tm, const uint8_t* src, int mode,
                                                        int steps, int row_blocks, int k_blocks, int* err, long long* cycles) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(sm + STAGES * TILE);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();
  const long long t0 = clock64();
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int i = 0; i < steps + STAGES && ok; ++i) {
      if (i >= STAGES) ok = wait_bounded(&full[(i - STAGES) % STAGES], ((i - STAGES) / STAGES) & 1, err);
      if (i < steps && ok) {
        const int s = i % STAGES;
        const int kb = i % k_blocks, rb = (int(blockIdx.x) * 7 + i / k_blocks) % row_blocks;   // 128 rows, then the next 128
        const long long tile = (long long)rb * k_blocks + kb;
        mbar_arrive_expect_tx(&full[s], TILE);
        if (mode == 0) {
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(smem_u32(sm + s * TILE)), "l"(src + tile * TILE), "r"((uint32_t)TILE), "r"(smem_u32(&full[s]))
                       : "memory");
        } else if (mode == 1) {
          tma_load_2d(sm + s * TILE, &tm, &full[s], kb * 64, rb * 128);
        } else {
          tma_load_2d(sm + s * TILE, &tm, &full[s], 0, int(tile) * 128);
        }
      }
    }
  }
  __syncthreads();
  const long long t1 = clock64();
  if (err != nullptr && *reinterpret_cast<volatile int*>(err) != 0) {
    for (int i = 0; i < 50; ++i) __nanosleep(20000);      // copies in flight land before the CTA leaves
  }
  if (threadIdx.x == 0) cycles[blockIdx.x] = t1 - t0;
}

}  // namespace fillprobe
}  // namespace ub

// buf: bf16 [rows][K] (rows % 128 == 0, K % 64 == 0), ideally smaller than L2.  cycles: int64 [number of SMs].
// Launches one CTA per SM on `stream`; each brings in `steps` tiles of 16 KB.  Returns the grid size, negative on error.
extern "C" int ub_fill_probe(const void* buf, int rows, int K, int mode, int steps, int* err, long long* cycles, void* stream) {
  using namespace ub;
  using namespace ub::fillprobe;
  if (rows <= 0 || rows % 128 != 0 || K <= 0 || K % 64 != 0 || mode < 0 || mode > 2 || steps <= 0) return -1;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  CUtensorMap tm;
  int rc = mode == 2 ? make_tmap_bf16_2d(&tm, buf, (long long)rows * K / 64, 64, 64, 128, 64)
                     : make_tmap_bf16_2d(&tm, buf, rows, K, K, 128, 64);
  if (rc != 0) return rc < 0 ? rc : -rc;
  const int smem = STAGES * TILE + 1024 + 256;
  cudaError_t e = cudaFuncSetAttribute(fill_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return -(int)e;
  fill_probe_kernel<<<sms, 64, smem, reinterpret_cast<cudaStream_t>(stream)>>>(tm, reinterpret_cast<const uint8_t*>(buf), mode, steps,
                                                                                rows / 128, K / 64, err, cycles);
  e = cudaGetLastError();
  return e == cudaSuccess ? sms : -(int)e;
}
