// K12: block-quantised weights on the GPU.  ub_dequant expands a tensor to bf16 (used once at load time when the
// tensor-core path is wanted); ub_qgemv multiplies up to 8 activation rows with a quantised matrix without ever
// materialising it, which is the decode path for GGUF checkpoints: the kernel streams 4.5-8.5 bits per weight
// instead of 16.  The reference keeps such tensors as candle QMatMul on the CPU
// (crates/runtime/src/weight_loader_core.rs:554-584).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../include/unillm_b200.h"
#include "quant_blocks.h"

namespace ub {

__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ blocks, __nv_bfloat16* __restrict__ out,
                                                      long long n8, int qtype, int be, int bb) {
  for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x; c < n8; c += (long long)gridDim.x * blockDim.x) {
    const long long e = c * 8;
    float v[8];
    ubq_decode8(blocks + (e / be) * bb, qtype, int(e % be), v);
    __nv_bfloat162 o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    *reinterpret_cast<uint4*>(out + e) = *reinterpret_cast<uint4*>(o);
  }
}

// One warp per output feature n; lanes take 8-element chunks of K round-robin.
template <int M>
__global__ void __launch_bounds__(256) qgemv_kernel(const uint8_t* __restrict__ w, const __nv_bfloat16* __restrict__ x,
                                                    __nv_bfloat16* __restrict__ out, int N, int K, int qtype, int be, int bb) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const uint8_t* row = w + (long long)n * (K / be) * bb;
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  for (int k = lane * 8; k < K; k += 256) {
    float v[8];
    ubq_decode8(row + (long long)(k / be) * bb, qtype, k % be, v);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + (long long)m * K + k));
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(xp[j]);
        acc[m] += v[2 * j] * f.x + v[2 * j + 1] * f.y;
      }
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float a = acc[m];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (lane == 0) out[(long long)m * N + n] = __float2bfloat16(a);
  }
}

}  // namespace ub

extern "C" int ub_dequant(const void* blocks, void* out_bf16, long long n_elems, int qtype, void* stream) {
  const int be = ubq_block_elems(qtype), bb = ubq_block_bytes(qtype);
  if (bb == 0) return -2;
  if (n_elems <= 0) return 0;
  if (n_elems % be != 0 || (reinterpret_cast<uintptr_t>(out_bf16) & 15)) return -3;
  const long long n8 = n_elems / 8;
  long long blocks_ll = (n8 + 255) / 256;
  const int grid = (int)(blocks_ll > 148 * 16 ? 148 * 16 : blocks_ll);
  ub::dequant_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(blocks), reinterpret_cast<__nv_bfloat16*>(out_bf16), n8, qtype, be, bb);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int ub_qgemv(const void* blocks, const void* x, void* out, int M, int N, int K, int qtype, void* stream) {
  const int be = ubq_block_elems(qtype), bb = ubq_block_bytes(qtype);
  if (bb == 0) return -2;
  if (M <= 0 || N <= 0) return 0;
  if (M > 8 || K % be != 0 || K % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15)) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const uint8_t* w = reinterpret_cast<const uint8_t*>(blocks);
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(out);
  const int grid = (N + 7) / 8;
#define UB_QGEMV(MM) ub::qgemv_kernel<MM><<<grid, 256, 0, st>>>(w, xp, op, N, K, qtype, be, bb)
  switch (M) {
    case 1: UB_QGEMV(1); break;
    case 2: UB_QGEMV(2); break;
    case 3: UB_QGEMV(3); break;
    case 4: UB_QGEMV(4); break;
    case 5: UB_QGEMV(5); break;
    case 6: UB_QGEMV(6); break;
    case 7: UB_QGEMV(7); break;
    default: UB_QGEMV(8); break;
  }
#undef UB_QGEMV
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
