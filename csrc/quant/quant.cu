// K12: block-quantised weights on the GPU.  ub_dequant expands a tensor to bf16 (used once at load time when the
// tensor-core path is wanted); ub_qgemv multiplies up to 8 activation rows with a quantised matrix without ever
// materialising it, which is the decode path for GGUF checkpoints: the kernel streams 4.5-8.5 bits per weight
// instead of 16.  The reference keeps such tensors as candle QMatMul on the CPU
// (crates/runtime/src/weight_loader_core.rs:554-584).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdlib.h>

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

// Q4_K fast path.  One warp owns RPW consecutive output rows; a lane takes one 64-value group of a block at a time
// (32 bytes of nibbles: the low nibbles are the group's first 32 values, the high nibbles its last 32), so the block
// header is decoded once per 64 weights and the activations of the group are loaded once for all RPW rows.  With
// v = d*s*q - dmin*m the dot product over a 32-value sub-block is d*s * sum(q x) - dmin*m * sum(x); sum(x) is shared
// by the rows.  MT is the activation-row count rounded up to a power of two (rows >= M repeat the last one).
template <int MT, int RPW>
__global__ void __launch_bounds__(256) qgemv_q4k_kernel(const uint8_t* __restrict__ w, const __nv_bfloat16* __restrict__ x,
                                                        __nv_bfloat16* __restrict__ out, int M, int N, int K) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * 8 + warp) * RPW;
  if (n0 >= N) return;
  const int nb = K >> 8, groups = nb << 2;
  float acc[RPW][MT];
#pragma unroll
  for (int r = 0; r < RPW; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
  for (int grp = lane; grp < groups; grp += 32) {
    const int b = grp >> 2, g = grp & 3;
    uint4 qa[RPW], qb[RPW];
    float ds0[RPW], ds1[RPW], dm0[RPW], dm1[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int n = min(n0 + r, N - 1);
      const uint8_t* blk = w + ((long long)n * nb + b) * 144;
      const uint4 h = __ldg(reinterpret_cast<const uint4*>(blk));
      qa[r] = __ldg(reinterpret_cast<const uint4*>(blk + 16 + g * 32));
      qb[r] = __ldg(reinterpret_cast<const uint4*>(blk + 32 + g * 32));
      const uint8_t* hb = reinterpret_cast<const uint8_t*>(&h);
      const float d = ubq_f16(hb), dmin = ubq_f16(hb + 2);
      const uint8_t* sc = hb + 4;
      int s[2], mn[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = 2 * g + e;
        if (j < 4) { s[e] = sc[j] & 63; mn[e] = sc[j + 4] & 63; }
        else { s[e] = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4); mn[e] = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
      }
      ds0[r] = d * (float)s[0]; ds1[r] = d * (float)s[1];
      dm0[r] = dmin * (float)mn[0]; dm1[r] = dmin * (float)mn[1];
    }
    float sx0[MT], sx1[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) sx0[m] = sx1[m] = 0.f;
    const long long xoff = (long long)b * 256 + g * 64;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      // bytes 8c..8c+7 of the group's nibbles: values 8c..8c+7 of the first half (low nibbles) and of the second half
      float ql[RPW][8], qh[RPW][8];
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const uint32_t* qw = (c < 2) ? reinterpret_cast<const uint32_t*>(&qa[r]) + 2 * c
                                     : reinterpret_cast<const uint32_t*>(&qb[r]) + 2 * (c - 2);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t byte = (qw[j >> 2] >> (8 * (j & 3))) & 0xFFu;
          ql[r][j] = (float)(byte & 0xFu);
          qh[r][j] = (float)(byte >> 4);
        }
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const long long row = (long long)min(m, M - 1) * K + xoff;
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(x + row + 8 * c));
        const uint4 bq = __ldg(reinterpret_cast<const uint4*>(x + row + 32 + 8 * c));
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&bq);
        float x0[8], x1[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fa = __bfloat1622float2(ap[j]), fb = __bfloat1622float2(bp[j]);
          x0[2 * j] = fa.x; x0[2 * j + 1] = fa.y;
          x1[2 * j] = fb.x; x1[2 * j + 1] = fb.y;
          sx0[m] += fa.x + fa.y;
          sx1[m] += fb.x + fb.y;
        }
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          float d0 = 0.f, d1 = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) { d0 += ql[r][j] * x0[j]; d1 += qh[r][j] * x1[j]; }
          acc[r][m] += ds0[r] * d0 + ds1[r] * d1;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[r][m] -= dm0[r] * sx0[m] + dm1[r] * sx1[m];
  }
#pragma unroll
  for (int r = 0; r < RPW; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float a = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      if (lane == 0 && m < M && n0 + r < N) out[(long long)m * N + n0 + r] = __float2bfloat16(a);
    }
}


// ------------------------------------------------------------------------------------------------------------
// Q4_K x bf16 on warp MMAs: the quantised weights are expanded to bf16 A fragments in registers and multiplied with
// up to 8 activation rows by m16n8k16 MMAs -- the weight-streaming GEMM of csrc/gemm/gemv.cu with a decode step in
// front.  A CTA owns 16 output columns; its warps split K by super-blocks of 256 weights.  Inside a super-block, lane
// (g = lane / 4, t = lane % 4) owns rows g and g + 8 and, in each of the eight 32-weight sub-blocks, the weights 8t ..
// 8t + 7: one 8-byte load per row and 64-weight group delivers them for two sub-blocks (low and high nibbles), and the
// matching activations x[token g][32 j + 8t ..] are one 16-byte load.  (A sum over k does not care which MMA k-slot a
// weight sits in, as long as the activation in the same slot is its partner.)  Nibbles become bf16 without integer
// conversions: byte 0x43 in front of a nibble q is the bf16 number 128 + q; q - 0 comes out of one exact subtraction and
// the weight d * s * q - dmin * m out of one bf16 FMA (scale and offset rounded to bf16, like the weight itself when the
// matrix is expanded to bf16).  The four lanes of a row each unpack two of the eight (scale, min) pairs and pass them
// on by shuffles.
// ------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void q_mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t bf16x2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// four bytes with one nibble value each -> (q0, q1) and (q2, q3) as bf16 pairs, scaled: q * s + c
__device__ __forceinline__ void q4_pairs(uint32_t nib, uint32_t s2, uint32_t c2, uint32_t& p01, uint32_t& p23) {
  const uint32_t k128 = 0x43004300u;
  p01 = bf16x2_fma(bf16x2_sub(__byte_perm(nib, 0x43434343u, 0x4140), k128), s2, c2);
  p23 = bf16x2_fma(bf16x2_sub(__byte_perm(nib, 0x43434343u, 0x4342), k128), s2, c2);
}

template <int NW>
__global__ void __launch_bounds__(NW * 32) qgemv_q4k_mma_kernel(const uint8_t* __restrict__ w, const __nv_bfloat16* __restrict__ x,
                                                                __nv_bfloat16* __restrict__ out, int M, int N, int K) {
  __shared__ float part[NW][16][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int col0 = blockIdx.x * 16;
  const int nb = K >> 8;
  const uint8_t* rowA = w + (long long)min(col0 + g, N - 1) * nb * 144;         // clamped rows are computed and dropped
  const uint8_t* rowB = w + (long long)min(col0 + g + 8, N - 1) * nb * 144;
  const __nv_bfloat16* xr = x + (long long)min(g, M - 1) * K;
  const bool has_x = g < M;
  float acc[2][4];
#pragma unroll
  for (int h = 0; h < 2; ++h) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;

  for (int b = warp; b < nb; b += NW) {
    const uint8_t* ba = rowA + b * 144;
    const uint8_t* bb = rowB + b * 144;
    const uint4 ha = __ldg(reinterpret_cast<const uint4*>(ba));     // d, dmin, 12 bytes of packed 6-bit scales / mins
    const uint4 hb = __ldg(reinterpret_cast<const uint4*>(bb));
    uint2 qa[4], qb[4];
#pragma unroll
    for (int gq = 0; gq < 4; ++gq) {
      qa[gq] = __ldcs(reinterpret_cast<const uint2*>(ba + 16 + 32 * gq + 8 * t));
      qb[gq] = __ldcs(reinterpret_cast<const uint2*>(bb + 16 + 32 * gq + 8 * t));
    }
    uint4 xv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      xv[j] = make_uint4(0, 0, 0, 0);
      if (has_x) xv[j] = __ldg(reinterpret_cast<const uint4*>(xr + (long long)b * 256 + 32 * j + 8 * t));
    }
    // this lane unpacks sub-blocks 2t and 2t + 1 of both rows: scale and offset as duplicated bf16 pairs
    uint32_t s2a[2], c2a[2], s2b[2], c2b[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int j = 2 * t + e;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const uint8_t* hp = reinterpret_cast<const uint8_t*>(rr == 0 ? &ha : &hb);
        const float d = ubq_f16(hp), dmin = ubq_f16(hp + 2);
        const uint8_t* sc = hp + 4;
        int sv, mv;
        if (j < 4) { sv = sc[j] & 63; mv = sc[j + 4] & 63; }
        else { sv = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4); mv = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
        const __nv_bfloat16 sb = __float2bfloat16(d * (float)sv), cb = __float2bfloat16(-dmin * (float)mv);
        const uint32_t s2 = (uint32_t)__bfloat16_as_ushort(sb) * 0x10001u, c2 = (uint32_t)__bfloat16_as_ushort(cb) * 0x10001u;
        if (rr == 0) { s2a[e] = s2; c2a[e] = c2; } else { s2b[e] = s2; c2b[e] = c2; }
      }
    }
#pragma unroll
    for (int gq = 0; gq < 4; ++gq) {
      // the (scale, offset) pairs of sub-blocks 2 gq and 2 gq + 1 live in lane gq of this row's quad
      const int src = (lane & ~3) | gq;
      const uint32_t sa0 = __shfl_sync(0xffffffffu, s2a[0], src), ca0 = __shfl_sync(0xffffffffu, c2a[0], src);
      const uint32_t sa1 = __shfl_sync(0xffffffffu, s2a[1], src), ca1 = __shfl_sync(0xffffffffu, c2a[1], src);
      const uint32_t sb0 = __shfl_sync(0xffffffffu, s2b[0], src), cb0 = __shfl_sync(0xffffffffu, c2b[0], src);
      const uint32_t sb1 = __shfl_sync(0xffffffffu, s2b[1], src), cb1 = __shfl_sync(0xffffffffu, c2b[1], src);
      uint32_t a01, a23, a45, a67, b01, b23, b45, b67;
      // low nibbles: sub-block 2 gq
      q4_pairs(qa[gq].x & 0x0F0F0F0Fu, sa0, ca0, a01, a23);
      q4_pairs(qa[gq].y & 0x0F0F0F0Fu, sa0, ca0, a45, a67);
      q4_pairs(qb[gq].x & 0x0F0F0F0Fu, sb0, cb0, b01, b23);
      q4_pairs(qb[gq].y & 0x0F0F0F0Fu, sb0, cb0, b45, b67);
      q_mma_bf16(acc[0], a01, b01, a23, b23, xv[2 * gq].x, xv[2 * gq].y);
      q_mma_bf16(acc[1], a45, b45, a67, b67, xv[2 * gq].z, xv[2 * gq].w);
      // high nibbles: sub-block 2 gq + 1
      q4_pairs((qa[gq].x >> 4) & 0x0F0F0F0Fu, sa1, ca1, a01, a23);
      q4_pairs((qa[gq].y >> 4) & 0x0F0F0F0Fu, sa1, ca1, a45, a67);
      q4_pairs((qb[gq].x >> 4) & 0x0F0F0F0Fu, sb1, cb1, b01, b23);
      q4_pairs((qb[gq].y >> 4) & 0x0F0F0F0Fu, sb1, cb1, b45, b67);
      q_mma_bf16(acc[0], a01, b01, a23, b23, xv[2 * gq + 1].x, xv[2 * gq + 1].y);
      q_mma_bf16(acc[1], a45, b45, a67, b67, xv[2 * gq + 1].z, xv[2 * gq + 1].w);
    }
  }
  // accumulator layout: c0 (row g, token 2t), c1 (row g, token 2t + 1), c2 (row g + 8, 2t), c3 (row g + 8, 2t + 1)
  part[warp][g][2 * t] = acc[0][0] + acc[1][0];
  part[warp][g][2 * t + 1] = acc[0][1] + acc[1][1];
  part[warp][g + 8][2 * t] = acc[0][2] + acc[1][2];
  part[warp][g + 8][2 * t + 1] = acc[0][3] + acc[1][3];
  __syncthreads();
  for (int i = threadIdx.x; i < 16 * 8; i += NW * 32) {
    const int cidx = i >> 3, m = i & 7;
    const int col = col0 + cidx;
    if (col >= N || m >= M) continue;
    float v = 0.f;
#pragma unroll
    for (int wq = 0; wq < NW; ++wq) v += part[wq][cidx][m];
    out[(long long)m * N + col] = __float2bfloat16(v);
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
  static int q4_mma = -1;
  if (q4_mma < 0) { const char* e = getenv("UB_Q4K_MMA"); q4_mma = (e != nullptr && e[0] == '0') ? 0 : 1; }
  if (q4_mma && qtype == UBQ_Q4_K && K % 256 == 0 && (reinterpret_cast<uintptr_t>(blocks) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    // warp-MMA kernel: nibbles expanded to bf16 fragments in registers, any row count up to 8 at the same cost
    const int nbk = K >> 8, tiles = (N + 15) / 16;
    int nw = 4;
    while (nw < 16 && tiles * nw < 148 * 16 && nbk >= 2 * nw) nw <<= 1;
    if (nw == 4) ub::qgemv_q4k_mma_kernel<4><<<tiles, 128, 0, st>>>(w, xp, op, M, N, K);
    else if (nw == 8) ub::qgemv_q4k_mma_kernel<8><<<tiles, 256, 0, st>>>(w, xp, op, M, N, K);
    else ub::qgemv_q4k_mma_kernel<16><<<tiles, 512, 0, st>>>(w, xp, op, M, N, K);
    cudaError_t e5 = cudaGetLastError();
    return e5 == cudaSuccess ? 0 : -(int)e5;
  }
  if (qtype == UBQ_Q4_K && K % 256 == 0 && (reinterpret_cast<uintptr_t>(blocks) & 15) == 0) {
    // specialised kernel: header decoded once per 64 weights, activations shared by 2 / 4 rows
    if (M == 1) ub::qgemv_q4k_kernel<1, 2><<<(N + 15) / 16, 256, 0, st>>>(w, xp, op, M, N, K);
    else if (M == 2) ub::qgemv_q4k_kernel<2, 2><<<(N + 15) / 16, 256, 0, st>>>(w, xp, op, M, N, K);
    else if (M <= 4) ub::qgemv_q4k_kernel<4, 4><<<(N + 31) / 32, 256, 0, st>>>(w, xp, op, M, N, K);
    else ub::qgemv_q4k_kernel<8, 4><<<(N + 31) / 32, 256, 0, st>>>(w, xp, op, M, N, K);
    cudaError_t e4 = cudaGetLastError();
    return e4 == cudaSuccess ? 0 : -(int)e4;
  }
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
