// K2s: the GEMM at one to 16 tokens (single-stream decode, small decode batches) as a weight-streaming kernel.
//
// At M <= 16 the product reads every weight once and does a handful of multiply-adds per element: it is a copy of the
// weight matrix.  The tcgen05 kernel is a poor fit there (a 128 x 16 tile per CTA, at most eight K slices per tile, a
// fill / drain per launch: 0.39 of the copy bandwidth at 16 tokens), and a CUDA-core dot product runs out of issue
// slots beyond two tokens (conversions and FMAs per element).  Here every CTA owns 16 output columns, its warps split
// K, the weights go from global memory straight into warp-MMA fragments with coalesced 16-byte loads, and the partial
// tiles of the warps meet in shared memory.  Same epilogue as ub_gemm_tn: scale, bias, activation, gated form
// (act(gate) * up), residual, bf16 or fp32 output.
//
// Replaces in the reference: the matmul of Linear::forward at batch 1 (crates/runtime/src/tensor_core.rs ops_fn::linear,
// crates/runtime/src/simd/matmul/gemm.rs) -- the reference's only generation mode.
#include <stdlib.h>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"

namespace ub {
namespace gemv {


// same formulas as the tcgen05 GEMM's epilogue
__device__ __forceinline__ float act_apply(float v, int act) {
  switch (act) {
    case UB_ACT_SILU: {
      float t;
      asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * v));
      return v * fmaf(0.5f, t, 0.5f);
    }
    case UB_ACT_GELU: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    case UB_ACT_GELU_TANH: {
      const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
      return 0.5f * v * (1.f + tanhf(u));
    }
    case UB_ACT_RELU: return fmaxf(v, 0.f);
    case UB_ACT_RELU2: { const float r = fmaxf(v, 0.f); return r * r; }
    case UB_ACT_QUICK_GELU: return v / (1.f + __expf(-1.702f * v));
    case UB_ACT_SIGMOID: return 1.f / (1.f + __expf(-v));
    case UB_ACT_TANH: return tanhf(v);
    case UB_ACT_SOFTPLUS: return v > 20.f ? v : log1pf(__expf(v));
    default: return v;
  }
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One CTA per tile of 16 output columns (gated form: the 16 gate rows and their 16 up rows); its NW warps split K.
//
// The dot products run on warp MMAs without shared-memory staging: a sum over k does not care about the order of k, so
// the 16 k-slots of an m16n8k16 step are mapped to memory the way a coalesced 16-byte load delivers them.  Lane
// (g = lane / 4, t = lane % 4) loads the 8 consecutive weights W[row g][kb + 8t ..] and W[row g + 8][kb + 8t ..] (one
// 16-byte load each) and the 8 activations x[token g][kb + 8t ..]; registers 0, 1 of the chunks feed one MMA (slots 2t,
// 2t + 1 and 2t + 8, 2t + 9 on the A side match the same physical k on the B side), registers 2, 3 a second one.  Per
// 32 columns of K a warp issues three 16-byte loads and two MMAs, for any token count up to 8.
// TWO: a second token tile (tokens 8..15): one more activation load and two more MMAs per step and weight tile; the
// weight traffic stays the same.
template <int NW, bool DUAL, bool TWO>
__global__ void __launch_bounds__(NW * 32) gemv_kernel(const UbGemmArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NT = DUAL ? 2 : 1;
  constexpr int U = 4;
  constexpr int MT = TWO ? 16 : 8;
  __shared__ float part[NW][NT][16][MT];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int col0 = blockIdx.x * 16;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x);
  const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(a.w);
  const uint4* wlo[NT];
  const uint4* whi[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int r0 = min(col0 + g, a.N - 1) + n * a.up_row_off;          // clamped rows are computed and dropped
    const int r1 = min(col0 + g + 8, a.N - 1) + n * a.up_row_off;
    wlo[n] = reinterpret_cast<const uint4*>(w + (long long)r0 * a.ldw);
    whi[n] = reinterpret_cast<const uint4*>(w + (long long)r1 * a.ldw);
  }
  const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)min(g, a.M - 1) * a.ldx);
  const uint4* xr2 = reinterpret_cast<const uint4*>(x + (long long)min(g + 8, a.M - 1) * a.ldx);
  const bool has_x = g < a.M, has_x2 = TWO && g + 8 < a.M;
  float acc[NT][2][4], acc2[NT][2][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      acc[n][h][0] = acc[n][h][1] = acc[n][h][2] = acc[n][h][3] = 0.f;
      acc2[n][h][0] = acc2[n][h][1] = acc2[n][h][2] = acc2[n][h][3] = 0.f;
    }
  const int nch = a.K / 8;                          // 16-byte chunks per row
  const int steps = (nch + 3) / 4;                  // k-steps of 4 chunks (32 columns)
  // warp `warp` takes the steps warp, warp + NW, ...: neighbouring warps read neighbouring 64-byte pieces of a row
  for (int s0 = warp; s0 < steps; s0 += NW * U) {
    uint4 lo[U][NT], hi[U][NT], xv[U], xw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = (s0 + u * NW) * 4 + t;
      const bool ok = (s0 + u * NW) < steps && c < nch;
      xv[u] = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        lo[u][n] = make_uint4(0, 0, 0, 0);
        hi[u][n] = make_uint4(0, 0, 0, 0);
        if (ok) {
          lo[u][n] = __ldcs(wlo[n] + c);
          hi[u][n] = __ldcs(whi[n] + c);
        }
      }
      if (ok && has_x) xv[u] = __ldg(xr + c);
      if (TWO) {
        xw[u] = make_uint4(0, 0, 0, 0);
        if (ok && has_x2) xw[u] = __ldg(xr2 + c);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        mma_bf16(acc[n][0], lo[u][n].x, hi[u][n].x, lo[u][n].y, hi[u][n].y, xv[u].x, xv[u].y);
        mma_bf16(acc[n][1], lo[u][n].z, hi[u][n].z, lo[u][n].w, hi[u][n].w, xv[u].z, xv[u].w);
        if (TWO) {
          mma_bf16(acc2[n][0], lo[u][n].x, hi[u][n].x, lo[u][n].y, hi[u][n].y, xw[u].x, xw[u].y);
          mma_bf16(acc2[n][1], lo[u][n].z, hi[u][n].z, lo[u][n].w, hi[u][n].w, xw[u].z, xw[u].w);
        }
      }
    }
  }
  // accumulator layout: c0 (row g, token 2t), c1 (row g, token 2t + 1), c2 (row g + 8, 2t), c3 (row g + 8, 2t + 1)
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    part[warp][n][g][2 * t] = acc[n][0][0] + acc[n][1][0];
    part[warp][n][g][2 * t + 1] = acc[n][0][1] + acc[n][1][1];
    part[warp][n][g + 8][2 * t] = acc[n][0][2] + acc[n][1][2];
    part[warp][n][g + 8][2 * t + 1] = acc[n][0][3] + acc[n][1][3];
    if (TWO) {
      part[warp][n][g][8 + 2 * t] = acc2[n][0][0] + acc2[n][1][0];
      part[warp][n][g][8 + 2 * t + 1] = acc2[n][0][1] + acc2[n][1][1];
      part[warp][n][g + 8][8 + 2 * t] = acc2[n][0][2] + acc2[n][1][2];
      part[warp][n][g + 8][8 + 2 * t + 1] = acc2[n][0][3] + acc2[n][1][3];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 16 * MT; i += NW * 32) {
    const int cidx = i / MT, m = i % MT;
    const int col = col0 + cidx;
    if (col >= a.N || m >= a.M) continue;
    float gsum = 0.f, usum = 0.f;
#pragma unroll
    for (int wq = 0; wq < NW; ++wq) {
      gsum += part[wq][0][cidx][m];
      if (DUAL) usum += part[wq][NT - 1][cidx][m];
    }
    const float sc = a.out_scale != 0.f ? a.out_scale : 1.f;
    gsum *= sc;
    float v;
    if (DUAL) {
      v = act_apply(gsum, a.act) * (usum * sc);
    } else {
      if (a.bias != nullptr) gsum += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.bias)[col]);
      v = act_apply(gsum, a.act);
    }
    if (a.residual != nullptr) v += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.residual)[(long long)m * a.ldr + col]);
    if (a.out_f32) reinterpret_cast<float*>(a.out)[(long long)m * a.ldo + col] = v;
    else reinterpret_cast<__nv_bfloat16*>(a.out)[(long long)m * a.ldo + col] = __float2bfloat16(v);
  }
}

template <bool DUAL, bool TWO>
static int launch(const UbGemmArgs& a, cudaStream_t st, int nw) {
  const int grid = (a.N + 15) / 16;
  cudaError_t e;
  // The number of warps fixes the order in which a column's partial sums are added, so it depends on N and K only:
  // a row gives the same bits whatever the token count of the launch (CUDA-graph steps are padded, eager ones are not).
  if (DUAL && nw > 8) nw = 8;
  switch (nw) {
    case 4: e = ub::launch_pdl(gemv_kernel<4, DUAL, TWO>, dim3(grid), dim3(128), (size_t)0, st, a); break;
    case 8: e = ub::launch_pdl(gemv_kernel<8, DUAL, TWO>, dim3(grid), dim3(256), (size_t)0, st, a); break;
    default: e = ub::launch_pdl(gemv_kernel<DUAL ? 8 : 16, DUAL, TWO>, dim3(grid), dim3(DUAL ? 256 : 512), (size_t)0, st, a); break;
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

}  // namespace gemv
}  // namespace ub

// 1 when ub_gemv can take the problem: at most 16 tokens, 16-byte aligned rows, none of the fused / grouped modes.
extern "C" int ub_gemv_supported(const UbGemmArgs* a) {
  if (a->M < 1 || a->M > 16 || a->N < 1 || a->K < 8 || a->K % 8 != 0) return 0;
  if (a->ldx % 8 != 0 || a->ldw % 8 != 0) return 0;
  if ((reinterpret_cast<uintptr_t>(a->x) & 15) || (reinterpret_cast<uintptr_t>(a->w) & 15)) return 0;
  if (a->rs_world > 0 || a->ag_world > 0 || a->grp_tiles != nullptr) return 0;
  return 1;
}

extern "C" int ub_gemv(const UbGemmArgs* a, void* stream) {
  using namespace ub::gemv;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!ub_gemv_supported(a)) return -2;
  // warps per CTA: enough warps on the device to keep its copy engines busy (about 16 per SM), at least two k-steps each
  const int tiles = (a->N + 15) / 16;
  const int steps = (a->K / 8 + 3) / 4;
  int nw = 4;
  while (nw < 16 && tiles * nw < 148 * 16 && steps >= 4 * nw) nw <<= 1;
  if (a->dual) return a->M <= 8 ? launch<true, false>(*a, st, nw) : launch<true, true>(*a, st, nw);
  return a->M <= 8 ? launch<false, false>(*a, st, nw) : launch<false, true>(*a, st, nw);
}
