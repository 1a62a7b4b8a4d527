// K9 / K10: the long tail of memory-bound element-wise ops, all with 16-byte vector access:
// embedding gather (+ scale for Gemma / MiniCPM), act(gate) * up for un-fused MLPs, unary
// activations (gelu, quick-gelu, relu^2, sigmoid, tanh, softplus, exp, scale), scaled add, and
// row-wise L2 normalisation.
//
// Replaces in the reference: ops_fn::embedding / gelu / silu / sigmoid / tanh / exp / scale / add /
// normalize (crates/runtime/src/tensor_core.rs:1038-1060, 1083-1159, 1274-1297, 1089-1110),
// quick-GELU (models_v2/clip.rs:1031), ReLU^2 (models_v2/rwkv4.rs:617-619), softplus
// (models_v2/mamba.rs:964-971) and the SIMD silu / mul / add (simd/arch/avx2.rs:326-349, neon.rs:214-417).
#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"

namespace ub {

__device__ __forceinline__ float act_fn(float v, int act) {
  switch (act) {
    case UB_ACT_SILU: return v / (1.f + __expf(-v));
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
    case UB_ACT_EXP: return __expf(v);
    default: return v;
  }
}

__global__ void embed_gather_kernel(const int* ids, const __nv_bfloat16* table, __nv_bfloat16* out, int T, int H,
                                    int V, float scale, int* err) {
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) set_err(err, ERR_BOUNDS, t);
    id = 0;
  }
  const __nv_bfloat16* src = table + (long long)id * H;
  __nv_bfloat16* dst = out + (long long)t * H;
  if (H % 8 == 0) {
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
      uint4 v = *reinterpret_cast<const uint4*>(src + c * 8);
      if (scale != 1.f) {
        uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) w[e] = pack_bf16x2(bf16_lo(w[e]) * scale, bf16_hi(w[e]) * scale);
      }
      *reinterpret_cast<uint4*>(dst + c * 8) = v;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = __float2bfloat16(__bfloat162float(src[i]) * scale);
  }
}

__global__ void act_mul_kernel(const __nv_bfloat16* gu, __nv_bfloat16* out, long long T, int I, int act) {
  const long long t = blockIdx.x;
  const __nv_bfloat16* g = gu + t * 2 * I;
  const __nv_bfloat16* u = g + I;
  __nv_bfloat16* o = out + t * I;
  if (I % 8 == 0) {
    for (int c = threadIdx.x; c < I / 8; c += blockDim.x) {
      const uint4 gv = *reinterpret_cast<const uint4*>(g + c * 8);
      const uint4 uv = *reinterpret_cast<const uint4*>(u + c * 8);
      const uint32_t* a = reinterpret_cast<const uint32_t*>(&gv);
      const uint32_t* b = reinterpret_cast<const uint32_t*>(&uv);
      uint32_t r[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        r[e] = pack_bf16x2(act_fn(bf16_lo(a[e]), act) * bf16_lo(b[e]), act_fn(bf16_hi(a[e]), act) * bf16_hi(b[e]));
      *reinterpret_cast<uint4*>(o + c * 8) = make_uint4(r[0], r[1], r[2], r[3]);
    }
  } else {
    for (int i = threadIdx.x; i < I; i += blockDim.x)
      o[i] = __float2bfloat16(act_fn(__bfloat162float(g[i]), act) * __bfloat162float(u[i]));
  }
}

__global__ void eltwise_kernel(const __nv_bfloat16* x, __nv_bfloat16* out, long long n, int act, float alpha) {
  const long long nv = n / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < nv; c += stride) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + c * 8);
    const uint32_t* a = reinterpret_cast<const uint32_t*>(&v);
    uint32_t r[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      r[e] = pack_bf16x2(act_fn(bf16_lo(a[e]) * alpha, act), act_fn(bf16_hi(a[e]) * alpha, act));
    *reinterpret_cast<uint4*>(out + c * 8) = make_uint4(r[0], r[1], r[2], r[3]);
  }
  for (long long i = nv * 8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = __float2bfloat16(act_fn(__bfloat162float(x[i]) * alpha, act));
}

__global__ void add_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out, long long n, float sa,
                           float sb) {
  const long long nv = n / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < nv; c += stride) {
    const uint4 va = *reinterpret_cast<const uint4*>(a + c * 8);
    const uint4 vb = *reinterpret_cast<const uint4*>(b + c * 8);
    const uint32_t* x = reinterpret_cast<const uint32_t*>(&va);
    const uint32_t* y = reinterpret_cast<const uint32_t*>(&vb);
    uint32_t r[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      r[e] = pack_bf16x2(bf16_lo(x[e]) * sa + bf16_lo(y[e]) * sb, bf16_hi(x[e]) * sa + bf16_hi(y[e]) * sb);
    *reinterpret_cast<uint4*>(out + c * 8) = make_uint4(r[0], r[1], r[2], r[3]);
  }
  for (long long i = nv * 8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = __float2bfloat16(__bfloat162float(a[i]) * sa + __bfloat162float(b[i]) * sb);
}

__global__ void l2norm_kernel(const __nv_bfloat16* x, __nv_bfloat16* out, int H, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) { const float v = __bfloat162float(x[t * H + i]); s += v * v; }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = v;
  }
  __syncthreads();
  const float inv = 1.f / fmaxf(sqrtf(red[0]), eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[t * H + i] = __float2bfloat16(__bfloat162float(x[t * H + i]) * inv);
}

static inline int last_err() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
static inline int grid_for(long long n) {
  long long g = (n / 8 + 255) / 256;
  if (g < 1) g = 1;
  if (g > 148 * 16) g = 148 * 16;
  return (int)g;
}

// Row softmax over the last dimension (bf16 in / out, fp32 inside): one warp per row, three passes over the row kept
// in L1 / L2.  Replaces ops_fn::softmax (crates/runtime/src/tensor_core.rs:1022-1036) and the SIMD softmax
// (simd/arch/avx2.rs:246-307) outside attention, the router and the sampler, which have it fused.
__global__ void __launch_bounds__(256) softmax_rows_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                           long long rows, int n) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * n;
  float mx = -3.4e38f;
  for (int i = lane; i < n; i += 32) mx = fmaxf(mx, __bfloat162float(xr[i]));
  mx = warp_max(mx);
  float sum = 0.f;
  for (int i = lane; i < n; i += 32) sum += __expf(__bfloat162float(xr[i]) - mx);
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  for (int i = lane; i < n; i += 32) out[row * n + i] = __float2bfloat16(__expf(__bfloat162float(xr[i]) - mx) * inv);
}

}  // namespace ub

extern "C" int ub_embed_gather(const int* ids, const void* table, void* out, int T, int H, int V, float scale,
                               int* err, void* st) {
  if (T <= 0) return 0;
  ub::embed_gather_kernel<<<T, 256, 0, (cudaStream_t)st>>>(ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, T,
                                                            H, V, scale, err);
  return ub::last_err();
}
extern "C" int ub_act_mul(const void* gate_up, void* out, long long T, int I, int act, void* st) {
  if (T <= 0) return 0;
  ub::act_mul_kernel<<<(unsigned)T, 256, 0, (cudaStream_t)st>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, T,
                                                                I, act);
  return ub::last_err();
}
extern "C" int ub_eltwise(const void* x, void* out, long long n, int act, float alpha, void* st) {
  if (n <= 0) return 0;
  ub::eltwise_kernel<<<ub::grid_for(n), 256, 0, (cudaStream_t)st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n,
                                                                    act, alpha);
  return ub::last_err();
}
extern "C" int ub_add(const void* a, const void* b, void* out, long long n, float sa, float sb, void* st) {
  if (n <= 0) return 0;
  ub::add_kernel<<<ub::grid_for(n), 256, 0, (cudaStream_t)st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                                (__nv_bfloat16*)out, n, sa, sb);
  return ub::last_err();
}
extern "C" int ub_l2_normalize(const void* x, void* out, int T, int H, float eps, void* st) {
  if (T <= 0) return 0;
  ub::l2norm_kernel<<<T, 256, 0, (cudaStream_t)st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, H, eps);
  return ub::last_err();
}

extern "C" int ub_softmax_rows(const void* x, void* out, long long rows, int n, void* stream) {
  if (rows <= 0 || n <= 0) return 0;
  ub::softmax_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(out), rows, n);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
