// K14-K17, K15: recurrences of the O(1)-state architectures.  All of them stream [B, L, C]-shaped bf16 activations
// once and keep the recurrent state in registers (fp32); the state tensor in global memory is read at the start and
// written at the end of a call, so prefill (L = prompt length) and decode (L = 1) are the same entry points.
//
// Reference math: selective scan crates/runtime/src/models_v2/mamba.rs:745-888 (per-timestep host loop), depthwise
// causal conv :632-742, WKV-4 rwkv4.rs:468-529, WKV-6 rwkv6.rs:483-553, simplified RG-LRU
// recurrent_gemma.rs:624-690.  Unlike the reference, prefill leaves the state behind, so decode can continue from it.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../include/unillm_b200.h"

namespace ub {

__device__ __forceinline__ float b2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(__expf(v)); }

// ---------------------------------------------------------------------------------------------
// K15 depthwise causal conv1d, channel-last.  out[b,l,c] = act(bias[c] + sum_k w[c,k] * xin[b, l-(Kw-1)+k, c]) where
// xin is the `state` rows (the Kw-1 inputs before this call) followed by x.
// ---------------------------------------------------------------------------------------------
constexpr int CONV_MAX_K = 8;

__global__ void __launch_bounds__(256) dwconv1d_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                       const float* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                                       const __nv_bfloat16* __restrict__ state, int L, int C, int Kw, int act_silu) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.z;
  float wk[CONV_MAX_K];
  for (int k = 0; k < Kw; ++k) wk[k] = w[c * Kw + k];
  const float bv = bias != nullptr ? bias[c] : 0.f;
  const __nv_bfloat16* xb = x + (long long)b * L * C;
  const __nv_bfloat16* sb = state != nullptr ? state + (long long)b * (Kw - 1) * C : nullptr;
  for (int l = blockIdx.y; l < L; l += gridDim.y) {
    float acc = bv;
    for (int k = 0; k < Kw; ++k) {
      const int src = l - (Kw - 1) + k;
      float v = 0.f;
      if (src >= 0) v = b2f(xb[(long long)src * C + c]);
      else if (sb != nullptr) v = b2f(sb[(long long)(src + Kw - 1) * C + c]);
      acc += wk[k] * v;
    }
    out[((long long)b * L + l) * C + c] = __float2bfloat16(act_silu ? silu_f(acc) : acc);
  }
}

// state <- last Kw-1 rows of [state ; x]
__global__ void __launch_bounds__(256) dwconv1d_state_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ state,
                                                             int L, int C, int Kw) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.y;
  __nv_bfloat16 keep[CONV_MAX_K];
  __nv_bfloat16* sb = state + (long long)b * (Kw - 1) * C;
  const __nv_bfloat16* xb = x + (long long)b * L * C;
  for (int j = 0; j < Kw - 1; ++j) {
    const int src = L + j;                      // index into [state(Kw-1) ; x(L)] of the j-th kept row
    keep[j] = src < Kw - 1 ? sb[(long long)src * C + c] : xb[(long long)(src - (Kw - 1)) * C + c];
  }
  for (int j = 0; j < Kw - 1; ++j) sb[(long long)j * C + c] = keep[j];
}

// ---------------------------------------------------------------------------------------------
// K14 selective scan.  NS lanes cooperate on one channel, each owning one state element.
//   dt = softplus?(delta);  h[n] = exp(dt*A[d,n]) * h[n] + dt * B[l,n] * u;  y = sum_n h[n]*C[l,n] + D[d]*u;  y *= silu(z)
// ---------------------------------------------------------------------------------------------
template <int NS>
__global__ void __launch_bounds__(128) selective_scan_kernel(const __nv_bfloat16* __restrict__ u, const __nv_bfloat16* __restrict__ delta,
                                                             const float* __restrict__ A, const __nv_bfloat16* __restrict__ Bm,
                                                             const __nv_bfloat16* __restrict__ Cm, const float* __restrict__ Dv,
                                                             const __nv_bfloat16* __restrict__ z, __nv_bfloat16* __restrict__ out,
                                                             float* __restrict__ state, int L, int Dm, int delta_softplus) {
  constexpr int CH = 128 / NS;                  // channels per block
  const int n = threadIdx.x % NS;
  const int d = blockIdx.x * CH + threadIdx.x / NS;
  const int b = blockIdx.y;
  if (d >= Dm) return;                          // whole NS-lane groups leave together
  const float a = A[d * NS + n];
  const float dskip = Dv != nullptr ? Dv[d] : 0.f;
  float h = state != nullptr ? state[((long long)b * Dm + d) * NS + n] : 0.f;
  const long long base = (long long)b * L;
#pragma unroll 4
  for (int l = 0; l < L; ++l) {
    const float uu = b2f(u[(base + l) * Dm + d]);
    float dt = b2f(delta[(base + l) * Dm + d]);
    if (delta_softplus) dt = softplus_f(dt);
    const float bn = b2f(Bm[(base + l) * NS + n]);
    const float cn = b2f(Cm[(base + l) * NS + n]);
    h = __expf(dt * a) * h + dt * bn * uu;
    float y = h * cn;
#pragma unroll
    for (int o = NS / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o, NS);
    if (n == 0) {
      y += dskip * uu;
      if (z != nullptr) y *= silu_f(b2f(z[(base + l) * Dm + d]));
      out[(base + l) * Dm + d] = __float2bfloat16(y);
    }
  }
  if (state != nullptr) state[((long long)b * Dm + d) * NS + n] = h;
}

// ---------------------------------------------------------------------------------------------
// K17 diagonal linear recurrence h = a*h + (one_minus ? (1-a) : 1) * x.   a: [C] (a_stride_l = 0) or [B, L, C].
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) linear_recurrence_kernel(const float* __restrict__ a, int a_per_step,
                                                                const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                                float* __restrict__ state, int L, int C, int one_minus) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.y;
  float h = state != nullptr ? state[(long long)b * C + c] : 0.f;
  const long long base = (long long)b * L;
  const float a0 = a_per_step ? 0.f : a[c];
#pragma unroll 4
  for (int l = 0; l < L; ++l) {
    const float av = a_per_step ? a[(base + l) * C + c] : a0;
    const float xv = b2f(x[(base + l) * C + c]);
    h = av * h + (one_minus ? (1.f - av) : 1.f) * xv;
    out[(base + l) * C + c] = __float2bfloat16(h);
  }
  if (state != nullptr) state[(long long)b * C + c] = h;
}

// ---------------------------------------------------------------------------------------------
// K16a WKV-4 with the running-maximum form (aa, bb, pp): equal to the plain (num, den) recurrence wherever that one
// does not overflow.  state: [B, 3, C] = aa, bb, pp; a fresh sequence starts from (0, 0, -1e38).
//   w[c] = -exp(time_decay[c]) (<= 0), u[c] = time_first[c]
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) wkv4_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                                   const float* __restrict__ w, const float* __restrict__ u,
                                                   __nv_bfloat16* __restrict__ out, float* __restrict__ state, int L, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.y;
  float aa = 0.f, bb = 0.f, pp = -1e38f;
  if (state != nullptr) {
    aa = state[((long long)b * 3 + 0) * C + c];
    bb = state[((long long)b * 3 + 1) * C + c];
    pp = state[((long long)b * 3 + 2) * C + c];
  }
  const float wc = w[c], uc = u[c];
  const long long base = (long long)b * L;
#pragma unroll 2
  for (int l = 0; l < L; ++l) {
    const float kk = b2f(k[(base + l) * C + c]), vv = b2f(v[(base + l) * C + c]);
    float ww = uc + kk;
    float p = fmaxf(pp, ww);
    float e1 = __expf(pp - p), e2 = __expf(ww - p);
    out[(base + l) * C + c] = __float2bfloat16((e1 * aa + e2 * vv) / (e1 * bb + e2));
    ww = pp + wc;
    p = fmaxf(ww, kk);
    e1 = __expf(ww - p);
    e2 = __expf(kk - p);
    aa = e1 * aa + e2 * vv;
    bb = e1 * bb + e2;
    pp = p;
  }
  if (state != nullptr) {
    state[((long long)b * 3 + 0) * C + c] = aa;
    state[((long long)b * 3 + 1) * C + c] = bb;
    state[((long long)b * 3 + 2) * C + c] = pp;
  }
}

// ---------------------------------------------------------------------------------------------
// K16b WKV-6.  One CTA per (batch, head), thread j owns column j of the Dh x Dh state.
//   out_t[j] = sum_i r_t[i] * (S[i][j] + u[i] k_t[i] v_t[j]);   S[i][j] = S[i][j] * exp(-exp(w_t[i])) + k_t[i] v_t[j]
// ---------------------------------------------------------------------------------------------
template <int DH>
__global__ void __launch_bounds__(DH) wkv6_kernel(const __nv_bfloat16* __restrict__ r, const __nv_bfloat16* __restrict__ k,
                                                  const __nv_bfloat16* __restrict__ v, const float* __restrict__ w,
                                                  const float* __restrict__ u, __nv_bfloat16* __restrict__ out,
                                                  float* __restrict__ state, int L, int H) {
  __shared__ float rs[DH], ks[DH], ws[DH], us[DH];
  const int b = blockIdx.y, h = blockIdx.x, j = threadIdx.x;
  const int C = H * DH;
  float S[DH];
  float* st = state != nullptr ? state + ((long long)b * H + h) * DH * DH : nullptr;
#pragma unroll
  for (int i = 0; i < DH; ++i) S[i] = st != nullptr ? st[i * DH + j] : 0.f;
  us[j] = u[h * DH + j];
  const long long base = (long long)b * L;
  for (int l = 0; l < L; ++l) {
    const long long o = (base + l) * C + h * DH + j;
    __syncthreads();
    rs[j] = b2f(r[o]);
    ks[j] = b2f(k[o]);
    ws[j] = __expf(-__expf(w[o]));
    __syncthreads();
    const float vj = b2f(v[o]);
    float y = 0.f;
#pragma unroll
    for (int i = 0; i < DH; ++i) {
      const float kv = ks[i] * vj;
      y += rs[i] * (S[i] + us[i] * kv);
      S[i] = S[i] * ws[i] + kv;
    }
    out[o] = __float2bfloat16(y);
  }
  if (st != nullptr) {
#pragma unroll
    for (int i = 0; i < DH; ++i) st[i * DH + j] = S[i];
  }
}

static int last_err() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

}  // namespace ub

using bf = __nv_bfloat16;

extern "C" int ub_causal_dwconv1d(const void* x, const float* w, const float* b, void* out, void* state, int B, int L, int C,
                                  int Kw, int act_silu, int update_state, void* stream) {
  if (B <= 0 || L <= 0 || C <= 0) return 0;
  if (Kw < 1 || Kw > ub::CONV_MAX_K) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int ly = L < 512 ? L : 512;
  dim3 grid((C + 255) / 256, ly, B);
  if (B > 65535) return -3;
  ub::dwconv1d_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const bf*>(x), w, b, reinterpret_cast<bf*>(out),
                                            reinterpret_cast<const bf*>(state), L, C, Kw, act_silu);
  if (state != nullptr && update_state && Kw > 1)
    ub::dwconv1d_state_kernel<<<dim3((C + 255) / 256, B), 256, 0, st>>>(reinterpret_cast<const bf*>(x), reinterpret_cast<bf*>(state), L, C, Kw);
  return ub::last_err();
}

extern "C" int ub_selective_scan(const void* u, const void* delta, const float* A, const void* Bm, const void* Cm, const float* Dv,
                                 const void* z, void* out, float* state, int B, int L, int Dm, int Ns, int delta_softplus,
                                 void* stream) {
  if (B <= 0 || L <= 0 || Dm <= 0) return 0;
  if (B > 65535) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define UB_SCAN(NS)                                                                                                   \
  ub::selective_scan_kernel<NS><<<dim3((Dm + 128 / NS - 1) / (128 / NS), B), 128, 0, st>>>(                           \
      reinterpret_cast<const bf*>(u), reinterpret_cast<const bf*>(delta), A, reinterpret_cast<const bf*>(Bm),         \
      reinterpret_cast<const bf*>(Cm), Dv, reinterpret_cast<const bf*>(z), reinterpret_cast<bf*>(out), state, L, Dm,  \
      delta_softplus)
  switch (Ns) {
    case 4: UB_SCAN(4); break;
    case 8: UB_SCAN(8); break;
    case 16: UB_SCAN(16); break;
    case 32: UB_SCAN(32); break;
    default: return -2;
  }
#undef UB_SCAN
  return ub::last_err();
}

extern "C" int ub_linear_recurrence(const float* a, int a_per_step, const void* x, void* out, float* state, int B, int L, int C,
                                    int one_minus, void* stream) {
  if (B <= 0 || L <= 0 || C <= 0) return 0;
  if (B > 65535) return -3;
  ub::linear_recurrence_kernel<<<dim3((C + 127) / 128, B), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      a, a_per_step, reinterpret_cast<const bf*>(x), reinterpret_cast<bf*>(out), state, L, C, one_minus);
  return ub::last_err();
}

extern "C" int ub_wkv4(const void* k, const void* v, const float* w, const float* u, void* out, float* state, int B, int L, int C,
                       void* stream) {
  if (B <= 0 || L <= 0 || C <= 0) return 0;
  if (B > 65535) return -3;
  ub::wkv4_kernel<<<dim3((C + 127) / 128, B), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const bf*>(k), reinterpret_cast<const bf*>(v), w, u, reinterpret_cast<bf*>(out), state, L, C);
  return ub::last_err();
}

extern "C" int ub_wkv6(const void* r, const void* k, const void* v, const float* w, const float* u, void* out, float* state, int B,
                       int L, int H, int Dh, void* stream) {
  if (B <= 0 || L <= 0 || H <= 0) return 0;
  if (B > 65535) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (Dh == 64)
    ub::wkv6_kernel<64><<<dim3(H, B), 64, 0, st>>>(reinterpret_cast<const bf*>(r), reinterpret_cast<const bf*>(k),
                                                   reinterpret_cast<const bf*>(v), w, u, reinterpret_cast<bf*>(out), state, L, H);
  else if (Dh == 32)
    ub::wkv6_kernel<32><<<dim3(H, B), 32, 0, st>>>(reinterpret_cast<const bf*>(r), reinterpret_cast<const bf*>(k),
                                                   reinterpret_cast<const bf*>(v), w, u, reinterpret_cast<bf*>(out), state, L, H);
  else
    return -2;
  return ub::last_err();
}
