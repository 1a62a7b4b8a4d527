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
// Chunked form of all scans below (long prefills): the sequence is cut into chunks of CL steps that run in parallel.
//   pass 1 (mode 1, one grid.z slice per chunk): every chunk runs from a ZERO state and writes only its summary -- the
//           end state Q and what the chunk does to an incoming state (for these recurrences a per-element factor P);
//   carry  : one thread per state element walks the chunks in order, h <- P_c * h + Q_c, and leaves in the place of Q_c
//           the state that ENTERS chunk c (a handful of steps: L / CL);
//   pass 2 (mode 2): every chunk runs again from its entering state and writes the outputs; the last one stores the
//           final state.
// The sequential depth drops from L to CL + L / CL at the price of reading the inputs twice.  mode 0 is the plain
// single-pass scan (decode steps and short prompts).  The workspace is the caller's.
template <int NS>
__global__ void __launch_bounds__(128) selective_scan_kernel(const __nv_bfloat16* __restrict__ u, const __nv_bfloat16* __restrict__ delta,
                                                             const float* __restrict__ A, const __nv_bfloat16* __restrict__ Bm,
                                                             const __nv_bfloat16* __restrict__ Cm, const float* __restrict__ Dv,
                                                             const __nv_bfloat16* __restrict__ z, __nv_bfloat16* __restrict__ out,
                                                             float* __restrict__ state, int L, int Dm, int delta_softplus,
                                                             int CL, int mode, float* __restrict__ ws) {
  constexpr int CH = 128 / NS;                  // channels per block
  const int n = threadIdx.x % NS;
  const int d = blockIdx.x * CH + threadIdx.x / NS;
  const int b = blockIdx.y;
  if (d >= Dm) return;                          // whole NS-lane groups leave together
  const int chunk = blockIdx.z, NC = gridDim.z;
  const int l0 = mode == 0 ? 0 : chunk * CL, l1 = mode == 0 ? L : min(L, l0 + CL);
  // workspace: Q / entering states [B][NC][Dm][NS], then the chunks' sums of dt [B][NC][Dm]
  float* wq = ws + (((long long)b * NC + chunk) * Dm + d) * NS + n;
  float* wdt = ws + (long long)gridDim.y * NC * Dm * NS + ((long long)b * NC + chunk) * Dm + d;
  const float a = A[d * NS + n];
  const float dskip = Dv != nullptr ? Dv[d] : 0.f;
  float h = 0.f;
  if (mode == 0) h = state != nullptr ? state[((long long)b * Dm + d) * NS + n] : 0.f;
  else if (mode == 2) h = *wq;
  float sdt = 0.f;
  const long long base = (long long)b * L;
#pragma unroll 4
  for (int l = l0; l < l1; ++l) {
    const float uu = b2f(u[(base + l) * Dm + d]);
    float dt = b2f(delta[(base + l) * Dm + d]);
    if (delta_softplus) dt = softplus_f(dt);
    const float bn = b2f(Bm[(base + l) * NS + n]);
    h = __expf(dt * a) * h + dt * bn * uu;
    if (mode == 1) { sdt += dt; continue; }
    const float cn = b2f(Cm[(base + l) * NS + n]);
    float y = h * cn;
#pragma unroll
    for (int o = NS / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o, NS);
    if (n == 0) {
      y += dskip * uu;
      if (z != nullptr) y *= silu_f(b2f(z[(base + l) * Dm + d]));
      out[(base + l) * Dm + d] = __float2bfloat16(y);
    }
  }
  if (mode == 1) {
    *wq = h;
    if (n == 0) *wdt = sdt;
  } else if (state != nullptr && (mode == 0 || chunk == NC - 1)) {
    state[((long long)b * Dm + d) * NS + n] = h;
  }
}

// carry of the selective scan: element (b, d, n); P_c = exp(A[d,n] * sum of dt over chunk c)
__global__ void __launch_bounds__(256) selective_scan_carry_kernel(const float* __restrict__ A, const float* __restrict__ state,
                                                                   float* __restrict__ ws, int Bn, int NC, int Dm, int NS) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (long long)Bn * Dm * NS) return;
  const int n = int(e % NS), d = int((e / NS) % Dm), b = int(e / ((long long)NS * Dm));
  const float a = A[d * NS + n];
  float h = state != nullptr ? state[e] : 0.f;
  const float* wdt = ws + (long long)Bn * NC * Dm * NS;
  for (int c = 0; c < NC; ++c) {
    float* q = ws + (((long long)b * NC + c) * Dm + d) * NS + n;
    const float qc = *q;
    *q = h;
    h = __expf(a * wdt[((long long)b * NC + c) * Dm + d]) * h + qc;
  }
}

// ---------------------------------------------------------------------------------------------
// K17 diagonal linear recurrence h = a*h + (one_minus ? (1-a) : 1) * x.   a: [C] (a_stride_l = 0) or [B, L, C].
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) linear_recurrence_kernel(const float* __restrict__ a, int a_per_step,
                                                                const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                                float* __restrict__ state, int L, int C, int one_minus,
                                                                int CL, int mode, float* __restrict__ ws) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.y, chunk = blockIdx.z, NC = gridDim.z;
  const int l0 = mode == 0 ? 0 : chunk * CL, l1 = mode == 0 ? L : min(L, l0 + CL);
  // workspace: Q / entering states [B][NC][C], then the chunks' decay products [B][NC][C]
  float* wq = ws + ((long long)b * NC + chunk) * C + c;
  float* wp = ws + (long long)gridDim.y * NC * C + ((long long)b * NC + chunk) * C + c;
  float h = 0.f, prod = 1.f;
  if (mode == 0) h = state != nullptr ? state[(long long)b * C + c] : 0.f;
  else if (mode == 2) h = *wq;
  const long long base = (long long)b * L;
  const float a0 = a_per_step ? 0.f : a[c];
#pragma unroll 4
  for (int l = l0; l < l1; ++l) {
    const float av = a_per_step ? a[(base + l) * C + c] : a0;
    const float xv = b2f(x[(base + l) * C + c]);
    h = av * h + (one_minus ? (1.f - av) : 1.f) * xv;
    if (mode == 1) prod *= av;
    else out[(base + l) * C + c] = __float2bfloat16(h);
  }
  if (mode == 1) {
    *wq = h;
    *wp = prod;
  } else if (state != nullptr && (mode == 0 || chunk == NC - 1)) {
    state[(long long)b * C + c] = h;
  }
}

// carry for recurrences whose chunk summary is (factor P, end state Q) per state element: n_state elements per
// (batch, chunk) in `ws`, the factors behind them at `p_off`; `p_stride_div` maps a state element to its factor
// (1: one factor per element; Dh: one factor per row of a Dh x Dh state, shared by its Dh columns).
__global__ void __launch_bounds__(256) diag_carry_kernel(const float* __restrict__ state, float* __restrict__ ws, int Bn, int NC,
                                                         long long n_state, long long p_off, long long n_factor, int p_div) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (long long)Bn * n_state) return;
  const long long b = e / n_state, i = e % n_state;
  float h = state != nullptr ? state[e] : 0.f;
  for (int c = 0; c < NC; ++c) {
    float* q = ws + (b * NC + c) * n_state + i;
    const float qc = *q;
    *q = h;
    h = ws[p_off + (b * NC + c) * n_factor + i / p_div] * h + qc;
  }
}

// ---------------------------------------------------------------------------------------------
// K16a WKV-4 with the running-maximum form (aa, bb, pp): equal to the plain (num, den) recurrence wherever that one
// does not overflow.  state: [B, 3, C] = aa, bb, pp; a fresh sequence starts from (0, 0, -1e38).
//   w[c] = -exp(time_decay[c]) (<= 0), u[c] = time_first[c]
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) wkv4_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                                   const float* __restrict__ w, const float* __restrict__ u,
                                                   __nv_bfloat16* __restrict__ out, float* __restrict__ state, int L, int C,
                                                   int CL, int mode, float* __restrict__ ws) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.y, chunk = blockIdx.z, NC = gridDim.z;
  const int l0 = mode == 0 ? 0 : chunk * CL, l1 = mode == 0 ? L : min(L, l0 + CL);
  float* wsc = ws + (((long long)b * NC + chunk) * 3) * C + c;      // workspace: (aa, bb, pp) per (batch, chunk, channel)
  float aa = 0.f, bb = 0.f, pp = -1e38f;
  if (mode == 0 && state != nullptr) {
    aa = state[((long long)b * 3 + 0) * C + c];
    bb = state[((long long)b * 3 + 1) * C + c];
    pp = state[((long long)b * 3 + 2) * C + c];
  } else if (mode == 2) {
    aa = wsc[0]; bb = wsc[C]; pp = wsc[2 * C];
  }
  const float wc = w[c], uc = u[c];
  const long long base = (long long)b * L;
#pragma unroll 2
  for (int l = l0; l < l1; ++l) {
    const float kk = b2f(k[(base + l) * C + c]), vv = b2f(v[(base + l) * C + c]);
    float ww = uc + kk;
    float p = fmaxf(pp, ww);
    float e1 = __expf(pp - p), e2 = __expf(ww - p);
    if (mode != 1) out[(base + l) * C + c] = __float2bfloat16((e1 * aa + e2 * vv) / (e1 * bb + e2));
    ww = pp + wc;
    p = fmaxf(ww, kk);
    e1 = __expf(ww - p);
    e2 = __expf(kk - p);
    aa = e1 * aa + e2 * vv;
    bb = e1 * bb + e2;
    pp = p;
  }
  if (mode == 1) {
    wsc[0] = aa; wsc[C] = bb; wsc[2 * C] = pp;
  } else if (state != nullptr && (mode == 0 || chunk == NC - 1)) {
    state[((long long)b * 3 + 0) * C + c] = aa;
    state[((long long)b * 3 + 1) * C + c] = bb;
    state[((long long)b * 3 + 2) * C + c] = pp;
  }
}

// carry of WKV-4: (aa, bb, pp) stand for the true sums aa * e^pp and bb * e^pp, which decay by e^(w * steps) over a
// chunk; an entering state is pushed through chunk c by adding w * len_c to its exponent and merging with the chunk's
// own sums under a common exponent.
__global__ void __launch_bounds__(256) wkv4_carry_kernel(const float* __restrict__ w, const float* __restrict__ state,
                                                         float* __restrict__ ws, int Bn, int NC, int C, int L, int CL) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (long long)Bn * C) return;
  const int c = int(e % C), b = int(e / C);
  float aa = 0.f, bb = 0.f, pp = -1e38f;
  if (state != nullptr) {
    aa = state[((long long)b * 3 + 0) * C + c];
    bb = state[((long long)b * 3 + 1) * C + c];
    pp = state[((long long)b * 3 + 2) * C + c];
  }
  const float wc = w[c];
  for (int ch = 0; ch < NC; ++ch) {
    float* q = ws + (((long long)b * NC + ch) * 3) * C + c;
    const float qa = q[0], qb = q[C], qp = q[2 * C];
    q[0] = aa; q[C] = bb; q[2 * C] = pp;
    const int len = min(L, (ch + 1) * CL) - ch * CL;
    const float pin = pp + wc * (float)len;
    const float p = fmaxf(pin, qp);
    const float e1 = __expf(pin - p), e2 = __expf(qp - p);
    aa = e1 * aa + e2 * qa;
    bb = e1 * bb + e2 * qb;
    pp = p;
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
                                                  float* __restrict__ state, int L, int H, int CL, int mode,
                                                  float* __restrict__ ws) {
  __shared__ float rs[DH], ks[DH], ws_[DH], us[DH];
  const int b = blockIdx.y, h = blockIdx.x, j = threadIdx.x;
  const int chunk = blockIdx.z, NC = gridDim.z;
  const int l0 = mode == 0 ? 0 : chunk * CL, l1 = mode == 0 ? L : min(L, l0 + CL);
  const int C = H * DH;
  // workspace: Q / entering states [B][NC][H][DH][DH], then the chunks' decay products per state row [B][NC][H][DH]
  float* wq = ws + (((long long)b * NC + chunk) * H + h) * DH * DH;
  float* wp = ws + (long long)gridDim.y * NC * H * DH * DH + (((long long)b * NC + chunk) * H + h) * DH;
  float S[DH];
  float* st = state != nullptr ? state + ((long long)b * H + h) * DH * DH : nullptr;
#pragma unroll
  for (int i = 0; i < DH; ++i) S[i] = mode == 0 ? (st != nullptr ? st[i * DH + j] : 0.f) : (mode == 2 ? wq[i * DH + j] : 0.f);
  us[j] = u[h * DH + j];
  float prod = 1.f;                             // mode 1: thread j tracks the decay product of state ROW j
  const long long base = (long long)b * L;
  for (int l = l0; l < l1; ++l) {
    const long long o = (base + l) * C + h * DH + j;
    __syncthreads();
    rs[j] = b2f(r[o]);
    ks[j] = b2f(k[o]);
    const float dec = __expf(-__expf(w[o]));
    ws_[j] = dec;
    prod *= dec;
    __syncthreads();
    const float vj = b2f(v[o]);
    float y = 0.f;
#pragma unroll
    for (int i = 0; i < DH; ++i) {
      const float kv = ks[i] * vj;
      y += rs[i] * (S[i] + us[i] * kv);
      S[i] = S[i] * ws_[i] + kv;
    }
    if (mode != 1) out[o] = __float2bfloat16(y);
  }
  if (mode == 1) {
#pragma unroll
    for (int i = 0; i < DH; ++i) wq[i * DH + j] = S[i];
    wp[j] = prod;
  } else if (st != nullptr && (mode == 0 || chunk == NC - 1)) {
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

// Chunk length of the chunked scans and the sequence length from which they are used.
static const int UB_SCAN_CHUNK = 256;

extern "C" int ub_scan_chunks(int L) { return L >= 4 * UB_SCAN_CHUNK ? (L + UB_SCAN_CHUNK - 1) / UB_SCAN_CHUNK : 1; }

/* Workspace (fp32 elements) of the chunked form of a scan, 0 when the sequence is short enough for the single pass.
   kind: 0 selective scan (n = Dm, m = Ns), 1 linear recurrence (n = C), 2 WKV-4 (n = C), 3 WKV-6 (n = H, m = Dh). */
extern "C" long long ub_scan_workspace_floats(int kind, int B, int L, int n, int m) {
  const long long nc = ub_scan_chunks(L);
  if (nc <= 1) return 0;
  switch (kind) {
    case 0: return (long long)B * nc * n * (m + 1);
    case 1: return (long long)B * nc * n * 2;
    case 2: return (long long)B * nc * n * 3;
    case 3: return (long long)B * nc * n * ((long long)m * m + m);
    default: return 0;
  }
}

extern "C" int ub_selective_scan(const void* u, const void* delta, const float* A, const void* Bm, const void* Cm, const float* Dv,
                                 const void* z, void* out, float* state, int B, int L, int Dm, int Ns, int delta_softplus,
                                 float* workspace, void* stream) {
  if (B <= 0 || L <= 0 || Dm <= 0) return 0;
  if (B > 65535) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int nc = workspace != nullptr ? ub_scan_chunks(L) : 1;
#define UB_SCAN(NS, GZ, MODE)                                                                                         \
  ub::selective_scan_kernel<NS><<<dim3((Dm + 128 / NS - 1) / (128 / NS), B, GZ), 128, 0, st>>>(                       \
      reinterpret_cast<const bf*>(u), reinterpret_cast<const bf*>(delta), A, reinterpret_cast<const bf*>(Bm),         \
      reinterpret_cast<const bf*>(Cm), Dv, reinterpret_cast<const bf*>(z), reinterpret_cast<bf*>(out), state, L, Dm,  \
      delta_softplus, UB_SCAN_CHUNK, MODE, workspace)
#define UB_SCAN_ALL(NS)                                                                                               \
  if (nc <= 1) { UB_SCAN(NS, 1, 0); }                                                                                 \
  else {                                                                                                              \
    UB_SCAN(NS, nc, 1);                                                                                               \
    ub::selective_scan_carry_kernel<<<(unsigned)(((long long)B * Dm * NS + 255) / 256), 256, 0, st>>>(A, state, workspace, B, nc, Dm, NS); \
    UB_SCAN(NS, nc, 2);                                                                                               \
  }
  switch (Ns) {
    case 4: UB_SCAN_ALL(4); break;
    case 8: UB_SCAN_ALL(8); break;
    case 16: UB_SCAN_ALL(16); break;
    case 32: UB_SCAN_ALL(32); break;
    default: return -2;
  }
#undef UB_SCAN_ALL
#undef UB_SCAN
  return ub::last_err();
}

extern "C" int ub_linear_recurrence(const float* a, int a_per_step, const void* x, void* out, float* state, int B, int L, int C,
                                    int one_minus, float* workspace, void* stream) {
  if (B <= 0 || L <= 0 || C <= 0) return 0;
  if (B > 65535) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int nc = workspace != nullptr ? ub_scan_chunks(L) : 1;
  auto launch = [&](int gz, int mode) {
    ub::linear_recurrence_kernel<<<dim3((C + 127) / 128, B, gz), 128, 0, st>>>(
        a, a_per_step, reinterpret_cast<const bf*>(x), reinterpret_cast<bf*>(out), state, L, C, one_minus, UB_SCAN_CHUNK, mode, workspace);
  };
  if (nc <= 1) {
    launch(1, 0);
  } else {
    launch(nc, 1);
    ub::diag_carry_kernel<<<(unsigned)(((long long)B * C + 255) / 256), 256, 0, st>>>(state, workspace, B, nc, C, (long long)B * nc * C, C, 1);
    launch(nc, 2);
  }
  return ub::last_err();
}

extern "C" int ub_wkv4(const void* k, const void* v, const float* w, const float* u, void* out, float* state, int B, int L, int C,
                       float* workspace, void* stream) {
  if (B <= 0 || L <= 0 || C <= 0) return 0;
  if (B > 65535) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int nc = workspace != nullptr ? ub_scan_chunks(L) : 1;
  auto launch = [&](int gz, int mode) {
    ub::wkv4_kernel<<<dim3((C + 127) / 128, B, gz), 128, 0, st>>>(reinterpret_cast<const bf*>(k), reinterpret_cast<const bf*>(v), w, u,
                                                                 reinterpret_cast<bf*>(out), state, L, C, UB_SCAN_CHUNK, mode, workspace);
  };
  if (nc <= 1) {
    launch(1, 0);
  } else {
    launch(nc, 1);
    ub::wkv4_carry_kernel<<<(unsigned)(((long long)B * C + 255) / 256), 256, 0, st>>>(w, state, workspace, B, nc, C, L, UB_SCAN_CHUNK);
    launch(nc, 2);
  }
  return ub::last_err();
}

extern "C" int ub_wkv6(const void* r, const void* k, const void* v, const float* w, const float* u, void* out, float* state, int B,
                       int L, int H, int Dh, float* workspace, void* stream) {
  if (B <= 0 || L <= 0 || H <= 0) return 0;
  if (B > 65535) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int nc = workspace != nullptr ? ub_scan_chunks(L) : 1;
  auto launch = [&](int gz, int mode) {
    if (Dh == 64)
      ub::wkv6_kernel<64><<<dim3(H, B, gz), 64, 0, st>>>(reinterpret_cast<const bf*>(r), reinterpret_cast<const bf*>(k),
                                                         reinterpret_cast<const bf*>(v), w, u, reinterpret_cast<bf*>(out), state, L, H,
                                                         UB_SCAN_CHUNK, mode, workspace);
    else
      ub::wkv6_kernel<32><<<dim3(H, B, gz), 32, 0, st>>>(reinterpret_cast<const bf*>(r), reinterpret_cast<const bf*>(k),
                                                         reinterpret_cast<const bf*>(v), w, u, reinterpret_cast<bf*>(out), state, L, H,
                                                         UB_SCAN_CHUNK, mode, workspace);
  };
  if (Dh != 64 && Dh != 32) return -2;
  if (nc <= 1) {
    launch(1, 0);
  } else {
    launch(nc, 1);
    const long long n_state = (long long)H * Dh * Dh;
    ub::diag_carry_kernel<<<(unsigned)(((long long)B * n_state + 255) / 256), 256, 0, st>>>(
        state, workspace, B, nc, n_state, (long long)B * nc * n_state, (long long)H * Dh, Dh);
    launch(nc, 2);
  }
  return ub::last_err();
}
