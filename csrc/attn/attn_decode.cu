// K4: paged decode attention (one query token per sequence), split-KV, GQA-aware.
//
// One CTA handles (sequence, kv head, split).  All G = Hq/Hkv query heads that share the kv head
// are processed together, so each K/V byte is fetched from HBM exactly once per step.  A group of
// D/8 lanes owns one token: each lane loads one 16-byte chunk of the K row, partial dots are
// reduced with xor-shuffles, and the same lanes own the matching 16-byte chunk of the output
// accumulator for the P*V pass.  K and V rows reach the lanes through a three-stage cp.async pipeline in shared
// memory (tiles of 4 * (32 / (D/8)) * 4 tokens gathered page by page through the block table), so two tiles are
// always in flight while one is consumed.  Four tokens per lane group are processed per iteration and the
// online-softmax rescale runs once per four tokens.  Partial (O, lse) of each split go to a
// scratch buffer and a second kernel merges them.  Sliding window, ALiBi and "suffix only"
// (kv_start, for cascade attention after a shared radix prefix) are predicates on the kv index.
// Block-table entries are bounds-checked; a bad entry sets the error word and is masked.
//
// Replaces in the reference: the cached attention path of LlamaAttention::forward_with_cache
// (crates/runtime/src/models_v2/llama.rs:1027-1156) where q_len == 1.
#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"
#include <math_constants.h>
#include <stdlib.h>

extern "C" int ub_attn_decode_mma_supported(const UbAttnArgs* a);
extern "C" int ub_attn_decode_mma_main(const UbAttnArgs* a, void* stream);
extern "C" int ub_attn_decode_persist_supported(const UbAttnArgs* a);
extern "C" int ub_attn_decode_persist(const UbAttnArgs* a, void* stream);
extern "C" int ub_attn_decode_warp_supported(const UbAttnArgs* a);
extern "C" int ub_attn_decode_warp(const UbAttnArgs* a, void* stream);

namespace ub {

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gsrc, bool pred) {
  const int sz = pred ? 16 : 0;         // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(sz) : "memory");
}

// Dynamic shared memory of the decode kernel: three K/V stages (reused by the cross-warp reduction), then q, then (m, l).
template <int D, int G>
struct DecodeSmem {
  static constexpr int TILE = 4 * (32 / (D / 8)) * 4;
  static constexpr int STAGE_BYTES = 2 * TILE * D * 2;
  static constexpr int RED_BYTES = 4 * G * D * 4;
  static constexpr int PIPE_BYTES = 3 * STAGE_BYTES > RED_BYTES ? 3 * STAGE_BYTES : RED_BYTES;
  static constexpr int Q_OFF = PIPE_BYTES;
  static constexpr int ML_OFF = Q_OFF + G * D * 4;
  static constexpr int TOTAL = ML_OFF + 4 * G * 2 * 4;
};

template <int D, int G>
__global__ void __launch_bounds__(128) attn_decode_kernel(const UbAttnArgs a, const int gchunks) {
  constexpr int LPT = D / 8;        // lanes per token
  constexpr int TPW = 32 / LPT;     // tokens per warp iteration
  constexpr int UN = 4;             // tokens in flight per lane group
  const int seq = blockIdx.x;
  const int kvh = blockIdx.y / gchunks;
  const int gc = blockIdx.y % gchunks;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane / LPT, chunk = lane % LPT;
  const int Gtot = a.Hq / a.Hkv;
  const int h0 = kvh * Gtot + gc * G;     // first query head of this CTA
  const int gn = min(G, Gtot - gc * G);   // valid heads in this chunk

  constexpr int TILE = 4 * TPW * UN;                 // tokens per pipeline stage
  constexpr int STAGES = 3;
  constexpr int STAGE_BYTES = 2 * TILE * D * 2;      // K tile then V tile
  extern __shared__ __align__(16) uint8_t dsm[];
  // the cross-warp reduction buffer reuses the pipeline stages (all copies have landed by then)
  float (*red_o)[G][D] = reinterpret_cast<float (*)[G][D]>(dsm);
  float (*q_s)[D] = reinterpret_cast<float (*)[D]>(dsm + DecodeSmem<D, G>::Q_OFF);
  float (*red_ml)[G][2] = reinterpret_cast<float (*)[G][2]>(dsm + DecodeSmem<D, G>::ML_OFF);

  const int kv_len = a.seq_lens[seq];
  const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(a.q) + (long long)seq * a.q_stride;
  for (int i = threadIdx.x; i < G * D; i += 128) {
    const int g = i / D, d = i % D;
    q_s[g][d] = g < gn ? __bfloat162float(qp[(long long)(h0 + g) * D + d]) * a.scale * LOG2E : 0.f;
  }
  __syncthreads();

  int lo = a.kv_start;
  if (a.window > 0) lo = max(lo, kv_len - a.window);
  lo = max(lo, 0);
  const int span = max(kv_len - lo, 0);
  int per = (span + a.splits - 1) / a.splits;
  per = (per + a.block_size - 1) / a.block_size * a.block_size;
  const int kv_lo = lo + split * per;
  const int kv_hi = min(kv_len, kv_lo + per);

  float m[G], l[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -CUDART_INF_F; l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  }
  float slope[G];
#pragma unroll
  for (int g = 0; g < G; ++g)
    slope[g] = (a.alibi_slopes != nullptr && g < gn) ? a.alibi_slopes[h0 + g] * LOG2E : 0.f;

  const int* bt = a.block_tables + (long long)seq * a.max_blocks_per_seq;
  const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(a.k_cache);
  const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(a.v_cache);

  const int n_tiles = kv_hi > kv_lo ? (kv_hi - kv_lo + TILE - 1) / TILE : 0;
  // cooperative gather of one tile: TILE tokens x (D/8) 16-byte chunks for K and for V
  auto issue_tile = [&](int t) {
    if (t < n_tiles) {
      uint8_t* st = dsm + (t % STAGES) * STAGE_BYTES;
      const int tile_base = kv_lo + t * TILE;
      for (int c = threadIdx.x; c < TILE * LPT; c += 128) {
        const int tk = c / LPT, part = c % LPT;
        const int pos = tile_base + tk;
        bool okc = pos < kv_hi;
        long long off = 0;
        if (okc) {
          const int bi = pos / a.block_size;
          const int blk = bi < a.max_blocks_per_seq ? bt[bi] : -1;
          if (blk < 0 || blk >= a.num_blocks) {
            set_err(a.err, ERR_BOUNDS, seq);
            okc = false;
          } else {
            off = (((long long)blk * a.Hkv + kvh) * a.block_size + (pos % a.block_size)) * D + part * 8;
          }
        }
        cp_async16_zfill(st + c * 16, kc + off, okc);
        cp_async16_zfill(st + TILE * D * 2 + c * 16, vc + off, okc);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  for (int t = 0; t < STAGES - 1; ++t) issue_tile(t);

  for (int t = 0; t < n_tiles; ++t) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();                    // tile t is visible to everyone; everyone is done with tile t-1
    issue_tile(t + STAGES - 1);         // goes into the stage tile t-1 used
    const uint8_t* ks = dsm + (t % STAGES) * STAGE_BYTES;
    const uint8_t* vs = ks + TILE * D * 2;
    const int base = kv_lo + t * TILE + warp * (TPW * UN);
    bool ok[UN];
    uint4 kk[UN];
    int srow[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int pos = base + u * TPW + grp;
      ok[u] = pos < kv_hi;
      srow[u] = (warp * (TPW * UN) + u * TPW + grp) * D * 2 + chunk * 16;
      kk[u] = *reinterpret_cast<const uint4*>(ks + srow[u]);
    }
    float s[UN][G];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&kk[u]);
      float kf[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) { kf[2 * e] = bf16_lo(w[e]); kf[2 * e + 1] = bf16_hi(w[e]); }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d += q_s[g][chunk * 8 + e] * kf[e];
        s[u][g] = d;
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u)
#pragma unroll
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int o = LPT / 2; o > 0; o >>= 1) s[u][g] += __shfl_xor_sync(0xffffffffu, s[u][g], o);
        const int pos = base + u * TPW + grp;
        s[u][g] = ok[u] ? s[u][g] + slope[g] * (float)(pos - (kv_len - 1)) : -CUDART_INF_F;
      }
    uint4 vv[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) vv[u] = *reinterpret_cast<const uint4*>(vs + srow[u]);
    float p[UN][G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = m[g];
#pragma unroll
      for (int u = 0; u < UN; ++u) mx = fmaxf(mx, s[u][g]);
      const float alpha = (mx == -CUDART_INF_F) ? 1.f : exp2f(m[g] - mx);
      float ps = 0.f;
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        p[u][g] = (s[u][g] == -CUDART_INF_F) ? 0.f : exp2f(s[u][g] - mx);
        ps += p[u][g];
      }
      l[g] = l[g] * alpha + ps;
      m[g] = mx;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] *= alpha;
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&vv[u]);
      float vf[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) { vf[2 * e] = bf16_lo(w[e]); vf[2 * e + 1] = bf16_hi(w[e]); }
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] += p[u][g] * vf[e];
    }
  }

  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                      // the stages are free: red_o lives there from here on

  // merge the token groups inside the warp (lanes that own the same chunk)
#pragma unroll
  for (int o = LPT; o < 32; o <<= 1) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m[g], o);
      const float l2 = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float mx = fmaxf(m[g], m2);
      const float s1 = (m[g] == -CUDART_INF_F) ? 0.f : exp2f(m[g] - mx);
      const float s2 = (m2 == -CUDART_INF_F) ? 0.f : exp2f(m2 - mx);
      l[g] = l[g] * s1 + l2 * s2;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float a2 = __shfl_xor_sync(0xffffffffu, acc[g][e], o);
        acc[g][e] = acc[g][e] * s1 + a2 * s2;
      }
      m[g] = mx;
    }
  }
  if (grp == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int e = 0; e < 8; ++e) red_o[warp][g][chunk * 8 + e] = acc[g][e];
      if (chunk == 0) { red_ml[warp][g][0] = m[g]; red_ml[warp][g][1] = l[g]; }
    }
  }
  __syncthreads();
  // merge the 4 warps; thread i handles output elements i, i+128, ...
  for (int i = threadIdx.x; i < gn * D; i += 128) {
    const int g = i / D, d = i % D;
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, red_ml[w][g][0]);
    float lt = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float sc = (red_ml[w][g][0] == -CUDART_INF_F) ? 0.f : exp2f(red_ml[w][g][0] - mx);
      lt += red_ml[w][g][1] * sc;
      o += red_o[w][g][d] * sc;
    }
    const float inv = lt > 0.f ? 1.f / lt : 0.f;
    const float lse = lt > 0.f ? (mx + log2f(lt)) * LN2 : -CUDART_INF_F;
    const int h = h0 + g;
    if (a.splits == 1) {
      reinterpret_cast<__nv_bfloat16*>(a.out)[(long long)seq * a.o_stride + (long long)h * D + d] =
          __float2bfloat16(o * inv);
      if (d == 0 && a.lse != nullptr) a.lse[(long long)seq * a.Hq + h] = lse;
    } else {
      float* sp = a.scratch + (((long long)seq * a.Hq + h) * a.splits + split) * (D + 2);
      sp[d] = o * inv;
      if (d == 0) sp[D] = lse;
    }
  }
}

// Merge the split partials: out = sum_i O_i * exp(lse_i - lse_max) / sum_i exp(lse_i - lse_max).
__global__ void attn_split_merge_kernel(const float* scratch, __nv_bfloat16* out, float* lse_out, int Hq, int D,
                                        int splits, long long o_stride) {
  const int seq = blockIdx.x, h = blockIdx.y;
  const float* sp = scratch + ((long long)seq * Hq + h) * splits * (D + 2);
  float mx = -CUDART_INF_F;
  for (int i = 0; i < splits; ++i) mx = fmaxf(mx, sp[i * (D + 2) + D]);
  float den = 0.f;
  for (int i = 0; i < splits; ++i) {
    const float ls = sp[i * (D + 2) + D];
    den += (ls == -CUDART_INF_F) ? 0.f : __expf(ls - mx);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f;
    for (int i = 0; i < splits; ++i) {
      const float ls = sp[i * (D + 2) + D];
      const float w = (ls == -CUDART_INF_F) ? 0.f : __expf(ls - mx);
      o += sp[i * (D + 2) + d] * w;
    }
    out[(long long)seq * o_stride + (long long)h * D + d] = __float2bfloat16(den > 0.f ? o / den : 0.f);
  }
  if (threadIdx.x == 0 && lse_out != nullptr)
    lse_out[(long long)seq * Hq + h] = den > 0.f ? mx + __logf(den) : -CUDART_INF_F;
}

// Merge two independently computed attention partials over disjoint key sets.
__global__ void attn_merge2_kernel(const __nv_bfloat16* oa, const float* la, const __nv_bfloat16* ob, const float* lb,
                                   __nv_bfloat16* out, float* lse_out, long long rows, int D) {
  const long long r = blockIdx.x;
  if (r >= rows) return;
  const float a = la[r], b = lb[r];
  const float mx = fmaxf(a, b);
  const float wa = (a == -CUDART_INF_F) ? 0.f : __expf(a - mx);
  const float wb = (b == -CUDART_INF_F) ? 0.f : __expf(b - mx);
  const float den = wa + wb;
  const float ia = den > 0.f ? wa / den : 0.f, ib = den > 0.f ? wb / den : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float v = __bfloat162float(oa[r * D + d]) * ia + __bfloat162float(ob[r * D + d]) * ib;
    out[r * D + d] = __float2bfloat16(v);
  }
  if (threadIdx.x == 0 && lse_out != nullptr) lse_out[r] = den > 0.f ? mx + __logf(den) : -CUDART_INF_F;
}

template <int D, int G>
static void launch_decode_g(const UbAttnArgs& a, dim3 grid, int gchunks, cudaStream_t st) {
  constexpr int SMEM = DecodeSmem<D, G>::TOTAL;
  static bool attr_set[UB_MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < UB_MAX_DEVICES && !attr_set[dev]) {
    cudaFuncSetAttribute(attn_decode_kernel<D, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    attr_set[dev] = true;
  }
  attn_decode_kernel<D, G><<<grid, 128, SMEM, st>>>(a, gchunks);
}

static bool decode_mma_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("UB_DECODE_MMA");     // UB_DECODE_MMA=0 keeps the CUDA-core kernel (A/B comparisons)
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// Short key ranges behind a shared prefix (kv_start > 0): the persistent kernel that overlaps one work item's tail with
// the next one's copies.  UB_DECODE_PERSIST=0 keeps the one-item-per-CTA kernel.
static bool decode_persist_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("UB_DECODE_PERSIST");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// Unsplit ranges with 16-key pages: the kernel with one independent copy / MMA pipeline per warp
// (attn_decode_warp.cu).  UB_DECODE_WARP=0 keeps the CTA-per-item kernels.
static bool decode_warp_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("UB_DECODE_WARP");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <int D>
static int launch_decode(const UbAttnArgs& a, cudaStream_t st) {
  const bool mma_ok = D <= 128 && decode_mma_enabled() && ub_attn_decode_mma_supported(&a);
  if (a.merge_o != nullptr && (!mma_ok || a.splits != 1)) return -7;   // fused merge lives in the warp-MMA kernels only
  // one warp per item needs enough items to keep every SM's copy engines busy; with fewer, an item is better served by
  // the four warps of a CTA
  if (mma_ok && a.splits == 1 && a.num_seqs * a.Hkv >= 256 && decode_warp_enabled() && ub_attn_decode_warp_supported(&a))
    return ub_attn_decode_warp(&a, st);
  if (mma_ok && a.kv_start > 0 && decode_persist_enabled() && ub_attn_decode_persist_supported(&a))
    return ub_attn_decode_persist(&a, st);
  if (mma_ok) {
    int rc = ub_attn_decode_mma_main(&a, st);
    if (rc != 0) return rc;
    if (a.splits > 1) {
      dim3 g2(a.num_seqs, a.Hq);
      attn_split_merge_kernel<<<g2, D <= 128 ? D : 128, 0, st>>>(a.scratch, reinterpret_cast<__nv_bfloat16*>(a.out),
                                                                 a.lse, a.Hq, D, a.splits, a.o_stride);
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return -(int)e;
    }
    return 0;
  }
  const int Gtot = a.Hq / a.Hkv;
  int G = 1;
  while (G < Gtot && G < 8) G <<= 1;
  if (D == 256 && G > 4) G = 4;
  const int gchunks = (Gtot + G - 1) / G;
  dim3 grid(a.num_seqs, a.Hkv * gchunks, a.splits);
  switch (G) {
    case 1: launch_decode_g<D, 1>(a, grid, gchunks, st); break;
    case 2: launch_decode_g<D, 2>(a, grid, gchunks, st); break;
    case 4: launch_decode_g<D, 4>(a, grid, gchunks, st); break;
    default:
      if constexpr (D <= 128) { launch_decode_g<D, 8>(a, grid, gchunks, st); }
      break;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return -(int)e;
  if (a.splits > 1) {
    dim3 g2(a.num_seqs, a.Hq);
    attn_split_merge_kernel<<<g2, D <= 128 ? D : 128, 0, st>>>(a.scratch, reinterpret_cast<__nv_bfloat16*>(a.out),
                                                               a.lse, a.Hq, D, a.splits, a.o_stride);
    e = cudaGetLastError();
    if (e != cudaSuccess) return -(int)e;
  }
  return 0;
}

}  // namespace ub

extern "C" int ub_attn_decode(const UbAttnArgs* a, void* stream_v) {
  using namespace ub;
  if (a->num_seqs <= 0) return 0;
  if (a->Hq % a->Hkv != 0 || a->splits < 1) return -2;
  if (a->splits > 1 && a->scratch == nullptr) return -3;
  cudaStream_t st = (cudaStream_t)stream_v;
  switch (a->D) {
    case 64: return launch_decode<64>(*a, st);
    case 128: return launch_decode<128>(*a, st);
    case 256: return launch_decode<256>(*a, st);
    default: return -4;
  }
}

extern "C" int ub_attn_merge(const void* o_a, const float* lse_a, const void* o_b, const float* lse_b, void* out,
                             float* lse_out, long long rows, int D, void* stream_v) {
  if (rows <= 0) return 0;
  ub::attn_merge2_kernel<<<(unsigned)rows, D <= 128 ? D : 128, 0, (cudaStream_t)stream_v>>>(
      (const __nv_bfloat16*)o_a, lse_a, (const __nv_bfloat16*)o_b, lse_b, (__nv_bfloat16*)out, lse_out, rows, D);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// ----------------------------------------------------------------------------------------------
// Allocation-free variant: the split-KV partials live in a fixed array inside the library image.
// See attn_decode_static.h for who needs this and for the rules of use.
// ----------------------------------------------------------------------------------------------
#include "attn_decode_static.h"
#include <mutex>
#include <stdio.h>

static __device__ __align__(256) float g_static_decode_scratch[UB_ATTN_STATIC_SCRATCH_FLOATS];

namespace {
std::mutex g_static_mu;
float* g_static_ptr[UB_MAX_DEVICES] = {};   // device address of the array, per device, filled on first use
thread_local char g_static_err[256] = "";
}  // namespace

extern "C" const char* ub_attn_decode_static_scratch_error(void) { return g_static_err; }

extern "C" int ub_attn_decode_static_scratch(const UbAttnArgs* a, void* stream_v) {
  g_static_err[0] = 0;
  if (a->num_seqs <= 0) return 0;
  if (a->splits < 1 || a->Hq <= 0 || a->D <= 0) {
    snprintf(g_static_err, sizeof(g_static_err), "bad arguments: splits=%d Hq=%d D=%d", a->splits, a->Hq, a->D);
    return -2;
  }
  const unsigned long long need = (unsigned long long)a->num_seqs * a->Hq * a->splits * (a->D + 2);
  if (a->splits > 1 && need > UB_ATTN_STATIC_SCRATCH_FLOATS) {
    snprintf(g_static_err, sizeof(g_static_err),
             "split-KV partials need %llu floats but the built-in scratch holds %u; lower splits or the batch",
             need, (unsigned)UB_ATTN_STATIC_SCRATCH_FLOATS);
    return UB_ERR_STATIC_SCRATCH_TOO_SMALL;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= UB_MAX_DEVICES) {
    snprintf(g_static_err, sizeof(g_static_err), "no usable current device (index %d)", dev);
    return UB_ERR_STATIC_SCRATCH_SETUP;
  }
  float* ptr;
  {
    std::lock_guard<std::mutex> g(g_static_mu);
    if (g_static_ptr[dev] == nullptr) {
      // In host code the array's name is only a handle; the address the kernel may use comes from here.
      void* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&p, g_static_decode_scratch);
      if (e != cudaSuccess || p == nullptr) {
        snprintf(g_static_err, sizeof(g_static_err), "cudaGetSymbolAddress failed on device %d: %s", dev,
                 cudaGetErrorString(e));
        return UB_ERR_STATIC_SCRATCH_SETUP;
      }
      g_static_ptr[dev] = static_cast<float*>(p);
    }
    ptr = g_static_ptr[dev];
  }
  UbAttnArgs b = *a;
  b.scratch = ptr;
  return ub_attn_decode(&b, stream_v);
}
