// K8: token sampling on the device.  One CTA (1024 threads) per batch row.
//   greedy            : argmax (lowest index wins ties), also returns the winning value so that
//                       vocab-parallel shards can be merged with a (value, index) reduction.
//   temperature/top-k/top-p : logits / T  ->  radix-select of the k-th largest key (4 x 8-bit
//                       histogram passes over the row, which stays L2-resident)  ->  the <= 1024
//                       survivors are sorted in shared memory (value desc, index asc: deterministic)
//                       ->  softmax, nucleus cut (smallest prefix whose mass >= top_p), inverse-CDF
//                       draw with a Philox4x32-10 uniform keyed by (seed, step, row).
//   temperature only  : inverse-CDF over the whole vocabulary with a segmented block scan.
// The repetition penalty uses a vocabulary bitmap in shared memory built from the token history.
//
// Replaces in the reference: Sampler::sample_greedy / sample_temperature / sample_top_p
// (crates/runtime/src/inference.rs:27-155), GreedySampler (crates/runtime/src/sampler.rs:22-67) and
// the per-model copies (crates/runtime/src/models_v2/llama.rs:566-612); unlike the reference,
// top_k and repetition_penalty are honoured.
#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"
#include <math_constants.h>

namespace ub {

constexpr int SB = 1024;      // threads per CTA == max candidates
constexpr int MAXV_BITMAP = 262144;

__device__ __forceinline__ uint32_t mulhilo(uint32_t a, uint32_t b, uint32_t* hi) {
  const uint64_t p = (uint64_t)a * b;
  *hi = (uint32_t)(p >> 32);
  return (uint32_t)p;
}
// Philox4x32-10; returns the first of the four output words mapped to [0, 1).
__device__ __forceinline__ float philox_uniform(unsigned long long seed, unsigned long long step, uint32_t row) {
  uint32_t c0 = (uint32_t)step, c1 = (uint32_t)(step >> 32), c2 = row, c3 = 0;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, hi1;
    const uint32_t lo0 = mulhilo(0xD2511F53u, c0, &hi0);
    const uint32_t lo1 = mulhilo(0xCD9E8D57u, c2, &hi1);
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return (float)(c0 >> 8) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ uint32_t f2key(float f) {  // order-preserving float -> uint
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct RowReader {
  const void* base; int f32; const uint32_t* bitmap; float pen; float inv_t;   // inv_t = 1 for pre-scaled candidates
  __device__ __forceinline__ float operator()(int i) const {
    float v = f32 ? reinterpret_cast<const float*>(base)[i]
                  : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
    if (bitmap != nullptr && (bitmap[i >> 5] >> (i & 31) & 1u)) v = v > 0.f ? v / pen : v * pen;
    return v * inv_t;
  }
};

__device__ __forceinline__ float blk_reduce_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < 32 ? red[threadIdx.x] : -CUDART_INF_F;
  if (threadIdx.x < 32) { t = warp_max(t); if (threadIdx.x == 0) red[0] = t; }
  __syncthreads();
  return red[0];
}
__device__ __forceinline__ float blk_reduce_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < 32 ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) { t = warp_sum(t); if (threadIdx.x == 0) red[0] = t; }
  __syncthreads();
  return red[0];
}
// exclusive scan of one float per thread over the CTA; returns the exclusive prefix, *total gets the sum
__device__ __forceinline__ float blk_excl_scan(float v, float* red, float* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { const float t = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += t; }
  __syncthreads();
  if (lane == 31) red[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    float w = red[lane];
    float wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const float t = __shfl_up_sync(0xffffffffu, wi, o); if (lane >= o) wi += t; }
    red[lane] = wi - w;
    if (lane == 31) red[32] = wi;
  }
  __syncthreads();
  *total = red[32];
  return red[warp] + inc - v;
}

__global__ void __launch_bounds__(SB) sample_kernel(const UbSampleArgs a) {
  extern __shared__ uint32_t dyn[];   // bitmap [ (V+31)/32 ] when a repetition penalty is active
  __shared__ float red[40];
  __shared__ int red_i[32];
  __shared__ uint32_t hist[256];
  __shared__ float cand_v[SB];
  __shared__ int cand_i[SB];
  __shared__ uint32_t sh_prefix, sh_need;
  __shared__ int sh_count, sh_pick;

  const int row = blockIdx.x, tid = threadIdx.x;
  const int V = a.V;
  const float temp = a.temperature != nullptr ? a.temperature[row] : 0.f;
  const bool greedy = !(temp > 0.f);
  const float pen = a.rep_penalty != nullptr ? a.rep_penalty[row] : 1.f;
  const uint32_t* bitmap = nullptr;
  if (pen != 1.f && a.prev_ids != nullptr && V <= MAXV_BITMAP) {
    const int words = (V + 31) / 32;
    for (int i = tid; i < words; i += SB) dyn[i] = 0u;
    __syncthreads();
    for (int i = tid; i < a.prev_ld; i += SB) {
      const int id = a.prev_ids[(long long)row * a.prev_ld + i];
      if (id >= 0 && id < V) atomicOr(&dyn[id >> 5], 1u << (id & 31));
    }
    __syncthreads();
    bitmap = dyn;
  }
  RowReader rd;
  rd.base = a.logits_f32 ? (const void*)(reinterpret_cast<const float*>(a.logits) + (long long)row * a.ld)
                         : (const void*)(reinterpret_cast<const __nv_bfloat16*>(a.logits) + (long long)row * a.ld);
  rd.f32 = a.logits_f32; rd.bitmap = bitmap; rd.pen = pen; rd.inv_t = (greedy || a.id_map != nullptr) ? 1.f : 1.f / temp;

  // ---- max / argmax ----
  float best = -CUDART_INF_F; int best_i = 0x7fffffff;
  for (int i = tid; i < V; i += SB) {
    const float v = rd(i);
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if ((tid & 31) == 0) { red[tid >> 5] = best; red_i[tid >> 5] = best_i; }
  __syncthreads();
  if (tid < 32) {
    best = red[tid]; best_i = red_i[tid];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (tid == 0) { red[33] = best; red_i[0] = best_i; }
  }
  __syncthreads();
  const float vmax = red[33];
  const int imax = red_i[0];
  if (greedy) {
    if (tid == 0) {
      const int pick = imax == 0x7fffffff ? 0 : imax;
      a.out_ids[row] = a.id_map != nullptr ? a.id_map[(long long)row * a.ld + pick] : pick + a.vocab_offset;
      if (a.out_vals != nullptr) a.out_vals[row] = vmax;
    }
    if (a.cand_vals != nullptr) {
      // stage 1 of a vocabulary-parallel draw, greedy row: the shard's winner is its only candidate
      for (int j = tid; j < a.cand_k; j += SB) {
        a.cand_vals[(long long)row * a.cand_k + j] = j == 0 ? vmax : -CUDART_INF_F;
        a.cand_ids[(long long)row * a.cand_k + j] = j == 0 ? (imax == 0x7fffffff ? 0 : imax) + a.vocab_offset : -1;
      }
    }
    return;
  }
  const float u = philox_uniform(a.seed, a.step, (uint32_t)row);
  int k = a.top_k != nullptr ? a.top_k[row] : 0;
  const float top_p = a.top_p != nullptr ? a.top_p[row] : 1.f;
  if (k <= 0 && (top_p < 1.f || a.cand_vals != nullptr)) k = SB;
  if (k > SB) k = SB;
  if (a.cand_vals != nullptr && k > a.cand_k) k = a.cand_k;
  if (k > V) k = V;

  if (k <= 0) {
    // ---- full-vocabulary inverse CDF ----
    const int seg = (V + SB - 1) / SB;
    const int lo = tid * seg, hi = min(V, lo + seg);
    float s = 0.f;
    for (int i = lo; i < hi; ++i) s += __expf(rd(i) - vmax);
    float total;
    const float excl = blk_excl_scan(s, red, &total);
    if (a.stats_out != nullptr) {
      // stage 1 of a vocabulary-parallel draw from the whole vocabulary: this shard's maximum and mass
      if (tid == 0) { a.stats_out[2 * row] = vmax; a.stats_out[2 * row + 1] = total; }
      return;
    }
    float target = u * total;
    if (a.target_in != nullptr) {
      // stage 2: the target inside this shard was worked out from all shards' masses; negative = not this shard's draw
      target = a.target_in[row];
      if (target < 0.f) {
        if (tid == 0) { a.out_ids[row] = -1; if (a.out_vals != nullptr) a.out_vals[row] = -CUDART_INF_F; }
        return;
      }
    }
    if (tid == 0) sh_pick = -1;
    __syncthreads();
    if (lo < hi && target >= excl && (target < excl + s || hi == V)) {
      float c = excl; int pick = hi - 1;
      for (int i = lo; i < hi; ++i) { c += __expf(rd(i) - vmax); if (c > target) { pick = i; break; } }
      atomicMax(&sh_pick, pick);   // at most one segment matches except at float boundaries
    }
    __syncthreads();
    if (tid == 0) {
      const int pick = sh_pick < 0 ? imax : sh_pick;
      a.out_ids[row] = a.id_map != nullptr ? a.id_map[(long long)row * a.ld + pick] : pick + a.vocab_offset;
      if (a.out_vals != nullptr) a.out_vals[row] = a.target_in != nullptr ? 1.f : vmax;
    }
    return;
  }

  // ---- radix select: key of the k-th largest element ----
  uint32_t prefix = 0, mask = 0; uint32_t need = (uint32_t)k;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = tid; i < 256; i += SB) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < V; i += SB) {
      const uint32_t key = f2key(rd(i));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t n = need; int b = 255;
      for (; b > 0; --b) { if (hist[b] >= n) break; n -= hist[b]; }
      sh_prefix = prefix | ((uint32_t)b << shift);
      sh_need = n;
    }
    __syncthreads();
    prefix = sh_prefix; need = sh_need; mask |= 255u << shift;
    __syncthreads();
  }
  const uint32_t thr = prefix;        // key of the k-th largest; `need` ties at thr are still wanted
  // ---- collect: everything above thr (any order), then the `need` lowest-index ties ----
  if (tid == 0) sh_count = 0;
  cand_v[tid] = -CUDART_INF_F; cand_i[tid] = 0x7fffffff;
  __syncthreads();
  for (int i = tid; i < V; i += SB) {
    const float v = rd(i);
    if (f2key(v) > thr) { const int p = atomicAdd(&sh_count, 1); if (p < SB) { cand_v[p] = v; cand_i[p] = i; } }
  }
  __syncthreads();
  const int above = min(sh_count, SB);
  {
    const int seg = (V + SB - 1) / SB;
    const int lo = tid * seg, hi = min(V, lo + seg);
    int cnt = 0;
    for (int i = lo; i < hi; ++i) cnt += (f2key(rd(i)) == thr);
    float total;
    const int excl = (int)blk_excl_scan((float)cnt, red, &total);   // counts < 2^24: exact in fp32
    int pos = excl;
    for (int i = lo; i < hi && pos < (int)need; ++i) {
      const float v = rd(i);
      if (f2key(v) == thr) { if (above + pos < SB) { cand_v[above + pos] = v; cand_i[above + pos] = i; } ++pos; }
    }
  }
  __syncthreads();
  const int ncand = min(above + (int)need, SB);
  // ---- bitonic sort (value desc, index asc) ----
  for (int sz = 2; sz <= SB; sz <<= 1) {
    for (int st = sz >> 1; st > 0; st >>= 1) {
      const int j = tid ^ st;
      if (j > tid) {
        const bool desc_block = ((tid & sz) == 0);
        const float va = cand_v[tid], vb = cand_v[j];
        const int ia = cand_i[tid], ib = cand_i[j];
        const bool a_first = (va > vb) || (va == vb && ia < ib);
        if (a_first != desc_block) { cand_v[tid] = vb; cand_v[j] = va; cand_i[tid] = ib; cand_i[j] = ia; }
      }
      __syncthreads();
    }
  }
  if (a.cand_vals != nullptr) {
    // stage 1 of a vocabulary-parallel draw: hand the sorted survivors to the merge
    for (int j = tid; j < a.cand_k; j += SB) {
      const bool ok = j < ncand && cand_i[j] != 0x7fffffff;
      a.cand_vals[(long long)row * a.cand_k + j] = ok ? cand_v[j] : -CUDART_INF_F;
      a.cand_ids[(long long)row * a.cand_k + j] = ok ? cand_i[j] + a.vocab_offset : -1;
    }
    return;
  }
  // ---- softmax over survivors, nucleus cut, draw ----
  const float pv = tid < ncand ? __expf(cand_v[tid] - vmax) : 0.f;
  float total;
  const float excl = blk_excl_scan(pv, red, &total);
  const float incl = excl + pv;
  if (tid == 0) sh_count = ncand - 1;
  __syncthreads();
  // cutoff = first index whose inclusive mass reaches top_p * total
  if (tid < ncand && incl >= top_p * total && excl < top_p * total) atomicMin(&sh_count, tid);
  __syncthreads();
  const int cut = sh_count;
  if (tid == cut) red[34] = incl;
  if (tid == 0) sh_pick = cut;
  __syncthreads();
  const float target = u * red[34];
  if (tid <= cut && incl > target && excl <= target) atomicMin(&sh_pick, tid);
  __syncthreads();
  if (tid == 0) {
    const int pick = cand_i[sh_pick];
    a.out_ids[row] = a.id_map != nullptr ? a.id_map[(long long)row * a.ld + pick] : pick + a.vocab_offset;
    if (a.out_vals != nullptr) a.out_vals[row] = vmax;
  }
}

// (value, index) merge of per-shard greedy winners: vals/ids are [world, B]; lowest global id wins ties.
__global__ void argmax_merge_kernel(const float* vals, const int* ids, int world, int B, int* out_ids) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  float bv = -CUDART_INF_F; int bi = 0x7fffffff;
  for (int w = 0; w < world; ++w) {
    const float v = vals[w * B + b]; const int i = ids[w * B + b];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  out_ids[b] = bi;
}

}  // namespace ub

extern "C" int ub_sample(const UbSampleArgs* a, void* stream_v) {
  if (a->B <= 0) return 0;
  if (a->cand_vals != nullptr && (a->cand_ids == nullptr || a->cand_k <= 0 || a->cand_k > ub::SB)) return -2;
  if (a->id_map != nullptr && (!a->logits_f32 || a->cand_vals != nullptr)) return -2;
  size_t dyn = 0;
  if (a->rep_penalty != nullptr && a->prev_ids != nullptr && a->V <= ub::MAXV_BITMAP) dyn = ((size_t)a->V + 31) / 32 * 4;
  ub::sample_kernel<<<a->B, ub::SB, dyn, (cudaStream_t)stream_v>>>(*a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int ub_argmax_merge(const float* vals, const int* ids, int world, int B, int* out_ids, void* stream_v) {
  if (B <= 0) return 0;
  ub::argmax_merge_kernel<<<(B + 127) / 128, 128, 0, (cudaStream_t)stream_v>>>(vals, ids, world, B, out_ids);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
