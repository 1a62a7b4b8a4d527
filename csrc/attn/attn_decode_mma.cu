// K4 on warp-level tensor-core MMA: paged decode attention (one query token per sequence) for head sizes 64 / 128.
//
// One CTA handles (sequence, kv head, split).  The up-to-16 query heads that share the kv head form the 16 rows of
// an m16n8k16 A operand, so the score and P*V products for all heads of the group cost one MMA stream instead of
// per-head dot products and shuffles: the CUDA-core version of this kernel (attn_decode.cu) was instruction-bound
// at about 40 % of HBM bandwidth.  K/V tiles of 64 tokens come through a three-stage cp.async ring, gathered page
// by page through the block table into XOR-swizzled shared memory; the four warps each take 16 tokens of a tile and
// keep their own online-softmax state, merged once at the end.  Split-KV partials, sliding window, ALiBi and
// kv_start (suffix after a shared prefix) behave exactly as in attn_decode.cu, whose merge kernels are reused.
//
// Replaces in the reference: the cached attention path of LlamaAttention::forward_with_cache
// (crates/runtime/src/models_v2/llama.rs:1027-1156) where q_len == 1.
#include <math_constants.h>

#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"

namespace ub {
namespace dmma {

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr int KT = 64;       // tokens per tile (16 per warp)
constexpr int ROWS = 16;     // query heads per CTA (MMA M)

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool pred) {
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// [rows][D] bf16 tile with 16-byte chunks XOR-swizzled by (row & 7)
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

// STAGES = 3 for long key ranges (two tiles in flight behind the one being used, two CTAs per SM); STAGES = 2 for
// the short suffix ranges of the cascade, where a CTA has only two to four tiles and what hides the latency of its
// dependent loads is a third resident CTA.
template <int D, int STAGES>
struct Smem {
  static constexpr int STAGE_BYTES = 2 * KT * D * 2;                 // K tile then V tile
  static constexpr int RED_BYTES = 4 * ROWS * D * 4;                 // per-warp partial outputs (fp32)
  static constexpr int PIPE_BYTES = STAGES * STAGE_BYTES > RED_BYTES ? STAGES * STAGE_BYTES : RED_BYTES;
  static constexpr int Q_OFF = PIPE_BYTES;                           // [16][D] bf16, swizzled
  static constexpr int ML_OFF = Q_OFF + ROWS * D * 2;                // [4][16][2] floats
  static constexpr int BT_OFF = ML_OFF + 4 * ROWS * 2 * 4;           // block-table entries of this CTA's key range
  static constexpr int BT_MAX = 256;
  static constexpr int TOTAL = BT_OFF + BT_MAX * 4;
};

template <int D, int STAGES>
__global__ void __launch_bounds__(128) attn_decode_mma_kernel(const UbAttnArgs a, const int gchunks) {
  pdl_launch_dependents();
  pdl_wait();          // no global access before the previous kernel has completed
  constexpr int CPR = D / 8;
  using S = Smem<D, STAGES>;
  extern __shared__ __align__(128) uint8_t dsm[];
  uint8_t* q_sm = dsm + S::Q_OFF;
  float (*red_o)[ROWS][D] = reinterpret_cast<float (*)[ROWS][D]>(dsm);
  float (*red_ml)[ROWS][2] = reinterpret_cast<float (*)[ROWS][2]>(dsm + S::ML_OFF);

  const int seq = blockIdx.x;
  const int kvh = blockIdx.y / gchunks, gc = blockIdx.y % gchunks;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Gtot = a.Hq / a.Hkv;
  const int h0 = kvh * Gtot + gc * ROWS;
  const int gn = min(ROWS, Gtot - gc * ROWS);          // valid rows (heads) of this CTA

  // Without a window or KV splits the first page of the range does not depend on the sequence length: fetch the
  // block-table entries together with the length instead of behind it (one dependent global latency less).
  int* bt_sm = reinterpret_cast<int*>(dsm + S::BT_OFF);
  const int* bt = a.block_tables + (long long)seq * a.max_blocks_per_seq;
  const bool bt_early = a.window == 0 && a.splits == 1;
  const int bs_shift = 31 - __clz(a.block_size);
  if (bt_early) {
    const int first = max(a.kv_start, 0) >> bs_shift;
    for (int i = threadIdx.x; i < min(S::BT_MAX, a.max_blocks_per_seq - first); i += 128) bt_sm[i] = bt[first + i];
  }
  const int kv_len = a.seq_lens[seq];
  int lo = a.kv_start;
  if (a.window > 0) lo = max(lo, kv_len - a.window);
  lo = max(lo, 0);
  const int span = max(kv_len - lo, 0);
  int per = (span + a.splits - 1) / a.splits;
  per = (per + a.block_size - 1) / a.block_size * a.block_size;
  const int kv_lo = lo + split * per;
  const int kv_hi = min(kv_len, kv_lo + per);
  const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(a.k_cache);
  const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(a.v_cache);
  const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(a.q) + (long long)seq * a.q_stride;

  // Q rows (heads of the group; rows past gn are zero)
  for (int i = threadIdx.x; i < ROWS * CPR; i += 128) {
    const int r = i / CPR, c = i % CPR;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < gn) v = *reinterpret_cast<const uint4*>(qp + (long long)(h0 + r) * D + c * 8);
    *reinterpret_cast<uint4*>(q_sm + tile_off<D>(r, c)) = v;
  }

  // Tiles start on a page boundary, so a tile is KT / block_size whole pages: one block-table lookup and one
  // base address per page, then 16-byte chunks at consecutive addresses (no per-chunk division).
  const int tile_origin = kv_lo & ~(a.block_size - 1);
  const int n_tiles = kv_hi > tile_origin ? (kv_hi - tile_origin + KT - 1) / KT : 0;
  // All block-table entries of the range are fetched at once, before the first copy: read one by one in front of
  // each page they put a dependent global load (and its latency) in front of every group of copies.
  const int page0 = tile_origin >> bs_shift;
  const int n_pages = kv_hi > tile_origin ? ((kv_hi - tile_origin + a.block_size - 1) >> bs_shift) : 0;
  if (!bt_early)
    for (int i = threadIdx.x; i < min(n_pages, S::BT_MAX); i += 128)
      bt_sm[i] = (page0 + i) < a.max_blocks_per_seq ? bt[page0 + i] : -1;
  __syncthreads();                                       // q_sm and bt_sm complete
  const int pages_per_tile = KT >> bs_shift;
  const int chunks_per_page = CPR << bs_shift;
  auto issue_tile = [&](int t) {
    if (t < n_tiles) {
      uint8_t* st = dsm + (t % STAGES) * S::STAGE_BYTES;
      const int t0 = tile_origin + t * KT;
      for (int pg = 0; pg < pages_per_tile; ++pg) {
        const int pos0 = t0 + (pg << bs_shift);
        const int nvalid = min(max(kv_hi - pos0, 0), a.block_size);      // tokens of this page that exist
        long long base = 0;
        if (nvalid > 0) {
          const int bi = pos0 >> bs_shift;
          const int blk = bi >= a.max_blocks_per_seq ? -1 : ((bi - page0) < S::BT_MAX ? bt_sm[bi - page0] : bt[bi]);
          if (blk < 0 || blk >= a.num_blocks) set_err(a.err, ERR_BOUNDS, seq);
          else base = (((long long)blk * a.Hkv + kvh) << bs_shift) * D;
        }
        for (int c = threadIdx.x; c < chunks_per_page; c += 128) {
          const int tr = c / CPR;                                        // token inside the page (CPR is a power of two)
          const int r = (pg << bs_shift) + tr;
          const bool ok = tr < nvalid;
          const uint32_t dst = tile_off<D>(r, c % CPR);
          cp_async16(st + dst, kc + base + c * 8, ok);
          cp_async16(st + KT * D * 2 + dst, vc + base + c * 8, ok);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  for (int t = 0; t < STAGES - 1; ++t) issue_tile(t);

  uint32_t qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int c = ks * 2 + (lane >> 4);
    ldsm_x4(smem_u32(q_sm + tile_off<D>(r, c)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }

  // this thread's rows: r_a = lane / 4 and r_b = r_a + 8 (rows are query heads)
  const int ra = lane >> 2, rb = ra + 8;
  float slope_a = 0.f, slope_b = 0.f;
  if (a.alibi_slopes != nullptr) {
    if (ra < gn) slope_a = a.alibi_slopes[h0 + ra] * LOG2E;
    if (rb < gn) slope_b = a.alibi_slopes[h0 + rb] * LOG2E;
  }
  const float sc = a.scale * LOG2E;
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_a = -CUDART_INF_F, m_b = -CUDART_INF_F, l_a = 0.f, l_b = 0.f;

  // The partial over the shared prefix that the epilogue folds in: fetched now, so that its latency runs under the
  // key / value copies instead of behind the last tile (first four output elements per thread = a GQA group of 4).
  constexpr int PRE = 4;
  float pre_la[PRE], pre_oa[PRE];
#pragma unroll
  for (int k = 0; k < PRE; ++k) {
    const int i = threadIdx.x + k * 128;
    pre_la[k] = 0.f;
    pre_oa[k] = 0.f;
    if (a.merge_o != nullptr && a.splits == 1 && i < gn * D) {
      const int h = h0 + i / D;
      pre_la[k] = a.merge_lse[(long long)seq * a.Hq + h];
      pre_oa[k] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.merge_o)[((long long)seq * a.Hq + h) * D + i % D]);
    }
  }

  for (int t = 0; t < n_tiles; ++t) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();                       // tile t visible to all; all are done with tile t-1
    issue_tile(t + STAGES - 1);
    const uint8_t* kb = dsm + (t % STAGES) * S::STAGE_BYTES;
    const uint8_t* vb = kb + KT * D * 2;
    const int tw0 = warp * 16;             // this warp's 16 tokens inside the tile
    const int t0 = tile_origin + t * KT + tw0;
    if (t0 >= kv_hi || t0 + 16 <= kv_lo) continue;   // warp-uniform: nothing visible in this warp's slice             // warp-uniform: nothing visible in this warp's slice

    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int mi = lane >> 3;
      const int r = tw0 + (mi >> 1) * 8 + (lane & 7);
      const int c = ks * 2 + (mi & 1);
      uint32_t b0, b1, b2, b3;
      ldsm_x4(smem_u32(kb + tile_off<D>(r, c)), b0, b1, b2, b3);
      mma_bf16(s[0], qf[ks], b0, b1);
      mma_bf16(s[1], qf[ks], b2, b3);
    }
    float mx_a = m_a, mx_b = m_b;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kpos = t0 + j * 8 + (lane & 3) * 2 + (e & 1);
        const bool is_b = e >= 2;
        float v = s[j][e] * sc + (is_b ? slope_b : slope_a) * (float)(kpos - (kv_len - 1));
        v = (kpos < kv_hi && kpos >= kv_lo) ? v : -CUDART_INF_F;
        s[j][e] = v;
        if (is_b) mx_b = fmaxf(mx_b, v); else mx_a = fmaxf(mx_a, v);
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float al_a = (mx_a == -CUDART_INF_F) ? 1.f : exp2f(m_a - mx_a);
    const float al_b = (mx_b == -CUDART_INF_F) ? 1.f : exp2f(m_b - mx_b);
    m_a = mx_a; m_b = mx_b;
    float ps_a = 0.f, ps_b = 0.f;
    uint32_t pf[4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float p0 = (s[j][0] == -CUDART_INF_F) ? 0.f : exp2f(s[j][0] - mx_a);
      const float p1 = (s[j][1] == -CUDART_INF_F) ? 0.f : exp2f(s[j][1] - mx_a);
      const float p2 = (s[j][2] == -CUDART_INF_F) ? 0.f : exp2f(s[j][2] - mx_b);
      const float p3 = (s[j][3] == -CUDART_INF_F) ? 0.f : exp2f(s[j][3] - mx_b);
      ps_a += p0 + p1; ps_b += p2 + p3;
      pf[j * 2 + 0] = pack_bf16x2(p0, p1);     // accumulator layout of two adjacent n8 tiles == A fragment of a k16 step
      pf[j * 2 + 1] = pack_bf16x2(p2, p3);
    }
    l_a = l_a * al_a + ps_a;
    l_b = l_b * al_b + ps_b;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b; }
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      const int mi = lane >> 3;
      const int r = tw0 + (mi & 1) * 8 + (lane & 7);
      const int c = dp * 2 + (mi >> 1);
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(smem_u32(vb + tile_off<D>(r, c)), b0, b1, b2, b3);
      mma_bf16(o[dp * 2], pf, b0, b1);
      mma_bf16(o[dp * 2 + 1], pf, b2, b3);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                           // the stages are free: red_o lives there from here on

  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    const int d = i * 8 + (lane & 3) * 2;
    if (ra < gn) { red_o[warp][ra][d] = o[i][0]; red_o[warp][ra][d + 1] = o[i][1]; }
    if (rb < gn) { red_o[warp][rb][d] = o[i][2]; red_o[warp][rb][d + 1] = o[i][3]; }
  }
  if ((lane & 3) == 0) {
    if (ra < gn) { red_ml[warp][ra][0] = m_a; red_ml[warp][ra][1] = l_a; }
    if (rb < gn) { red_ml[warp][rb][0] = m_b; red_ml[warp][rb][1] = l_b; }
  }
  __syncthreads();
  for (int i = threadIdx.x, it = 0; i < gn * D; i += 128, ++it) {
    const int g = i / D, d = i % D;
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, red_ml[w][g][0]);
    float lt = 0.f, ov = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float scw = (red_ml[w][g][0] == -CUDART_INF_F) ? 0.f : exp2f(red_ml[w][g][0] - mx);
      lt += red_ml[w][g][1] * scw;
      ov += red_o[w][g][d] * scw;
    }
    const float inv = lt > 0.f ? 1.f / lt : 0.f;
    float lse = lt > 0.f ? (mx + log2f(lt)) * LN2 : -CUDART_INF_F;
    const int h = h0 + g;
    if (a.splits == 1) {
      float val = ov * inv;
      if (a.merge_o != nullptr) {
        // fold in the partial result over the other key set (shared prefix): weights exp(lse_x - max)
        float la, oa;
        if (it < PRE) {
          // static indices keep the prefetched values in registers
          la = it == 0 ? pre_la[0] : it == 1 ? pre_la[1] : it == 2 ? pre_la[2] : pre_la[3];
          oa = it == 0 ? pre_oa[0] : it == 1 ? pre_oa[1] : it == 2 ? pre_oa[2] : pre_oa[3];
        } else {
          la = a.merge_lse[(long long)seq * a.Hq + h];
          oa = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.merge_o)[((long long)seq * a.Hq + h) * D + d]);
        }
        const float mm = fmaxf(la, lse);
        const float wa = (la == -CUDART_INF_F) ? 0.f : __expf(la - mm);
        const float wb = (lse == -CUDART_INF_F) ? 0.f : __expf(lse - mm);
        const float den = wa + wb;
        val = den > 0.f ? (wa * oa + wb * val) / den : 0.f;
        lse = den > 0.f ? mm + __logf(den) : -CUDART_INF_F;
      }
      reinterpret_cast<__nv_bfloat16*>(a.out)[(long long)seq * a.o_stride + (long long)h * D + d] = __float2bfloat16(val);
      if (d == 0 && a.lse != nullptr) a.lse[(long long)seq * a.Hq + h] = lse;
    } else {
      float* sp = a.scratch + (((long long)seq * a.Hq + h) * a.splits + split) * (D + 2);
      sp[d] = ov * inv;
      if (d == 0) sp[D] = lse;
    }
  }
}

template <int D, int STAGES>
static int launch(const UbAttnArgs& a, cudaStream_t st) {
  constexpr int SMEM = Smem<D, STAGES>::TOTAL;
  static bool attr_set[UB_MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < UB_MAX_DEVICES && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel<D, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return -(int)e;
    attr_set[dev] = true;
  }
  const int Gtot = a.Hq / a.Hkv;
  const int gchunks = (Gtot + ROWS - 1) / ROWS;
  dim3 grid(a.num_seqs, a.Hkv * gchunks, a.splits);
  ub::launch_pdl(attn_decode_mma_kernel<D, STAGES>, grid, dim3(128), (size_t)SMEM, st, a, gchunks);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

}  // namespace dmma
}  // namespace ub

// The main kernel of the decode step for head sizes 64 / 128 (the split merge, if any, is launched by the caller).
extern "C" int ub_attn_decode_mma_supported(const UbAttnArgs* a) {
  if (a->D != 64 && a->D != 128) return 0;
  if (a->block_size < 8 || a->block_size > 64 || (a->block_size & (a->block_size - 1))) return 0;   // whole pages per 64-token tile
  if (a->Hkv <= 0 || a->Hq % a->Hkv != 0 || a->q_stride % 8 != 0) return 0;
  if ((reinterpret_cast<uintptr_t>(a->q) & 15) || (reinterpret_cast<uintptr_t>(a->k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(a->v_cache) & 15))
    return 0;
  return 1;
}

extern "C" int ub_attn_decode_mma_main(const UbAttnArgs* a, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // suffix ranges after a shared prefix are short (two to four tiles): a third resident CTA per SM hides more of the
  // chain of dependent latencies than a deeper ring does (68.8 us vs 83.3 us per layer on the serving step);
  // UB_DECODE_STAGES=3 keeps the deep ring there
  static const int suffix_stages = [] {
    const char* e = getenv("UB_DECODE_STAGES");
    return (e != nullptr && atoi(e) == 3) ? 3 : 2;
  }();
  if (a->kv_start > 0 && suffix_stages == 2) return a->D == 64 ? ub::dmma::launch<64, 2>(*a, st) : ub::dmma::launch<128, 2>(*a, st);
  return a->D == 64 ? ub::dmma::launch<64, 3>(*a, st) : ub::dmma::launch<128, 3>(*a, st);
}
