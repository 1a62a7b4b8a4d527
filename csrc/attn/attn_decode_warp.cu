// K4, short and medium key ranges: paged decode attention with one independent pipeline per WARP.
//
// The other decode kernels give a (sequence, KV head) work item to a CTA of four warps: every 64-key tile costs a
// block barrier, the copy of a tile is spread over 128 threads that each recompute page addresses, and an item ends
// with a reduction of four partial outputs through shared memory.  On the suffix pass of the cascade (128..256 keys
// per item) that instruction stream, not HBM, set the pace (about 950 warp instructions per warp and tile, issue
// slots 43 % used at 0.49 of the copy bandwidth).  Here a warp owns its items outright:
//
//   * one page (16 keys) per pipeline stage, copied by the warp's own 16-byte cp.async with destination offsets
//     that are computed once per kernel; the stages of a warp form a ring that only this warp touches, so the
//     only synchronisation in the main loop is cp.async.wait_group + __syncwarp;
//   * the query rows live in registers as MMA A fragments loaded straight from global memory (for a GQA group of up
//     to 8 heads the fragments of rows 8..15 are the constant zero and cost no registers);
//   * the warp keeps the whole online-softmax state and all D output columns of its item, so there is no cross-warp
//     reduction: the epilogue folds in the partial over the shared prefix and stores the rows;
//   * the next item's sequence length and block-table entries are requested while the current item streams.
//
// Same math as attn_decode_mma.cu (m16n8k16 warp MMAs, the GQA group as MMA rows, base-2 online softmax).
// Restrictions: page size 16, head size 64 / 128, no sliding window, no ALiBi, no KV splits; the caller falls back
// to the other kernels otherwise.
//
// Replaces in the reference: the cached attention path of LlamaAttention::forward_with_cache
// (crates/runtime/src/models_v2/llama.rs:1027-1156) where q_len == 1.
#include <math_constants.h>
#include <stdlib.h>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"

namespace ub {
namespace dwarp {

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr int PAGE = 16;     // keys per page and per pipeline stage
constexpr int WARPS = 4;     // per CTA

__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(bytes) : "memory");
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
__device__ __forceinline__ float ex2a(float x) {        // 2^x, approximate; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// D = head size, S = ring stages per warp, SMALLG = the GQA group has at most 8 heads (MMA rows 8..15 stay zero)
template <int D, int S, bool SMALLG>
__global__ void __launch_bounds__(WARPS * 32, (D == 128 ? (S <= 3 ? 2 : 1) : 3))
attn_decode_warp_kernel(const UbAttnArgs a, const int gchunks, const int n_items) {
  constexpr int CPR = D / 8;                       // 16-byte chunks per key row
  constexpr int ROWB = D * 2;                      // bytes per key row
  constexpr int PB = PAGE * ROWB;                  // bytes of one page of K (or V)
  constexpr int NI = PAGE * CPR / 32;              // 16-byte copies per lane, page and tensor
  constexpr int STAGE = 2 * PB;                    // K page then V page
  extern __shared__ __align__(128) uint8_t dsm[];

  pdl_launch_dependents();
  pdl_wait();          // no global access before the previous kernel has completed

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ring = smem_u32(dsm) + warp * (S * STAGE);
  const int Gtot = a.Hq / a.Hkv;
  const int per_seq = a.Hkv * gchunks;
  const int kv_lo = max(a.kv_start, 0);
  const int p0 = kv_lo / PAGE;
  const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(a.k_cache);
  const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(a.v_cache);
  const __nv_bfloat16* mo = reinterpret_cast<const __nv_bfloat16*>(a.merge_o);
  const float sc = a.scale * LOG2E;

  // destination of this lane's i-th 16-byte copy inside a page (swizzled by the row), and its row
  uint32_t dsto[NI];
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int j = lane + 32 * i, r = j / CPR, c = j % CPR;
    dsto[i] = (uint32_t)(r * ROWB + ((c ^ (r & 7)) << 4));
  }
  // ldmatrix source offsets of this lane: K rows for S = Q K^T, V rows (transposed load) for O += P V
  const int mi = lane >> 3;
  const int kr = (mi >> 1) * 8 + (lane & 7), kcb = mi & 1;          // K: matrix mi covers keys (mi>>1)*8.., chunk ks*2 + (mi&1)
  const int vr = (mi & 1) * 8 + (lane & 7), vcb = mi >> 1;          // V: matrix mi covers keys (mi&1)*8.., chunk dp*2 + (mi>>1)
  const uint32_t krow = kr * ROWB, vrow = PB + vr * ROWB;
  const int kx = kr & 7, vx = vr & 7;

  const int gw = blockIdx.x * WARPS + warp, gstride = gridDim.x * WARPS;
  int item = gw;
  if (item >= n_items) return;
  // metadata of the item after the current one, requested one item ahead
  int nx_len = 0, nx_bt = -1;
  auto request = [&](int it) {
    const int seq = it / per_seq;
    nx_len = a.seq_lens[seq];
    const int bi = p0 + lane;
    nx_bt = bi < a.max_blocks_per_seq ? a.block_tables[(long long)seq * a.max_blocks_per_seq + bi] : -1;
  };
  request(item);

  const int ra = lane >> 2;                          // this lane's MMA rows: ra and ra + 8
  while (true) {
    const int seq = item / per_seq;
    const int rem = item - seq * per_seq;
    const int kvh = rem / gchunks, gc = rem - kvh * gchunks;
    const int h0 = kvh * Gtot + gc * 16;
    const int gn = min(16, Gtot - gc * 16);
    const int kv_hi = nx_len;
    int bt = nx_bt;                                  // block-table entries p0 + lane (reloaded every 32 pages)
    const int P = kv_hi > kv_lo ? (kv_hi + PAGE - 1) / PAGE - p0 : 0;
    const int next_item = item + gstride;
    const bool has_next = next_item < n_items;

    // ---- query rows as A fragments, straight from global memory
    uint32_t qf[D / 16][4];
    {
      const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(a.q) + (long long)seq * a.q_stride + (long long)h0 * D;
      const int cq = (lane & 3) * 2;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        qf[ks][0] = qf[ks][1] = qf[ks][2] = qf[ks][3] = 0u;
        if (ra < gn) {
          qf[ks][0] = *reinterpret_cast<const uint32_t*>(qp + (long long)ra * D + ks * 16 + cq);
          qf[ks][2] = *reinterpret_cast<const uint32_t*>(qp + (long long)ra * D + ks * 16 + 8 + cq);
        }
        if (!SMALLG && ra + 8 < gn) {
          qf[ks][1] = *reinterpret_cast<const uint32_t*>(qp + (long long)(ra + 8) * D + ks * 16 + cq);
          qf[ks][3] = *reinterpret_cast<const uint32_t*>(qp + (long long)(ra + 8) * D + ks * 16 + 8 + cq);
        }
      }
    }

    // copies page `pi` of the item into stage pi % S: whole rows, rows past the end of the sequence zero-filled
    auto issue = [&](int pi) {
      if (pi > 0 && (pi & 31) == 0) {
        const int bi = p0 + pi + lane;
        bt = bi < a.max_blocks_per_seq ? a.block_tables[(long long)seq * a.max_blocks_per_seq + bi] : -1;
      }
      int blk = __shfl_sync(0xffffffffu, bt, pi & 31);
      const int nvalid = min(kv_hi - (p0 + pi) * PAGE, PAGE);
      bool ok = true;
      if (blk < 0 || blk >= a.num_blocks) {
        if (lane == 0) set_err(a.err, ERR_BOUNDS, seq);
        blk = 0;
        ok = false;
      }
      const long long base = ((long long)blk * a.Hkv + kvh) * (PAGE * D) + lane * 8;
      const uint32_t st = ring + (pi % S) * STAGE;
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        const int r = (lane + 32 * i) / CPR;
        const int bytes = (ok && r < nvalid) ? 16 : 0;
        cp_async16(st + dsto[i], kc + base + i * 256, bytes);
        cp_async16(st + PB + dsto[i], vc + base + i * 256, bytes);
      }
    };

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_a = -CUDART_INF_F, m_b = -CUDART_INF_F, l_a = 0.f, l_b = 0.f;

    __syncwarp();                                    // every lane is done with the previous item's stages
#pragma unroll
    for (int pi = 0; pi < S - 1; ++pi) {
      if (pi < P) issue(pi);
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if (has_next) request(next_item);                // its loads run under this item's stream

    for (int ci = 0; ci < P; ++ci) {
      asm volatile("cp.async.wait_group %0;" ::"n"(S - 2) : "memory");
      __syncwarp();                                  // page ci is visible to the warp; everyone has left page ci - 1
      if (ci + S - 1 < P) issue(ci + S - 1);
      asm volatile("cp.async.commit_group;" ::: "memory");

      const uint32_t kb = ring + (ci % S) * STAGE;
      const int t0 = (p0 + ci) * PAGE;
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kb + krow + (((ks * 2 + kcb) ^ kx) << 4), b0, b1, b2, b3);
        mma_bf16(s[0], qf[ks], b0, b1);
        mma_bf16(s[1], qf[ks], b2, b3);
      }
      float mx_a = m_a, mx_b = m_b;
      if (t0 >= kv_lo && t0 + PAGE <= kv_hi) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          s[j][0] *= sc; s[j][1] *= sc;
          mx_a = fmaxf(mx_a, fmaxf(s[j][0], s[j][1]));
          if (!SMALLG) { s[j][2] *= sc; s[j][3] *= sc; mx_b = fmaxf(mx_b, fmaxf(s[j][2], s[j][3])); }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < (SMALLG ? 2 : 4); ++e) {
            const int kpos = t0 + j * 8 + (lane & 3) * 2 + (e & 1);
            const float v = (kpos < kv_hi && kpos >= kv_lo) ? s[j][e] * sc : -CUDART_INF_F;
            s[j][e] = v;
            if (e >= 2) mx_b = fmaxf(mx_b, v); else mx_a = fmaxf(mx_a, v);
          }
        }
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      const float ref_a = (mx_a == -CUDART_INF_F) ? 0.f : mx_a;
      const float al_a = (mx_a == m_a) ? 1.f : ex2a(m_a - ref_a);
      m_a = mx_a;
      float ref_b = 0.f, al_b = 1.f;
      if (!SMALLG) {
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        ref_b = (mx_b == -CUDART_INF_F) ? 0.f : mx_b;
        al_b = (mx_b == m_b) ? 1.f : ex2a(m_b - ref_b);
        m_b = mx_b;
      }
      float ps_a = 0.f, ps_b = 0.f;
      uint32_t pf[4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float q0 = ex2a(s[j][0] - ref_a), q1 = ex2a(s[j][1] - ref_a);
        ps_a += q0 + q1;
        pf[j * 2 + 0] = pack_bf16x2(q0, q1);       // accumulator layout of two adjacent n8 tiles == A fragment of a k16 step
        if (!SMALLG) {
          const float q2 = ex2a(s[j][2] - ref_b), q3 = ex2a(s[j][3] - ref_b);
          ps_b += q2 + q3;
          pf[j * 2 + 1] = pack_bf16x2(q2, q3);
        } else {
          pf[j * 2 + 1] = 0u;
        }
      }
      l_a = l_a * al_a + ps_a;
      if (!SMALLG) l_b = l_b * al_b + ps_b;
      // the running maximum seldom moves after the first pages: skip the rescale of the accumulators then
      if (__any_sync(0xffffffffu, al_a != 1.f || al_b != 1.f)) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          o[i][0] *= al_a; o[i][1] *= al_a;
          if (!SMALLG) { o[i][2] *= al_b; o[i][3] *= al_b; }
        }
      }
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(kb + vrow + (((dp * 2 + vcb) ^ vx) << 4), b0, b1, b2, b3);
        mma_bf16(o[dp * 2], pf, b0, b1);
        mma_bf16(o[dp * 2 + 1], pf, b2, b3);
      }
    }

    // ---- epilogue: the lanes of a quad share a row; fold in the partial over the other key set and store
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    if (!SMALLG) {
      l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
      l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    }
#pragma unroll
    for (int half = 0; half < (SMALLG ? 1 : 2); ++half) {
      const int gq = ra + half * 8;
      if (gq >= gn) continue;
      const int h = h0 + gq;
      const float m = half ? m_b : m_a, lt = half ? l_b : l_a;
      float mine = lt > 0.f ? 1.f / lt : 0.f;          // factor on this pass's unnormalised output
      float lse = lt > 0.f ? (m + log2f(lt)) * LN2 : -CUDART_INF_F;
      float ca = 0.f;
      const long long row = (long long)seq * a.Hq + h;
      if (mo != nullptr) {
        const float la = a.merge_lse[row];
        const float mm = fmaxf(la, lse);
        const float wa = (la == -CUDART_INF_F) ? 0.f : __expf(la - mm);
        const float wb = (lse == -CUDART_INF_F) ? 0.f : __expf(lse - mm);
        const float den = wa + wb;
        ca = den > 0.f ? wa / den : 0.f;
        mine = den > 0.f ? mine * wb / den : 0.f;
        lse = den > 0.f ? mm + __logf(den) : -CUDART_INF_F;
      }
      if (a.lse != nullptr && (lane & 3) == 0) a.lse[row] = lse;
      __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(a.out) + (long long)seq * a.o_stride + (long long)h * D;
      const int cq = (lane & 3) * 2;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        float v0 = o[i][half * 2] * mine, v1 = o[i][half * 2 + 1] * mine;
        if (mo != nullptr) {
          const uint32_t pr = *reinterpret_cast<const uint32_t*>(mo + row * D + i * 8 + cq);
          v0 += bf16_lo(pr) * ca;
          v1 += bf16_hi(pr) * ca;
        }
        *reinterpret_cast<uint32_t*>(op + i * 8 + cq) = pack_bf16x2(v0, v1);
      }
    }
    if (!has_next) break;
    item = next_item;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <int D, int S, bool SMALLG>
static int launch(const UbAttnArgs& a, cudaStream_t st, int gchunks, int n_items, int ctas) {
  constexpr int SMEM = WARPS * S * 2 * PAGE * D * 2;
  static bool attr_set[UB_MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= UB_MAX_DEVICES) return -1;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_warp_kernel<D, S, SMALLG>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return -(int)e;
    attr_set[dev] = true;
  }
  cudaError_t e = ub::launch_pdl(attn_decode_warp_kernel<D, S, SMALLG>, dim3(ctas), dim3(WARPS * 32), (size_t)SMEM, st, a,
                                 gchunks, n_items);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

static int num_sms() {
  static int sms[UB_MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= UB_MAX_DEVICES) return 148;
  if (sms[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    sms[dev] = v;
  }
  return sms[dev];
}

}  // namespace dwarp
}  // namespace ub

extern "C" int ub_attn_decode_warp_supported(const UbAttnArgs* a) {
  if (a->D != 64 && a->D != 128) return 0;
  if (a->block_size != ub::dwarp::PAGE) return 0;
  if (a->Hkv <= 0 || a->Hq % a->Hkv != 0 || a->q_stride % 2 != 0 || a->o_stride % 2 != 0) return 0;
  if (a->window > 0 || a->alibi_slopes != nullptr || a->splits != 1) return 0;
  if ((reinterpret_cast<uintptr_t>(a->q) & 3) || (reinterpret_cast<uintptr_t>(a->out) & 3) ||
      (reinterpret_cast<uintptr_t>(a->k_cache) & 15) || (reinterpret_cast<uintptr_t>(a->v_cache) & 15))
    return 0;
  if (a->merge_o != nullptr && (reinterpret_cast<uintptr_t>(a->merge_o) & 3)) return 0;
  return 1;
}

extern "C" int ub_attn_decode_warp(const UbAttnArgs* a, void* stream) {
  using namespace ub::dwarp;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int Gtot = a->Hq / a->Hkv;
  const int gchunks = (Gtot + 15) / 16;
  const int n_items = a->num_seqs * a->Hkv * gchunks;
  if (n_items <= 0) return 0;
  const int sms = num_sms();
  const bool smallg = Gtot <= 8;
  if (a->D == 64) {
    int ctas = 3 * sms;
    if (ctas * WARPS > n_items) ctas = (n_items + WARPS - 1) / WARPS;
    return smallg ? launch<64, 4, true>(*a, st, gchunks, n_items, ctas) : launch<64, 4, false>(*a, st, gchunks, n_items, ctas);
  }
  // Many items: two CTAs per SM with three stages per warp.  Fewer items than half of those warps: one CTA per SM
  // with six stages per warp, i.e. five pages in flight for each of the few streams.
  if (n_items * 2 > 2 * sms * WARPS) {
    int ctas = 2 * sms;
    if (ctas * WARPS > n_items) ctas = (n_items + WARPS - 1) / WARPS;
    return smallg ? launch<128, 3, true>(*a, st, gchunks, n_items, ctas) : launch<128, 3, false>(*a, st, gchunks, n_items, ctas);
  }
  int ctas = sms;
  if (ctas * WARPS > n_items) ctas = (n_items + WARPS - 1) / WARPS;
  return smallg ? launch<128, 6, true>(*a, st, gchunks, n_items, ctas) : launch<128, 6, false>(*a, st, gchunks, n_items, ctas);
}
