// K3: paged prefill ("flash") attention over block tables, ragged batch, GQA-packed.
//
// Work unit: 64 packed query rows of one (sequence, kv head).  A packed row is (token, head in the
// GQA group), so one K/V tile fetched into shared memory serves all G query heads of the group.
// K/V tiles of 64 tokens (four 16-token pages, gathered through the block table with 16-byte
// cp.async) are double-buffered; scores never leave registers (online softmax, exp2 domain).
// Masks are predicates on (query position, key position): causal with offset for chunked prefill
// and prefix-cache hits, sliding window, ALiBi, and kv_start for suffix-only passes.  Optionally
// returns the log-sum-exp so partial results over disjoint key sets can be merged (cascade
// attention over a shared radix prefix; split-KV).
//
// This kernel uses warp-level mma (m16n8k16) with fp32 accumulation; the GEMM-shaped bulk of the
// model runs on tcgen05 (csrc/gemm).  Head dims 64 and 128.
//
// Replaces in the reference: ops_fn::flash_attention (crates/runtime/src/tensor_core.rs:1318-1383,
// which materialises the full score matrix and a host-built mask) and the prefill case of
// LlamaAttention::forward_with_cache (crates/runtime/src/models_v2/llama.rs:1109-1143).
#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"
#include <math_constants.h>
#include <stdlib.h>

namespace ub {

constexpr float P_LOG2E = 1.4426950408889634f;
constexpr float P_LN2 = 0.6931471805599453f;
constexpr int QT = 64;   // packed query rows per CTA
constexpr int KT = 64;   // kv tokens per tile

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool pred) {
  const uint32_t d = smem_u32(smem_dst);
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

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

// smem tile [rows][D] bf16 with 16-byte chunks XOR-swizzled by (row & 7)
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

template <int D>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const UbAttnArgs a) {
  constexpr int CPR = D / 8;  // 16-byte chunks per row
  extern __shared__ __align__(128) uint8_t smem_p[];
  uint8_t* q_sm = smem_p;                    // [QT][D]
  uint8_t* k_sm = q_sm + QT * D * 2;         // [2][KT][D]
  uint8_t* v_sm = k_sm + 2 * KT * D * 2;     // [2][KT][D]

  const int seq = blockIdx.z, kvh = blockIdx.y;
  const int G = a.Hq / a.Hkv;
  const int qs = a.q_start != nullptr ? a.q_start[seq] : seq;
  const int q_len = a.q_start != nullptr ? a.q_start[seq + 1] - qs : 1;
  const int rows_total = q_len * G;
  const int row0 = blockIdx.x * QT;
  if (row0 >= rows_total) return;
  const int kv_len = a.seq_lens[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* bt = a.block_tables + (long long)seq * a.max_blocks_per_seq;
  const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(a.k_cache);
  const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(a.v_cache);
  const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(a.q);

  // ---- load the Q tile (packed rows) ----
  for (int i = threadIdx.x; i < QT * CPR; i += 128) {
    const int r = i / CPR, c = i % CPR;
    const int row = row0 + r;
    const bool ok = row < rows_total;
    const int tok = ok ? row / G : 0, hg = ok ? row % G : 0;
    const __nv_bfloat16* src = qg + (long long)(qs + tok) * a.q_stride + (long long)(kvh * G + hg) * D + c * 8;
    cp_async16(q_sm + tile_off<D>(r, c), src, ok);
  }
  cp_async_commit();

  // kv range needed by this tile
  const int last_row = min(row0 + QT, rows_total) - 1;
  const int first_qpos = kv_len - q_len + row0 / G;
  const int last_qpos = kv_len - q_len + last_row / G;
  int kv_end = a.causal ? min(kv_len, last_qpos + 1) : kv_len;
  int kv_begin = max(a.kv_start, 0);
  if (a.window > 0) kv_begin = max(kv_begin, first_qpos - a.window + 1);
  kv_begin = kv_begin / KT * KT;
  const int ntiles = kv_end > kv_begin ? (kv_end - kv_begin + KT - 1) / KT : 0;

  auto load_kv = [&](int tile, int buf) {
    const int t0 = kv_begin + tile * KT;
    for (int i = threadIdx.x; i < KT * CPR; i += 128) {
      const int r = i / CPR, c = i % CPR;
      const int pos = t0 + r;
      bool ok = pos < kv_end;
      long long off = 0;
      if (ok) {
        const int bi = pos / a.block_size;
        const int blk = bi < a.max_blocks_per_seq ? bt[bi] : -1;
        if (blk < 0 || blk >= a.num_blocks) {
          set_err(a.err, ERR_BOUNDS, seq);
          ok = false;
        } else {
          off = (((long long)blk * a.Hkv + kvh) * a.block_size + (pos % a.block_size)) * D + c * 8;
        }
      }
      cp_async16(k_sm + buf * KT * D * 2 + tile_off<D>(r, c), kc + off, ok);
      cp_async16(v_sm + buf * KT * D * 2 + tile_off<D>(r, c), vc + off, ok);
    }
  };

  if (ntiles > 0) load_kv(0, 0);
  cp_async_commit();

  // per-thread row bookkeeping: this thread owns rows r_a = warp*16 + lane/4 and r_b = r_a + 8
  const int ra = warp * 16 + (lane >> 2), rb = ra + 8;
  const int rowa = row0 + ra, rowb = row0 + rb;
  const int qpos_a = kv_len - q_len + min(rowa, rows_total - 1) / G;
  const int qpos_b = kv_len - q_len + min(rowb, rows_total - 1) / G;
  float slope_a = 0.f, slope_b = 0.f;
  if (a.alibi_slopes != nullptr) {
    slope_a = a.alibi_slopes[kvh * G + min(rowa, rows_total - 1) % G] * P_LOG2E;
    slope_b = a.alibi_slopes[kvh * G + min(rowb, rows_total - 1) % G] * P_LOG2E;
  }
  const float sc = a.scale * P_LOG2E;

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_a = -CUDART_INF_F, m_b = -CUDART_INF_F, l_a = 0.f, l_b = 0.f;

  cp_async_wait<1>();  // Q has landed (first kv tile may still be in flight)
  __syncthreads();
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int c = ks * 2 + (lane >> 4);
    ldsm_x4(smem_u32(q_sm + tile_off<D>(r, c)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }

  for (int tile = 0; tile < ntiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < ntiles) load_kv(tile + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint8_t* kb = k_sm + buf * KT * D * 2;
    const uint8_t* vb = v_sm + buf * KT * D * 2;
    const int t0 = kv_begin + tile * KT;

    // S = Q K^T  (16 x 64 per warp)
    float s[KT / 8][4];
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int jp = 0; jp < KT / 16; ++jp) {
        const int mi = lane >> 3;
        const int r = jp * 16 + (mi >> 1) * 8 + (lane & 7);
        const int c = ks * 2 + (mi & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(kb + tile_off<D>(r, c)), b0, b1, b2, b3);
        mma_bf16(s[jp * 2], qf[ks], b0, b1);
        mma_bf16(s[jp * 2 + 1], qf[ks], b2, b3);
      }
    }
    // scale, mask, online softmax
    float mx_a = m_a, mx_b = m_b;
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kpos = t0 + j * 8 + (lane & 3) * 2 + (e & 1);
        const bool rowsel_b = e >= 2;
        const int qpos = rowsel_b ? qpos_b : qpos_a;
        bool vis = kpos < kv_end && kpos >= a.kv_start;
        if (a.causal) vis = vis && kpos <= qpos;
        if (a.window > 0) vis = vis && kpos > qpos - a.window;
        float v = s[j][e] * sc + (rowsel_b ? slope_b : slope_a) * (float)(kpos - qpos);
        v = vis ? v : -CUDART_INF_F;
        s[j][e] = v;
        if (rowsel_b) mx_b = fmaxf(mx_b, v); else mx_a = fmaxf(mx_a, v);
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
    uint32_t pf[KT / 16][4];
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) {
      const float p0 = (s[j][0] == -CUDART_INF_F) ? 0.f : exp2f(s[j][0] - mx_a);
      const float p1 = (s[j][1] == -CUDART_INF_F) ? 0.f : exp2f(s[j][1] - mx_a);
      const float p2 = (s[j][2] == -CUDART_INF_F) ? 0.f : exp2f(s[j][2] - mx_b);
      const float p3 = (s[j][3] == -CUDART_INF_F) ? 0.f : exp2f(s[j][3] - mx_b);
      ps_a += p0 + p1; ps_b += p2 + p3;
      // accumulator layout of two adjacent n8 tiles == A fragment of one k16 step
      pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16x2(p0, p1);
      pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16x2(p2, p3);
    }
    l_a = l_a * al_a + ps_a;
    l_b = l_b * al_b + ps_b;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b; }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        const int mi = lane >> 3;
        const int r = kk * 16 + (mi & 1) * 8 + (lane & 7);
        const int c = dp * 2 + (mi >> 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(vb + tile_off<D>(r, c)), b0, b1, b2, b3);
        mma_bf16(o[dp * 2], pf[kk], b0, b1);
        mma_bf16(o[dp * 2 + 1], pf[kk], b2, b3);
      }
    }
    __syncthreads();  // everyone is done with `buf` before the next iteration overwrites it
  }
  cp_async_wait<0>();

  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
  __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(a.out);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = half ? rowb : rowa;
    if (row >= rows_total) continue;
    const int tok = row / G, hg = row % G;
    const float inv = half ? inv_b : inv_a;
    __nv_bfloat16* dst = og + (long long)(qs + tok) * a.o_stride + (long long)(kvh * G + hg) * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int d = i * 8 + (lane & 3) * 2;
      *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16x2(o[i][half * 2] * inv, o[i][half * 2 + 1] * inv);
    }
    if ((lane & 3) == 0 && a.lse != nullptr) {
      const float l = half ? l_b : l_a, m = half ? m_b : m_a;
      a.lse[(long long)(qs + tok) * a.Hq + kvh * G + hg] = l > 0.f ? (m + log2f(l)) * P_LN2 : -CUDART_INF_F;
    }
  }
}

template <int D>
static int launch_prefill(const UbAttnArgs& a, cudaStream_t st) {
  const int G = a.Hq / a.Hkv;
  const size_t smem = (size_t)(QT + 4 * KT) * D * 2;
  static bool attr_set[UB_MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < UB_MAX_DEVICES && !attr_set[dev]) {
    cudaFuncSetAttribute(attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set[dev] = true;
  }
  dim3 grid(((long long)a.max_q_len * G + QT - 1) / QT, a.Hkv, a.num_seqs);
  attn_prefill_kernel<D><<<grid, 128, smem, st>>>(a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

}  // namespace ub

extern "C" int ub_attn_prefill_tc_supported(const UbAttnArgs* a);
extern "C" int ub_attn_prefill_tc(const UbAttnArgs* a, void* stream);

// UB_ATTN_TC=0 keeps every problem on the warp-MMA kernel (A/B comparisons).
static bool tc_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("UB_ATTN_TC");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

static int g_last_path = 0;   // 1: tcgen05 kernel, 2: warp-MMA kernel (what the last call on this host thread used)
extern "C" int ub_attn_prefill_last_path() { return g_last_path; }

extern "C" int ub_attn_prefill(const UbAttnArgs* a, void* stream_v) {
  using namespace ub;
  if (a->num_seqs <= 0 || a->max_q_len <= 0) return 0;
  if (tc_enabled() && ub_attn_prefill_tc_supported(a)) {
    g_last_path = 1;
    return ub_attn_prefill_tc(a, stream_v);
  }
  if (a->merge_o != nullptr || a->splits > 1) return -7;   // fused merge and key split live in the tensor-core kernel only
  g_last_path = 2;
  if (a->Hq % a->Hkv != 0) return -2;
  if (a->q_stride % 8 != 0) return -3;
  cudaStream_t st = (cudaStream_t)stream_v;
  switch (a->D) {
    case 64: return launch_prefill<64>(*a, st);
    case 128: return launch_prefill<128>(*a, st);
    default: return -4;
  }
}
