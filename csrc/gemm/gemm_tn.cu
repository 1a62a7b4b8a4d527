// K1/K2/F1/F3: bf16 "TN" GEMM on 5th-gen tensor cores:  out[M, N] = epilogue(x[M, K] @ w[N, K]^T).
//
// Design (sm_100a only):
//  * Weights stay in the on-disk HF layout [out_features, in_features]; both operands are K-major.
//  * The weight tile is ALWAYS the 128-row MMA "A" operand and the token tile is the MMA "N"
//    operand (16..256 tokens).  A decode batch of 16 tokens and a prefill chunk of 8192 tokens
//    run the same kernel; only the token-tile width changes.  The accumulator in TMEM therefore
//    holds out^T: TMEM lane = output feature, TMEM column = token.
//  * Warp roles: warp 0 = TMA producer, warp 1 = tcgen05.mma issuer and TMEM owner,
//    warps 2..9 = epilogue (TMEM -> registers -> smem transpose -> 16-byte global stores) in two groups of four:
//    a warp may read one quarter of the TMEM lanes, so two warps share every quarter and take alternate 32-token
//    chunks of the accumulator (the exposed epilogue of a single-tile CTA halves).
//  * Two scheduling modes share the main loop:
//      - PERSISTENT: one CTA per SM walks a static list of output tiles; the accumulator is
//        double-buffered in TMEM so the epilogue of tile i overlaps the MMAs of tile i+1.
//      - SPLIT-K: when there are far fewer tiles than SMs (decode, tensor-parallel shards) a
//        thread-block cluster of S CTAs shares one tile, each CTA reduces 1/S of K, and the
//        partial accumulators are summed through distributed shared memory in a fixed order
//        (deterministic, no global workspace, no atomics).  TMA loads are per-CTA (no multicast).
//  * DUAL mode (K2): two weight tiles (gate rows, up rows) share one token tile and fill two
//    accumulators; the epilogue writes act(gate) * up, so SwiGLU/GeGLU never touches HBM.
//  * Collective fusion.  F1 (GEMM + reduce-scatter): the epilogue stores each output row straight
//    into the symmetric receive buffer of the rank that owns that token (peer pointer, plain
//    16-byte stores over NVLink), then every CTA bumps a counter on every peer.  F3 (all-gather +
//    GEMM): the TMA producer waits (bounded) on the per-source counters before it loads token rows
//    that another rank pushed into this rank's gather buffer.
//  * Every wait is bounded; a timeout sets the error word and the kernel drains and frees TMEM.
//
// Replaces in the reference: ops_fn::matmul (crates/runtime/src/tensor_core.rs:843-892), the
// QMatMul call sites (models_v2/llama.rs:1184-1195) and fused_swiglu (tensor_core.rs:1385-1396).
#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"
#include <stdlib.h>
#include <mutex>

namespace ub {

constexpr int BM_W = 128;  // weight rows per tile (MMA M)
constexpr int BK = 64;     // K elements per stage (one 128-byte swizzle atom of bf16)
constexpr int UMMA_K = 16;
constexpr int STAGING_BYTES = 16 * 1024;  // epilogue staging: one [32][128] bf16 (or [16][128] fp32) buffer per epilogue group
constexpr int EPI_THREADS = 256;          // eight epilogue warps: two per TMEM lane quarter, taking alternate 32-token chunks
constexpr int GEMM_THREADS = 64 + EPI_THREADS;

struct GemmParams {
  int M, N, K;
  __nv_bfloat16* out;
  long long ldo;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null
  long long ldr;
  int act;          // UB_ACT_*
  int up_row_off;   // DUAL: row offset of the "up" half inside w
  int out_f32;      // 1: out is float* (ldo in floats)
  float out_scale;  // multiplies the accumulator before bias / activation
  int* err;
  int splits;       // SPLIT-K: cluster size
  // F1: reduce-scatter push.  rs_world == 0 disables.
  int rs_world, rs_rank, rs_rows_per_rank;
  __nv_bfloat16* rs_peer_out[UB_MAX_RANKS];  // each: [world][rows_per_rank][ldo]
  uint32_t* rs_peer_flag[UB_MAX_RANKS];      // counter to bump on each peer
  uint32_t* rs_local_count;                  // local arrival counter of this use (see publish_to_peers)
  uint32_t rs_total;                         // CTAs that arrive on it per use
  // F3: all-gather wait.  ag_world == 0 disables.
  int ag_world, ag_rows_per_rank;
  const uint32_t* ag_flags;     // [world] counters in local memory, one per source rank
  const uint32_t* ag_epoch;     // unused (kept for ABI stability)
  uint32_t ag_signals_per_use;  // counter increments per source rank per use
  // K13 grouped mode (MoE experts).  grp_tiles == null disables.  One int4 per token tile:
  // {expert (-1: no work), first row, end row, unused}; rows index the expert-sorted activation matrix.
  const int4* grp_tiles;
  int grp_max_tiles;  // token-tile slots in the table
  int grp_w_rows;     // rows of w per expert; expert e's weights are rows [e*grp_w_rows, (e+1)*grp_w_rows)
  int tile_begin, tile_end;   // work units of this launch; tile_end == 0 means all
  // Stream-K schedule of the CTA-pair kernel (sk_on != 0, see PairWalk): teams of pairs take equal shares of the (weight
  // row, k-block) space; partial tiles are summed through sk_ws (fp32, one slot per CTA) under sk_flags (one per CTA).
  int sk_on;
  float* sk_ws;
  uint32_t* sk_flags;
  int dbg;                    // UB_GEMM_DEBUG bits: 1 = no L2 prefetch, 2 = no L2 cache hints
};

// Coordinates of work unit u.  m0/m_end: token rows; nw: row of the weight tile in w; no: first output feature.
struct TileCoord { int m0, m_end, nw, no; bool valid; };
__device__ __forceinline__ TileCoord tile_coord(const GemmParams& p, int u, int num_m, int tn) {
  TileCoord c;
  const int mt = u % num_m, wn = u / num_m;
  c.no = wn * BM_W;
  if (p.grp_tiles == nullptr) {
    c.m0 = mt * tn; c.m_end = p.M; c.nw = c.no; c.valid = true;
  } else {
    const int4 t = __ldg(p.grp_tiles + mt);
    c.valid = t.x >= 0;
    c.m0 = t.y; c.m_end = t.z; c.nw = t.x * p.grp_w_rows + c.no;
  }
  return c;
}

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case UB_ACT_SILU: {
      // v * sigmoid(v) with sigmoid(v) = 0.5 * (1 + tanh(v / 2)): one MUFU instruction, no division
      float t;
      asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * v));
      return v * fmaf(0.5f, t, 0.5f);
    }
    case UB_ACT_GELU: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    case UB_ACT_GELU_TANH: {
      float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
      return 0.5f * v * (1.f + tanhf(u));
    }
    case UB_ACT_RELU: return fmaxf(v, 0.f);
    case UB_ACT_RELU2: { float r = fmaxf(v, 0.f); return r * r; }
    case UB_ACT_QUICK_GELU: return v / (1.f + __expf(-1.702f * v));
    case UB_ACT_SIGMOID: return 1.f / (1.f + __expf(-v));
    case UB_ACT_TANH: return tanhf(v);
    default: return v;
  }
}

// The activation is chosen ONCE per chunk of accumulator values: a switch inside the per-value loop makes the
// compiler evaluate every branch (erf, tanh, exp ...) for every value, which dominated the epilogue.
template <int N, bool DUAL, int ACT>
__device__ __forceinline__ void epi_values_t(uint32_t (&r)[N], const uint32_t (&r2)[N], float scale, float bias_v) {
  // The two hot forms run on packed fp32x2 instructions (the epilogue warps are bound by instruction issue):
  // silu(gate) * up with sigmoid(v) = 0.5 * (1 + tanh(v / 2)), four instructions per value instead of seven, and the
  // plain scale-and-bias as one multiply-add per two values.
  if constexpr (DUAL && ACT == UB_ACT_SILU) {
    const uint64_t s2 = pack_f32x2(scale, scale), h2 = pack_f32x2(0.5f, 0.5f);
#pragma unroll
    for (int j = 0; j < N; j += 2) {
      const uint64_t g = mul_f32x2(pack_f32x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), s2);
      const uint64_t u = mul_f32x2(pack_f32x2(__uint_as_float(r2[j]), __uint_as_float(r2[j + 1])), s2);
      float a0, a1, t0, t1, o0, o1;
      unpack_f32x2(mul_f32x2(g, h2), a0, a1);
      asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(a0));
      asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(a1));
      const uint64_t sig = fma_f32x2(pack_f32x2(t0, t1), h2, h2);
      unpack_f32x2(mul_f32x2(mul_f32x2(g, sig), u), o0, o1);
      r[j] = __float_as_uint(o0);
      r[j + 1] = __float_as_uint(o1);
    }
    return;
  }
  if constexpr (!DUAL && ACT == UB_ACT_NONE) {
    const uint64_t s2 = pack_f32x2(scale, scale), b2 = pack_f32x2(bias_v, bias_v);
#pragma unroll
    for (int j = 0; j < N; j += 2) {
      float o0, o1;
      unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), s2, b2), o0, o1);
      r[j] = __float_as_uint(o0);
      r[j + 1] = __float_as_uint(o1);
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < N; ++j) {
    float v = __uint_as_float(r[j]) * scale;
    if (DUAL) v = apply_act(v, ACT) * (__uint_as_float(r2[j]) * scale);
    else v = apply_act(v + bias_v, ACT);
    r[j] = __float_as_uint(v);
  }
}
template <int N, bool DUAL>
__device__ __forceinline__ void epi_values(uint32_t (&r)[N], const uint32_t (&r2)[N], float scale, float bias_v, int act) {
  switch (act) {
    case UB_ACT_NONE: epi_values_t<N, DUAL, UB_ACT_NONE>(r, r2, scale, bias_v); break;
    case UB_ACT_SILU: epi_values_t<N, DUAL, UB_ACT_SILU>(r, r2, scale, bias_v); break;
    case UB_ACT_GELU: epi_values_t<N, DUAL, UB_ACT_GELU>(r, r2, scale, bias_v); break;
    case UB_ACT_GELU_TANH: epi_values_t<N, DUAL, UB_ACT_GELU_TANH>(r, r2, scale, bias_v); break;
    case UB_ACT_RELU: epi_values_t<N, DUAL, UB_ACT_RELU>(r, r2, scale, bias_v); break;
    case UB_ACT_RELU2: epi_values_t<N, DUAL, UB_ACT_RELU2>(r, r2, scale, bias_v); break;
    case UB_ACT_QUICK_GELU: epi_values_t<N, DUAL, UB_ACT_QUICK_GELU>(r, r2, scale, bias_v); break;
    case UB_ACT_SIGMOID: epi_values_t<N, DUAL, UB_ACT_SIGMOID>(r, r2, scale, bias_v); break;
    case UB_ACT_TANH: epi_values_t<N, DUAL, UB_ACT_TANH>(r, r2, scale, bias_v); break;
    default: epi_values_t<N, DUAL, UB_ACT_NONE>(r, r2, scale, bias_v); break;
  }
}

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add_u32(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}

template <int TN, int STAGES, bool DUAL, bool SPLITK>
struct GemmSmem {
  static constexpr int A_BYTES = BM_W * BK * 2;  // 16 KB
  static constexpr int B_BYTES = TN * BK * 2;
  static constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * A_BYTES + B_BYTES;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  // SPLIT-K parks its fp32 partial tile on top of the (then idle) pipeline stages.
  static constexpr int PARTIAL_BYTES = (DUAL ? 2 : 1) * (TN + 8) * BM_W * 4;   // splits x ceil(TN / splits) rows, splits <= 8
  static constexpr int DATA_BYTES = SPLITK ? (TILE_BYTES > PARTIAL_BYTES ? TILE_BYTES : PARTIAL_BYTES)
                                           : TILE_BYTES + STAGING_BYTES;
  static constexpr int TOTAL = DATA_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
  static_assert(TOTAL <= 227 * 1024, "shared memory budget exceeded");
};

// Final stage of every epilogue: 8 consecutive features of one token row.
__device__ __forceinline__ void emit8(const GemmParams& p, int m, int m_end, int nn, float (&v)[8], bool vec_ok) {
  if (m >= m_end || nn >= p.N) return;
  if (p.residual != nullptr) {
    if (vec_ok) {
      const uint4 rr = *reinterpret_cast<const uint4*>(p.residual + (long long)m * p.ldr + nn);
      const uint32_t* b = reinterpret_cast<const uint32_t*>(&rr);
#pragma unroll
      for (int e = 0; e < 4; ++e) { v[2 * e] += bf16_lo(b[e]); v[2 * e + 1] += bf16_hi(b[e]); }
    } else {
      for (int e = 0; e < 8 && nn + e < p.N; ++e) v[e] += __bfloat162float(p.residual[(long long)m * p.ldr + nn + e]);
    }
  }
  if (p.out_f32) {
    float* dst = reinterpret_cast<float*>(p.out) + (long long)m * p.ldo + nn;
    if (nn + 8 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
      *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      for (int e = 0; e < 8 && nn + e < p.N; ++e) dst[e] = v[e];
    }
    return;
  }
  __nv_bfloat16* dst_base = p.out;
  long long row = m;
  if (p.rs_world > 0 && p.rs_peer_out[0] != nullptr) {
    // (with a null rs_peer_out the partial rows stay in `out`, which the consumers read through the multicast address)
    int owner = m / p.rs_rows_per_rank;
    if (owner >= p.rs_world) owner = p.rs_world - 1;
    dst_base = p.rs_peer_out[owner];
    row = (long long)p.rs_rank * p.rs_rows_per_rank + (m - owner * p.rs_rows_per_rank);
  }
  __nv_bfloat16* dst = dst_base + row * p.ldo + nn;
  if (vec_ok) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                                pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
  } else {
    for (int e = 0; e < 8 && nn + e < p.N; ++e) dst[e] = __float2bfloat16(v[e]);
  }
}

// Optional timeline of one launch (UB_GEMM_DEBUG bit 4): each CTA of the 1-CTA kernel records the global timer at a few
// points of its first tile; ub_gemm_debug_timeline copies the table out.  Slots: 0 kernel entry, 1 setup done,
// 2 first operand stage landed, 3 last MMA of the first tile issued, 4 accumulator complete, 5 epilogue stores
// issued, 6 split-K reduction done (or 0), 7 CTA exit, 8 first cluster barrier passed, 9 partial rows pushed,
// 10 second cluster barrier passed (8-10: split-K only).
constexpr int TS_CTAS = 512;
__device__ unsigned long long g_gemm_ts[TS_CTAS][12];
__device__ __forceinline__ void ts_mark(const GemmParams& p, int slot) {
  if (p.dbg & 4) {
    const unsigned cta = blockIdx.x + gridDim.x * blockIdx.y;
    if (cta < TS_CTAS) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
      g_gemm_ts[cta][slot] = t;
    }
  }
}

// Split-K finish.  The CTAs of a cluster hold partial accumulators of the same tile; CTA d of the cluster finishes the
// token rows [d * per, (d + 1) * per).  Every CTA PUSHES its partial rows into a slot of the owner's shared memory
// (slot = sender's split index) with distributed-shared-memory stores, which are fire-and-forget; after one cluster
// barrier each owner sums its slots with local loads and runs the epilogue.  (Pulling the partials with remote
// loads instead cost 10 us per 128 x 256 tile: every load pays the SM-to-SM round trip.)  The slots overlay the
// pipeline stages, so the pushes start only after a cluster barrier that follows everybody's last MMA.
// Slot layout in the owner: [splits][per][128] floats, then the same again for the up half of a gated GEMM.
__device__ __forceinline__ void st_dsmem_f32(uint32_t addr, uint32_t bits) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(addr), "r"(bits) : "memory");
}

template <int TN, int CH, bool DUAL>
__device__ __forceinline__ void splitk_scatter(const GemmParams& p, uint32_t smem_base, uint32_t lane_addr, int et,
                                               int my_split, uint32_t rank_stride, uint32_t rank_off, int grp) {
  const int S = p.splits, per = (TN + S - 1) / S;
  const uint32_t up_off = uint32_t(S * per) * BM_W * 4u;
#pragma unroll 1
  for (int c = grp; c < TN / CH; c += 2) {
    uint32_t r[CH], r2[CH];
    if constexpr (CH == 32) {
      tmem_ld_32x32(lane_addr + c * CH, r);
      if (DUAL) tmem_ld_32x32(lane_addr + TN + c * CH, r2);
    } else {
      tmem_ld_32x16(lane_addr + c * CH, r);
      if (DUAL) tmem_ld_32x16(lane_addr + TN + c * CH, r2);
    }
    tmem_ld_wait();
    int d = (c * CH) / per;
    int next = (d + 1) * per;
    uint32_t win = mapa_u32(smem_base, uint32_t(d) * rank_stride + rank_off);
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const int tok = c * CH + j;
      if (tok >= next) {
        ++d;
        next += per;
        win = mapa_u32(smem_base, uint32_t(d) * rank_stride + rank_off);
      }
      const uint32_t off = uint32_t((my_split * per + (tok - (next - per))) * BM_W + et) * 4u;
      st_dsmem_f32(win + off, r[j]);
      if (DUAL) st_dsmem_f32(win + up_off + off, r2[j]);
    }
  }
}

template <bool DUAL, int ACT>
__device__ __forceinline__ void splitk_finish_t(const GemmParams& p, const uint8_t* smem, int tn, int r0, int r1, int tid_e,
                                                int m0, int n0, bool vec_ok) {
  const int S = p.splits, per = (tn + S - 1) / S;
  const float* part = reinterpret_cast<const float*>(smem);
  const float* part_up = part + (size_t)S * per * BM_W;
  const int n_items = (r1 - r0) * 16;
  for (int idx = tid_e; idx < n_items; idx += EPI_THREADS) {
    const int lt = idx >> 4, c8 = idx & 15;
    float g[8] = {0, 0, 0, 0, 0, 0, 0, 0}, up[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int sp = 0; sp < S; ++sp) {
      const float* src = part + ((size_t)(sp * per + lt) * BM_W + c8 * 8);
      const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
      g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w; g[4] += b.x; g[5] += b.y; g[6] += b.z; g[7] += b.w;
      if (DUAL) {
        const float* su = part_up + ((size_t)(sp * per + lt) * BM_W + c8 * 8);
        const float4 c = *reinterpret_cast<const float4*>(su), d = *reinterpret_cast<const float4*>(su + 4);
        up[0] += c.x; up[1] += c.y; up[2] += c.z; up[3] += c.w; up[4] += d.x; up[5] += d.y; up[6] += d.z; up[7] += d.w;
      }
    }
    const int nn = n0 + c8 * 8;
    uint32_t gv[8], uv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float x = g[e];
      if (!DUAL && p.bias != nullptr && nn + e < p.N) x += __bfloat162float(p.bias[nn + e]) / p.out_scale;
      gv[e] = __float_as_uint(x);
      uv[e] = __float_as_uint(up[e]);
    }
    epi_values_t<8, DUAL, ACT>(gv, uv, p.out_scale, 0.f);
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(gv[e]);
    emit8(p, m0 + r0 + lt, p.M, nn, v, vec_ok);
  }
}

// The activation is chosen once, outside the loop over output rows: with the switch inside, the compiler turned the
// eight-value bodies into predicated code that evaluated every activation for every value (880 cycles per 8 outputs).
template <bool DUAL>
__device__ __forceinline__ void splitk_finish(const GemmParams& p, const uint8_t* smem, int tn, int r0, int r1, int tid_e,
                                              int m0, int n0, bool vec_ok) {
  switch (p.act) {
    case UB_ACT_SILU: splitk_finish_t<DUAL, UB_ACT_SILU>(p, smem, tn, r0, r1, tid_e, m0, n0, vec_ok); break;
    case UB_ACT_GELU: splitk_finish_t<DUAL, UB_ACT_GELU>(p, smem, tn, r0, r1, tid_e, m0, n0, vec_ok); break;
    case UB_ACT_GELU_TANH: splitk_finish_t<DUAL, UB_ACT_GELU_TANH>(p, smem, tn, r0, r1, tid_e, m0, n0, vec_ok); break;
    case UB_ACT_RELU: splitk_finish_t<DUAL, UB_ACT_RELU>(p, smem, tn, r0, r1, tid_e, m0, n0, vec_ok); break;
    case UB_ACT_RELU2: splitk_finish_t<DUAL, UB_ACT_RELU2>(p, smem, tn, r0, r1, tid_e, m0, n0, vec_ok); break;
    case UB_ACT_QUICK_GELU: splitk_finish_t<DUAL, UB_ACT_QUICK_GELU>(p, smem, tn, r0, r1, tid_e, m0, n0, vec_ok); break;
    case UB_ACT_SIGMOID: splitk_finish_t<DUAL, UB_ACT_SIGMOID>(p, smem, tn, r0, r1, tid_e, m0, n0, vec_ok); break;
    case UB_ACT_TANH: splitk_finish_t<DUAL, UB_ACT_TANH>(p, smem, tn, r0, r1, tid_e, m0, n0, vec_ok); break;
    default: splitk_finish_t<DUAL, UB_ACT_NONE>(p, smem, tn, r0, r1, tid_e, m0, n0, vec_ok); break;
  }
}

template <int TN, int STAGES, bool DUAL, bool SPLITK>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const GemmParams p) {
  using S = GemmSmem<TN, STAGES, DUAL, SPLITK>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::DATA_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;   // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = p.grp_tiles != nullptr ? p.grp_max_tiles : (p.M + TN - 1) / TN;
  const int num_n = (p.N + BM_W - 1) / BM_W;
  // [tile_begin, tile_end) is this launch's share of the num_m * num_n work units (two-phase schedule, see plan_gemm)
  const int tile_begin = p.tile_begin;
  const int total_tiles = p.tile_end > 0 ? p.tile_end : num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t ACC_COLS = (DUAL ? 2 : 1) * TN;
  // Two accumulator buffers when they fit in the 512 TMEM columns (epilogue overlaps the next tile's MMAs).
  constexpr int NBUF = (SPLITK || 2 * ACC_COLS > 512) ? 1 : 2;
  constexpr uint32_t NEED_COLS = NBUF * ACC_COLS;
  constexpr uint32_t TMEM_COLS = NEED_COLS < 32 ? 32 : NEED_COLS;
  static_assert(TMEM_COLS <= 512, "TMEM budget exceeded");

  // Work assignment.
  int unit_begin, unit_step, kb0 = 0, kb1 = num_kb, crank = 0;
  if (SPLITK) {
    crank = blockIdx.x;  // cluster = (splits, 1, 1) and gridDim.x == splits
    unit_begin = tile_begin + blockIdx.y;
    unit_step = 1 << 30;  // exactly one tile per cluster
    const int per = (num_kb + p.splits - 1) / p.splits;
    kb0 = crank * per;
    kb1 = min(num_kb, kb0 + per);
  } else {
    unit_begin = tile_begin + blockIdx.x;
    unit_step = gridDim.x;
  }

  if (threadIdx.x == 0) {
    ts_mark(p, 0);
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], EPI_THREADS);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: this CTA owns its TMEM columns and barriers now, so the next kernel's CTAs may be
  // scheduled; nothing global has been touched yet, and nothing is before the previous kernel has completed.
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) ts_mark(p, 1);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      uint32_t ag_ready = 0;  // bitmask of source ranks already seen complete
      int it = 0;
      bool dead = false;
      constexpr int PF = 12;                 // L2 prefetch distance in k-blocks
      int pf_issued = 0, pf_u = unit_begin, pf_kb = kb0, pf_n0 = 0;
      bool pf_valid = true;
      for (int u = unit_begin; u < total_tiles && !dead; u += unit_step) {
        const TileCoord tc = tile_coord(p, u, num_m, TN);
        if (!tc.valid) continue;
        const int m0 = tc.m0, n0 = tc.nw;
        if (p.ag_world > 0) {
          // Token rows [m0, m0+TN) were pushed by the ranks that own them; wait for those sources.
          // Counters are zeroed by the consumer side between uses (see csrc/norm/norm.cu), so the target is
          // simply the number of producer CTAs of one use.
          const uint32_t want = p.ag_signals_per_use;
          const int r_lo = m0 / p.ag_rows_per_rank;
          int r_hi = (min(m0 + TN, p.M) - 1) / p.ag_rows_per_rank;
          if (r_hi >= p.ag_world) r_hi = p.ag_world - 1;
          const uint64_t t0 = wait_ticks();
          bool waited = false;
          for (int r = r_lo; r <= r_hi; ++r) {
            if (ag_ready >> r & 1u) continue;
            uint32_t spin = 0;
            while (int32_t(ld_acquire_sys_u32(p.ag_flags + r) - want) < 0) {
              if ((++spin & 31u) == 0 && wait_expired(t0, p.err)) {
                *abort_flag = 1;
                set_err(p.err, ERR_FLAG_TIMEOUT, r);
                break;
              }
            }
            ag_ready |= 1u << r;
            waited = true;
          }
          if (waited) asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          // Weights come from HBM (about 2 us away under load) while the few smem stages cover far less
          // time than that: ask L2 for the weight tile PF k-blocks ahead, so the smem copies hit in L2.
          for (; pf_issued < it + PF + 1; ++pf_issued) {
            if (pf_u >= total_tiles || (p.dbg & 1)) break;
            if (pf_kb == kb0) {
              const TileCoord pc = tile_coord(p, pf_u, num_m, TN);
              pf_valid = pc.valid;
              pf_n0 = pc.nw;
              if (!pf_valid) { pf_u += unit_step; --pf_issued; continue; }
            }
            tma_prefetch_l2_2d(&tmap_w, pf_kb * BK, pf_n0);
            if (DUAL) tma_prefetch_l2_2d(&tmap_w, pf_kb * BK, pf_n0 + p.up_row_off);
            if (++pf_kb >= kb1) { pf_kb = kb0; pf_u += unit_step; }
          }
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.err, 100 + s)) { dead = true; break; }
          uint8_t* st = smem + s * S::STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], S::STAGE_BYTES);
          if (p.dbg & 2) {
            tma_load_2d(st, &tmap_w, &full_bar[s], kb * BK, n0);
            if (DUAL) tma_load_2d(st + S::A_BYTES, &tmap_w, &full_bar[s], kb * BK, n0 + p.up_row_off);
            tma_load_2d(st + (DUAL ? 2 : 1) * S::A_BYTES, &tmap_x, &full_bar[s], kb * BK, m0);
          } else {
            tma_load_2d_hint(st, &tmap_w, &full_bar[s], kb * BK, n0, pol_w);
            if (DUAL) tma_load_2d_hint(st + S::A_BYTES, &tmap_w, &full_bar[s], kb * BK, n0 + p.up_row_off, pol_w);
            tma_load_2d_hint(st + (DUAL ? 2 : 1) * S::A_BYTES, &tmap_x, &full_bar[s], kb * BK, m0, pol_x);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM_W, TN, 0, 0);
      const uint64_t desc_base = make_smem_desc_sw128(smem_u32(smem), 16, 1024);     // stage 0, k-step 0 of the weight tile
      int it = 0, ui = 0;
      bool dead = false;
      for (int u = unit_begin; u < total_tiles && !dead; u += unit_step) {
        if (p.grp_tiles != nullptr && __ldg(&p.grp_tiles[u % num_m].x) < 0) continue;
        const int ab = NBUF == 1 ? 0 : (ui & 1);
        const uint32_t aph = NBUF == 1 ? (ui & 1) : ((ui >> 1) & 1);
        ++ui;
        if (!mbar_wait(&tmem_empty_bar[ab], aph ^ 1, abort_flag, p.err, 400 + ab)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * ACC_COLS;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.err, 200 + s)) { dead = true; break; }
          if (it == 0) ts_mark(p, 2);
          tc_fence_after();
          const uint64_t adesc0 = smem_desc_advance(desc_base, uint32_t(s) * S::STAGE_BYTES);
          const uint64_t bdesc0 = smem_desc_advance(adesc0, (DUAL ? 2 : 1) * S::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t bdesc = smem_desc_advance(bdesc0, k * UMMA_K * 2);
            const uint64_t adesc = smem_desc_advance(adesc0, k * UMMA_K * 2);
            const uint32_t acc = (kb != kb0 || k != 0) ? 1u : 0u;
            umma_bf16_ss(d_tmem, adesc, bdesc, idesc, acc);
            if (DUAL) umma_bf16_ss(d_tmem + TN, smem_desc_advance(adesc, S::A_BYTES), bdesc, idesc, acc);
          }
          umma_commit(&empty_bar[s]);  // stage is free once these MMAs have read it
        }
        umma_commit(&tmem_full_bar[ab]);
        if (ui == 1) ts_mark(p, 3);
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..9) ------------------------------
    const int q = warp & 3;           // TMEM lane quarter this warp may read
    const int et = q * 32 + lane;     // 0..127 : output feature inside the tile == TMEM lane
    const int tid_e = threadIdx.x - 64;
    const int grp = tid_e >> 7;       // epilogue group: takes the chunks c with (c & 1) == grp
    const int tid_g = tid_e & 127;
    const int bar_id = 1 + grp;       // named barrier of the group (128 threads)
    constexpr int CH = TN >= 32 ? 32 : 16;
    constexpr int NCH = TN / CH;
    const bool vec_ok = (p.N % 8 == 0) && (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                        (p.residual == nullptr ||
                         ((p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0)));
    const bool raw_ok = vec_ok && p.residual == nullptr && p.rs_world == 0 && !p.out_f32;
    int ui = 0;
    for (int u = unit_begin; u < total_tiles; u += unit_step) {
      const TileCoord tc = tile_coord(p, u, num_m, TN);
      if (!tc.valid) continue;
      const int m0 = tc.m0, n0 = tc.no, m_end = tc.m_end;
      const int ab = NBUF == 1 ? 0 : (ui & 1);
      const uint32_t aph = NBUF == 1 ? (ui & 1) : ((ui >> 1) & 1);
      ++ui;
      mbar_wait(&tmem_full_bar[ab], aph, abort_flag, p.err, 300 + ab);
      if (ui == 1 && tid_e == 0) ts_mark(p, 4);
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + ab * ACC_COLS + (uint32_t(q * 32) << 16);
      if constexpr (SPLITK) {
        // the partial stays in TMEM until every CTA of the cluster has finished its MMAs (see below)
        (void)lane_addr;
      } else {
        const int n = n0 + et;
        float bias_v = 0.f;
        if (p.bias != nullptr && n < p.N) bias_v = __bfloat162float(p.bias[n]);
        uint8_t* staging = smem + S::TILE_BYTES + grp * (STAGING_BYTES / 2);
        if (grp >= NCH) {
          // a tile of a single chunk: this group has nothing to read and hands the buffer back at once
          tc_fence_before();
          mbar_arrive(&tmem_empty_bar[ab]);
        }
#pragma unroll 1
        for (int c = grp; c < NCH; c += 2) {
          uint32_t r[CH], r2[CH];
          if constexpr (CH == 32) {
            tmem_ld_32x32(lane_addr + c * CH, r);
            if (DUAL) tmem_ld_32x32(lane_addr + TN + c * CH, r2);
          } else {
            tmem_ld_32x16(lane_addr + c * CH, r);
            if (DUAL) tmem_ld_32x16(lane_addr + TN + c * CH, r2);
          }
          tmem_ld_wait();
          if (c + 2 >= NCH) {
            // This group's share of the accumulator is read: hand the TMEM buffer back to the MMA warp.
            tc_fence_before();
            mbar_arrive(&tmem_empty_bar[ab]);
          }
          epi_values<CH, DUAL>(r, r2, p.out_scale, bias_v, p.act);
          if (p.out_f32) {
            // fp32 rows are twice as wide: the group's 8 KB buffer holds 16 tokens at a time
            float* stf = reinterpret_cast<float*>(staging);
#pragma unroll
            for (int hh = 0; hh < CH / 16; ++hh) {
#pragma unroll
              for (int j = 0; j < 16; ++j) stf[j * BM_W + et] = __uint_as_float(r[hh * 16 + j]);
              asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
              for (int idx = tid_g; idx < 16 * 16; idx += 128) {
                const int tok = idx >> 4, c8 = idx & 15;
                const float4 lo = *reinterpret_cast<const float4*>(stf + tok * BM_W + c8 * 8);
                const float4 hi = *reinterpret_cast<const float4*>(stf + tok * BM_W + c8 * 8 + 4);
                float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                emit8(p, m0 + c * CH + hh * 16 + tok, m_end, n0 + c8 * 8, v, vec_ok);
              }
              asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
            }
          } else {
            __nv_bfloat16* stb = reinterpret_cast<__nv_bfloat16*>(staging);
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              stb[j * BM_W + et] = __float2bfloat16(__uint_as_float(r[j]));
            }
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
            for (int idx = tid_g; idx < CH * 16; idx += 128) {
              const int tok = idx >> 4, c8 = idx & 15;
              const uint4 raw = *reinterpret_cast<const uint4*>(stb + tok * BM_W + c8 * 8);
              if (raw_ok) {
                // nothing to add and a local bf16 destination: the staged 16 bytes are the output bytes
                const int m = m0 + c * CH + tok, nn = n0 + c8 * 8;
                if (m < m_end && nn < p.N) *reinterpret_cast<uint4*>(p.out + (long long)m * p.ldo + nn) = raw;
                continue;
              }
              const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
              float v[8];
#pragma unroll
              for (int e = 0; e < 4; ++e) { v[2 * e] = bf16_lo(w[e]); v[2 * e + 1] = bf16_hi(w[e]); }
              emit8(p, m0 + c * CH + tok, m_end, n0 + c8 * 8, v, vec_ok);
            }
            // the group's buffer is read: the next chunk may overwrite it
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
          }
        }
      }
    }
    if (tid_e == 0) ts_mark(p, 5);
    if (!SPLITK && p.rs_world > 0) {
      // Publish: the epilogue warps meet, then one thread arrives for the CTA (the last CTA of the launch tells the peers).
      asm volatile("bar.sync 3, 256;" ::: "memory");
      if (tid_e == 0) publish_to_peers(p.rs_local_count, p.rs_total, p.rs_peer_flag, p.rs_world);
    }
  }

  if constexpr (SPLITK) {
    // Every CTA's MMAs are complete (its epilogue warps have seen tmem_full), so the operand stages of all CTAs may be
    // overwritten by the partial-tile slots.
    tc_fence_before();
    cluster_sync_all();
    if (threadIdx.x == 64) ts_mark(p, 8);
    const bool sk_valid = tile_begin + (int)blockIdx.y < total_tiles;
    if (warp >= 2 && sk_valid) {
      tc_fence_after();
      constexpr int CHS = TN >= 32 ? 32 : 16;
      const int q = warp & 3;
      splitk_scatter<TN, CHS, DUAL>(p, smem_u32(smem), tmem_base + (uint32_t(q * 32) << 16), q * 32 + lane, crank, 1u, 0u,
                                    (int(threadIdx.x) - 64) >> 7);
    }
    if (threadIdx.x == 64) ts_mark(p, 9);
    tc_fence_before();
    cluster_sync_all();                       // all slots are written (release / acquire at cluster scope)
    if (threadIdx.x == 64) ts_mark(p, 10);
    if (warp >= 2 && sk_valid) {
      const int u = tile_begin + blockIdx.y;
      const int m0 = (u % num_m) * TN, n0 = (u / num_m) * BM_W;
      const int tid_e = threadIdx.x - 64;
      const int per = (TN + p.splits - 1) / p.splits;
      const int r0 = min(TN, crank * per), r1 = min(TN, r0 + per);
      const bool vec_ok = (p.N % 8 == 0) && (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                          (p.residual == nullptr ||
                           ((p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0)));
      splitk_finish<DUAL>(p, smem, TN, r0, r1, tid_e, m0, n0, vec_ok);
      if (p.rs_world > 0) {
        asm volatile("bar.sync 3, 256;" ::: "memory");
        if (tid_e == 0) publish_to_peers(p.rs_local_count, p.rs_total, p.rs_peer_flag, p.rs_world);
      }
    }
    if (threadIdx.x == 64) ts_mark(p, 6);
    cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait gave up: let bulk copies that are still in flight land before the CTA's smem is reused.
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0) ts_mark(p, 7);
}

// ----------------------------------------------------------------------------
// 2-CTA variant (tcgen05 cta_group::2).  A thread-block cluster of two CTAs on neighbouring SMs computes one tile of
// 256 weight rows x TN tokens: every CTA stages its own 128 weight rows and HALF of the token tile, the leader CTA
// issues MMAs that read both shared memories, and every CTA ends up with its 128 rows of the result in its own
// TMEM.  Per MMA a CTA therefore moves 2/3 of the bytes of the 1-CTA kernel from L2 into shared memory, which is
// what bounds large-token-count tiles.  Barrier protocol:
//   full[s]  (leader's)  : both producers' TMA loads complete_tx on it (cta_group::2 loads, barrier address mapped
//                          to CTA 0); the leader's producer arrives with the byte count of both CTAs
//   empty[s] (each CTA's): the leader's tcgen05.commit arrives on its own and on the peer's barrier
//   tmem_full (each CTA's): same, by commit;  tmem_empty (leader's): 256 arrivals, the peer's come over DSMEM
// No load is multicast.  Plain, bias / residual / activation epilogues, the gated (dual) form and the F1 / F3
// collective hooks are supported; split-K and the grouped mode stay on the 1-CTA kernel.
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void tmem_alloc_cg2(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_cg2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_cg2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// TMA tile load whose completion bytes go to a barrier that may live in the peer CTA (cluster address).
__device__ __forceinline__ void tma_load_2d_cg2(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y,
                                                uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, "
      "{%3, %4}], [%2], %5;" ::"r"(smem_u32(smem_dst)),
      "l"(m), "r"(bar_cluster_addr), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_ss_cg2(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at a cluster shared address once all MMAs issued so far by this thread are complete.
__device__ __forceinline__ void umma_commit_cg2(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// Work of one CTA pair, segment by segment.  Tile mode: whole tiles u, u + step, ... with the K range [kb0, kb1) fixed.
// Stream-K mode (nkb > 0): the pairs form teams of num_m (one member per token tile); a team takes the units
// [pos, pos_end) of the linear (row of weight tiles, k-block) space, cut at row boundaries, and its members walk them in
// lockstep, each on its own token tile -- so a weight k-block is still pulled by num_m pairs at the same time and
// comes from HBM once (with one range per pair the pairs of a weight row drift apart in K and every one of them
// streams the weights from HBM again: 1020 x 4096 x 14336 took 102 us instead of 91).
struct PairWalk {
  int u, kb0, kb1;
  int step, end;
  int pos, pos_end, nkb;
  int row, mul, add;      // stream-K: unit row = pos / nkb is a row of weight tiles; this pair's tile in it is row * mul + add
  __device__ __forceinline__ bool valid() const { return nkb > 0 ? pos < pos_end : u < end; }
  __device__ __forceinline__ void seg() {
    row = pos / nkb;
    u = row * mul + add;
    kb0 = pos - row * nkb;
    kb1 = min(nkb, kb0 + (pos_end - pos));
  }
  __device__ __forceinline__ void next() {
    if (nkb > 0) {
      pos += kb1 - kb0;
      if (pos < pos_end) seg();
    } else {
      u += step;
    }
  }
};
constexpr int SK_SLOT_FLOATS = 256 * BM_W;          // workspace slot of one CTA: a 128 x 256 fp32 accumulator

template <int TN, int STAGES, bool DUAL, bool SPLITK = false>
struct Gemm2Smem {
  static constexpr int A_BYTES = BM_W * BK * 2;            // this CTA's 128 weight rows: 16 KB
  static constexpr int B_BYTES = (TN / 2) * BK * 2;        // this CTA's half of the token tile
  static constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * A_BYTES + B_BYTES;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  // split-K parks the fp32 partial tile [TN][128] on top of the (then idle) pipeline stages
  static constexpr int PARTIAL_BYTES = (DUAL ? 2 : 1) * (TN + 8) * BM_W * 4;   // splits x ceil(TN / splits) rows, splits <= 8
  static_assert(!SPLITK || PARTIAL_BYTES <= TILE_BYTES, "partial tile does not fit in the stage memory");
  static constexpr int DATA_BYTES = TILE_BYTES + STAGING_BYTES;
  static constexpr int TOTAL = DATA_BYTES + 1024 + 256;
  static_assert(TOTAL <= 227 * 1024, "shared memory budget exceeded");
};

template <int TN, int STAGES, bool DUAL, bool SPLITK>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tn_2cta_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                    const GemmParams p) {
  using S = Gemm2Smem<TN, STAGES, DUAL, SPLITK>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::DATA_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;   // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Cluster = one CTA pair, or (split-K) `splits` pairs that share a tile and each reduce 1/splits of K.
  const uint32_t crank = cluster_ctarank();
  const uint32_t rank = crank & 1u;               // rank inside the pair; 0 = leader (issues the MMAs)
  const uint32_t pidx = crank >> 1;               // pair index == K slice in split-K mode
  const uint32_t lead = crank & ~1u;              // cluster rank of this pair's leader; the peer is lead + 1
  const bool leader = rank == 0;
  const int num_m = (p.M + TN - 1) / TN;
  const int num_n = (p.N + 2 * BM_W - 1) / (2 * BM_W);
  // [tile_begin, tile_end) is this launch's share of the pair tiles (two-phase schedule, see plan_gemm)
  const int tile_begin = p.tile_begin;
  const int total_tiles = p.tile_end > 0 ? p.tile_end : num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t ACC_COLS = (DUAL ? 2 : 1) * TN;
  constexpr int NBUF = (SPLITK || 2 * ACC_COLS > 512) ? 1 : 2;
  constexpr uint32_t NEED_COLS = NBUF * ACC_COLS;
  constexpr uint32_t TMEM_COLS = NEED_COLS < 32 ? 32 : NEED_COLS;
  static_assert(TMEM_COLS <= 512, "TMEM budget exceeded");
  int unit_begin, unit_step, kb0 = 0, kb1 = num_kb;
  if (SPLITK) {
    unit_begin = tile_begin + blockIdx.y;         // grid = (2 * splits, tiles): one tile per cluster
    unit_step = 1 << 30;
    const int per = (num_kb + p.splits - 1) / p.splits;
    kb0 = int(pidx) * per;
    kb1 = min(num_kb, kb0 + per);
  } else {
    unit_begin = tile_begin + (blockIdx.x >> 1);
    unit_step = gridDim.x >> 1;
  }
  PairWalk walk0;
  walk0.u = unit_begin; walk0.kb0 = kb0; walk0.kb1 = kb1;
  walk0.step = unit_step; walk0.end = total_tiles;
  walk0.pos = 0; walk0.pos_end = 0; walk0.nkb = 0;
  walk0.row = 0; walk0.mul = 0; walk0.add = 0;
  const int sk_pair = blockIdx.x >> 1;
  const int sk_teams = int(gridDim.x >> 1) / num_m, sk_team = sk_pair / num_m;
  const long long sk_total = (long long)num_n * num_kb;
  if (!SPLITK && p.sk_on) {
    walk0.nkb = num_kb;
    walk0.mul = num_m;
    walk0.add = sk_pair - sk_team * num_m;
    if (sk_team < sk_teams) {                     // pairs beyond the last whole team have no work
      walk0.pos = int(sk_total * sk_team / sk_teams);
      walk0.pos_end = int(sk_total * (sk_team + 1) / sk_teams);
    }
    if (walk0.pos < walk0.pos_end) walk0.seg();
  }

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 2 * EPI_THREADS);       // epilogue threads of both CTAs (only the leader's copy is used)
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc_cg2(tmem_slot, TMEM_COLS);
    tmem_relinquish_cg2();
  }
  tc_fence_before();
  cluster_sync_all();                              // barriers of both CTAs are initialised before anyone uses them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch (see gemm_tn_kernel): TMEM and barriers are set up, nothing global has been touched.
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      uint32_t ag_ready = 0;
      int it = 0;
      bool dead = false;
      for (PairWalk wk = walk0; wk.valid() && !dead; wk.next()) {
        const int u = wk.u, kb0 = wk.kb0, kb1 = wk.kb1;
        const int m0 = (u % num_m) * TN + int(rank) * (TN / 2);          // this CTA's half of the token tile
        const int n0 = (u / num_m) * (2 * BM_W) + int(rank) * BM_W;      // this CTA's weight rows
        if (p.ag_world > 0) {
          const uint32_t want = p.ag_signals_per_use;
          const int r_lo = m0 / p.ag_rows_per_rank;
          int r_hi = (min(m0 + TN / 2, p.M) - 1) / p.ag_rows_per_rank;
          if (r_hi >= p.ag_world) r_hi = p.ag_world - 1;
          const uint64_t t0 = wait_ticks();
          bool waited = false;
          for (int r = r_lo; r <= r_hi; ++r) {
            if (ag_ready >> r & 1u) continue;
            uint32_t spin = 0;
            while (int32_t(ld_acquire_sys_u32(p.ag_flags + r) - want) < 0) {
              if ((++spin & 31u) == 0 && wait_expired(t0, p.err)) {
                *abort_flag = 1;
                set_err(p.err, ERR_FLAG_TIMEOUT, r);
                break;
              }
            }
            ag_ready |= 1u << r;
            waited = true;
          }
          if (waited) asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.err, 600 + s)) { dead = true; break; }
          uint8_t* st = smem + s * S::STAGE_BYTES;
          if (leader) mbar_arrive_expect_tx(&full_bar[s], 2 * S::STAGE_BYTES);   // bytes of both CTAs
          const uint32_t fb = mapa_u32(smem_u32(&full_bar[s]), lead);           // the leader's barrier
          tma_load_2d_cg2(st, &tmap_w, fb, kb * BK, n0, pol_w);
          if (DUAL) tma_load_2d_cg2(st + S::A_BYTES, &tmap_w, fb, kb * BK, n0 + p.up_row_off, pol_w);
          tma_load_2d_cg2(st + (DUAL ? 2 : 1) * S::A_BYTES, &tmap_x, fb, kb * BK, m0, pol_x);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM_W, TN, 0, 0);
      const uint64_t desc_base = make_smem_desc_sw128(smem_u32(smem), 16, 1024);     // stage 0, k-step 0 of the weight tile
      int it = 0, ui = 0;
      bool dead = false;
      for (PairWalk wk = walk0; wk.valid() && !dead; wk.next()) {
        const int kb0 = wk.kb0, kb1 = wk.kb1;
        const int ab = NBUF == 1 ? 0 : (ui & 1);
        const uint32_t aph = NBUF == 1 ? (ui & 1) : ((ui >> 1) & 1);
        ++ui;
        if (!mbar_wait(&tmem_empty_bar[ab], aph ^ 1, abort_flag, p.err, 610 + ab)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * ACC_COLS;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.err, 620 + s)) { dead = true; break; }
          tc_fence_after();
          const uint64_t adesc0 = smem_desc_advance(desc_base, uint32_t(s) * S::STAGE_BYTES);
          const uint64_t bdesc0 = smem_desc_advance(adesc0, (DUAL ? 2 : 1) * S::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t bdesc = smem_desc_advance(bdesc0, k * UMMA_K * 2);
            const uint64_t adesc = smem_desc_advance(adesc0, k * UMMA_K * 2);
            const uint32_t acc = (kb != kb0 || k != 0) ? 1u : 0u;
            umma_bf16_ss_cg2(d_tmem, adesc, bdesc, idesc, acc);
            if (DUAL) umma_bf16_ss_cg2(d_tmem + TN, smem_desc_advance(adesc, S::A_BYTES), bdesc, idesc, acc);
          }
          // the stage is free in BOTH CTAs once these MMAs have read it
          const uint32_t eb = smem_u32(&empty_bar[s]);
          umma_commit_cg2(mapa_u32(eb, lead));
          umma_commit_cg2(mapa_u32(eb, lead + 1));
        }
        const uint32_t tf = smem_u32(&tmem_full_bar[ab]);
        umma_commit_cg2(mapa_u32(tf, lead));
        umma_commit_cg2(mapa_u32(tf, lead + 1));
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..9, both CTAs) ------------------------------
    const int q = warp & 3;
    const int et = q * 32 + lane;
    const int tid_e = threadIdx.x - 64;
    const int grp = tid_e >> 7;       // epilogue group: takes the chunks c with (c & 1) == grp
    const int tid_g = tid_e & 127;
    const int bar_id = 1 + grp;
    constexpr int CH = 32;
    constexpr int NCH = TN / CH;      // TN >= 64 here: both groups always have chunks
    const bool vec_ok = (p.N % 8 == 0) && (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                        (p.residual == nullptr ||
                         ((p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0)));
    const bool raw_ok = vec_ok && p.residual == nullptr && p.rs_world == 0 && !p.out_f32;
    int ui = 0;
    for (PairWalk wk = walk0; wk.valid(); wk.next()) {
      const int u = wk.u;
      const int m0 = (u % num_m) * TN;                                   // all TN tokens: the accumulator is 128 x TN
      const int n0 = (u / num_m) * (2 * BM_W) + int(rank) * BM_W;
      const int ab = NBUF == 1 ? 0 : (ui & 1);
      const uint32_t aph = NBUF == 1 ? (ui & 1) : ((ui >> 1) & 1);
      ++ui;
      // Stream-K (plain GEMMs): a segment that does not cover the whole K range of its tile.  The pair that holds the
      // head of the tile (kb0 == 0) owns it; every other segment parks its fp32 partial in this CTA's workspace slot
      // and raises its flag.  A team works through its range front to back, so the partials of a tile's later K ranges
      // (the first segments of the following teams) are written long before the owner reaches its last segment: the
      // owner checks the flags and requests the first chunk of partials while its own MMAs are still running.
      int sk_contrib = 0;
      bool sk_part = false;
      float pre[CH];
      auto sk_slot = [&](int i) {
        return p.sk_ws + (size_t)((sk_pair + i * num_m) * 2 + int(rank)) * SK_SLOT_FLOATS + et;
      };
      auto sk_prefetch = [&](int c) {
        const float* src = sk_slot(1) + c * CH * BM_W;
#pragma unroll
        for (int j = 0; j < CH; ++j) pre[j] = __ldcg(src + j * BM_W);
      };
      if constexpr (!SPLITK && !DUAL) {
        if (wk.nkb > 0 && !(wk.kb0 == 0 && wk.kb1 == wk.nkb)) {
          sk_part = wk.kb0 > 0;
          if (!sk_part) {
            // owner: the same members of the following teams whose ranges start inside this row hold the rest of its K range
            const long long row_end_pos = (long long)(wk.row + 1) * wk.nkb;
            while (sk_team + 1 + sk_contrib < sk_teams &&
                   sk_total * (sk_team + 1 + sk_contrib) / sk_teams < row_end_pos)
              ++sk_contrib;
            if (tid_e == 0) {
              const uint64_t t0 = wait_ticks();
              for (int i = 1; i <= sk_contrib; ++i) {
                const uint32_t* f = p.sk_flags + (sk_pair + i * num_m) * 2 + int(rank);
                uint32_t spin = 0, v = 0;
                while (true) {
                  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                  if (v != 0) break;
                  if ((++spin & 31u) == 0 && (*abort_flag || wait_expired(t0, p.err))) {
                    *abort_flag = 1;
                    set_err(p.err, ERR_FLAG_TIMEOUT, 640);
                    break;
                  }
                }
              }
            }
            asm volatile("bar.sync 3, 256;" ::: "memory");
            if (sk_contrib > 0) sk_prefetch(grp);
          }
        }
      }
      mbar_wait(&tmem_full_bar[ab], aph, abort_flag, p.err, 630 + ab);
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + ab * ACC_COLS + (uint32_t(q * 32) << 16);
      if constexpr (SPLITK) {
        // the partial stays in TMEM until every CTA of the cluster has finished its MMAs (see below)
        (void)lane_addr;
        continue;
      }
      if (sk_part) {
        float* dst = p.sk_ws + (size_t)(sk_pair * 2 + int(rank)) * SK_SLOT_FLOATS + et;
#pragma unroll 1
        for (int c = grp; c < NCH; c += 2) {
          uint32_t r[CH];
          tmem_ld_32x32(lane_addr + c * CH, r);
          tmem_ld_wait();
          if (c + 2 >= NCH) {
            tc_fence_before();
            mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty_bar[ab]), lead));
          }
#pragma unroll
          for (int j = 0; j < CH; ++j) dst[(c * CH + j) * BM_W] = __uint_as_float(r[j]);
        }
        __threadfence();
        asm volatile("bar.sync 3, 256;" ::: "memory");
        if (tid_e == 0)
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.sk_flags + sk_pair * 2 + int(rank)), "r"(1u) : "memory");
        continue;
      }
      const int n = n0 + et;
      float bias_v = 0.f;
      if (p.bias != nullptr && n < p.N) bias_v = __bfloat162float(p.bias[n]);
      uint8_t* staging = smem + S::TILE_BYTES + grp * (STAGING_BYTES / 2);
#pragma unroll 1
      for (int c = grp; c < NCH; c += 2) {
        uint32_t r[CH], r2[CH];
        tmem_ld_32x32(lane_addr + c * CH, r);
        if (DUAL) tmem_ld_32x32(lane_addr + TN + c * CH, r2);
        tmem_ld_wait();
        if (c + 2 >= NCH) {
          tc_fence_before();
          mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty_bar[ab]), lead));   // hand the buffer back to the leader's MMA thread
        }
        if (sk_contrib > 0) {
#pragma unroll
          for (int j = 0; j < CH; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + pre[j]);
          for (int i = 2; i <= sk_contrib; ++i) {
            const float* src = sk_slot(i) + c * CH * BM_W;
#pragma unroll
            for (int j = 0; j < CH; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldcg(src + j * BM_W));
          }
          if (c + 2 < NCH) sk_prefetch(c + 2);       // in flight while this chunk is converted, staged and stored
        }
        epi_values<CH, DUAL>(r, r2, p.out_scale, bias_v, p.act);
        if (p.out_f32) {
          float* stf = reinterpret_cast<float*>(staging);
#pragma unroll
          for (int hh = 0; hh < CH / 16; ++hh) {
#pragma unroll
            for (int j = 0; j < 16; ++j) stf[j * BM_W + et] = __uint_as_float(r[hh * 16 + j]);
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
            for (int idx = tid_g; idx < 16 * 16; idx += 128) {
              const int tok = idx >> 4, c8 = idx & 15;
              const float4 lo = *reinterpret_cast<const float4*>(stf + tok * BM_W + c8 * 8);
              const float4 hi = *reinterpret_cast<const float4*>(stf + tok * BM_W + c8 * 8 + 4);
              float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
              emit8(p, m0 + c * CH + hh * 16 + tok, p.M, n0 + c8 * 8, v, vec_ok);
            }
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
          }
        } else {
          __nv_bfloat16* stb = reinterpret_cast<__nv_bfloat16*>(staging);
#pragma unroll
          for (int j = 0; j < CH; ++j) {
            stb[j * BM_W + et] = __float2bfloat16(__uint_as_float(r[j]));
          }
          asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
          for (int idx = tid_g; idx < CH * 16; idx += 128) {
            const int tok = idx >> 4, c8 = idx & 15;
            const uint4 raw = *reinterpret_cast<const uint4*>(stb + tok * BM_W + c8 * 8);
            if (raw_ok) {
              // nothing to add and a local bf16 destination: the staged 16 bytes are the output bytes
              const int m = m0 + c * CH + tok, nn = n0 + c8 * 8;
              if (m < p.M && nn < p.N) *reinterpret_cast<uint4*>(p.out + (long long)m * p.ldo + nn) = raw;
              continue;
            }
            const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
            float v[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) { v[2 * e] = bf16_lo(w[e]); v[2 * e + 1] = bf16_hi(w[e]); }
            emit8(p, m0 + c * CH + tok, p.M, n0 + c8 * 8, v, vec_ok);
          }
          asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
        }
      }
      if (sk_contrib > 0) {
        // every thread has read the partials: lower the flags for the next launch that uses this workspace
        asm volatile("bar.sync 3, 256;" ::: "memory");
        if (tid_e == 0)
          for (int i = 1; i <= sk_contrib; ++i)
            asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p.sk_flags + (sk_pair + i * num_m) * 2 + int(rank)), "r"(0u) : "memory");
      }
    }
    if (!SPLITK && p.rs_world > 0) {
      asm volatile("bar.sync 3, 256;" ::: "memory");
      if (tid_e == 0) publish_to_peers(p.rs_local_count, p.rs_total, p.rs_peer_flag, p.rs_world);
    }
  }

  if constexpr (SPLITK) {
    // Every pair's MMAs are complete, so the operand stages of all CTAs may be overwritten by the partial-tile slots.
    // Pair d of the cluster finishes the token rows [d * per, (d + 1) * per); inside a pair each CTA owns its own 128
    // features, so partial rows travel between the CTAs of equal rank in their pair.
    tc_fence_before();
    cluster_sync_all();
    const bool sk_valid = tile_begin + (int)blockIdx.y < total_tiles;
    if (warp >= 2 && sk_valid) {
      tc_fence_after();
      const int q = warp & 3;
      splitk_scatter<TN, 32, DUAL>(p, smem_u32(smem), tmem_base + (uint32_t(q * 32) << 16), q * 32 + lane, int(pidx), 2u,
                                   uint32_t(rank), (int(threadIdx.x) - 64) >> 7);
    }
    tc_fence_before();
    cluster_sync_all();                       // all slots are written (release / acquire at cluster scope)
    if (warp >= 2 && sk_valid) {
      const int u = tile_begin + blockIdx.y;
      const int m0 = (u % num_m) * TN;
      const int n0 = (u / num_m) * (2 * BM_W) + int(rank) * BM_W;
      const int tid_e = threadIdx.x - 64;
      const int per = (TN + p.splits - 1) / p.splits;
      const int r0 = min(TN, int(pidx) * per), r1 = min(TN, r0 + per);
      const bool vec_ok = (p.N % 8 == 0) && (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                          (p.residual == nullptr ||
                           ((p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0)));
      splitk_finish<DUAL>(p, smem, TN, r0, r1, tid_e, m0, n0, vec_ok);
      if (p.rs_world > 0) {
        asm volatile("bar.sync 3, 256;" ::: "memory");
        if (tid_e == 0) publish_to_peers(p.rs_local_count, p.rs_total, p.rs_peer_flag, p.rs_world);
      }
    }
  }

  tc_fence_before();
  cluster_sync_all();       // nobody leaves while the peer may still touch its barriers, shared memory or TMEM
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_cg2(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------
// Host side
// ----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 tensor map, rows x cols (cols contiguous), box = box_rows x box_cols, 128-byte swizzle.
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld_elems,
                      int box_rows, int box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld_elems * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  static int promo = -1;
  if (promo < 0) {
    const char* e = getenv("UB_TMAP_L2_PROMOTION");   // 0 none, 1 64B, 2 128B, 3 256B (default)
    promo = e ? atoi(e) : 3;
    if (promo < 0 || promo > 3) promo = 3;
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, (CUtensorMapL2promotion)promo,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
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

struct GemmPlan {
  int tn, splits, ctas, tiles;
  int tail_tiles, tail_splits;
  int pair;
  int tail_units;     // pair plans of a gated GEMM: 1-CTA tiles (128 tokens) that cover the tail's pair tiles
  int sk;             // pair plans: stream-K schedule (one contiguous range of (tile, k-block) units per pair)
};

// ---- stream-K workspace: per device, a few lanes (one per stream that launches GEMMs), each with one fp32 slot and one
// flag per CTA.  Allocated once, outside stream capture; a lane is bound to the first stream that asks for it.
constexpr int SK_PAIRS_MAX = 80;
constexpr int SK_LANES = 4;
constexpr size_t SK_LANE_FLOATS = (size_t)SK_PAIRS_MAX * 2 * SK_SLOT_FLOATS;
constexpr int SK_LANE_FLAGS = 256;
struct SkDevice {
  float* ws = nullptr;
  uint32_t* flags = nullptr;
  cudaStream_t owner[SK_LANES] = {};
  int used = 0;
  bool failed = false;
};
static SkDevice g_sk[UB_MAX_DEVICES];
static std::mutex g_sk_mu;
static thread_local bool tl_no_sk = false;     // plan_gemm: leave the stream-K schedule out (no workspace for this stream)

static bool sk_workspace(cudaStream_t st, float** ws, uint32_t** flags) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= UB_MAX_DEVICES) return false;
  std::lock_guard<std::mutex> lock(g_sk_mu);
  SkDevice& d = g_sk[dev];
  if (d.failed) return false;
  if (d.ws == nullptr) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
      (void)cudaGetLastError();
      return false;                             // no allocation while a capture is open; the caller plans without it
    }
    float* w = nullptr;
    uint32_t* f = nullptr;
    if (cudaMalloc(&w, SK_LANES * SK_LANE_FLOATS * sizeof(float)) != cudaSuccess ||
        cudaMalloc(&f, SK_LANES * SK_LANE_FLAGS * sizeof(uint32_t)) != cudaSuccess ||
        cudaMemset(f, 0, SK_LANES * SK_LANE_FLAGS * sizeof(uint32_t)) != cudaSuccess) {
      (void)cudaGetLastError();
      if (w != nullptr) cudaFree(w);
      d.failed = true;
      return false;
    }
    d.ws = w;
    d.flags = f;
  }
  int lane = -1;
  for (int i = 0; i < d.used; ++i)
    if (d.owner[i] == st) lane = i;
  if (lane < 0) {
    if (d.used >= SK_LANES) return false;
    lane = d.used++;
    d.owner[lane] = st;
  }
  *ws = d.ws + (size_t)lane * SK_LANE_FLOATS;
  *flags = d.flags + lane * SK_LANE_FLAGS;
  return true;
}

// How many thread-block clusters of `csize` CTAs (one CTA per SM, ~200 KB of shared memory each) the device can run at
// the same time.  A cluster lives inside one GPC, so this is less than SMs / csize: split-K launches that ask for
// more clusters than this run in two waves and take twice as long.
static int max_active_clusters(int csize) {
  static int cache[UB_MAX_DEVICES][9] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (csize < 2) return num_sms();
  if (csize > 8) csize = 8;
  if (dev < UB_MAX_DEVICES && cache[dev][csize] > 0) return cache[dev][csize];
  auto kern = gemm_tn_kernel<128, 6, false, true>;
  using S = GemmSmem<128, 6, false, true>;
  int n = 0;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL) == cudaSuccess) {
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.gridDim = dim3(csize, 4096, 1);          // far more clusters than fit: the answer must not be capped by the grid
    cfg.dynamicSmemBytes = S::TOTAL;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) n = 0;
  }
  (void)cudaGetLastError();
  if (n <= 0) n = (num_sms() / csize) * 7 / 8;      // the query failed: assume some GPCs do not divide evenly
  if (dev < UB_MAX_DEVICES) cache[dev][csize] = n;
  return n;
}

static GemmPlan plan_gemm(const UbGemmArgs* a) {
  GemmPlan pl;
  const bool dual = a->dual != 0;
  int tn = a->tile_tokens;
  if (tn <= 0) {
    tn = 16;
    // gated GEMMs keep two 128-column accumulators double-buffered; the single-buffered 2 x 256 variant
    // measured slower at every size
    while (tn < a->M && tn < (dual ? 128 : 256)) tn <<= 1;
  }
  const bool grouped = a->grp_tiles != nullptr;
  if (a->tile_tokens <= 0 && !grouped && !dual) {
    // Short K (per-rank o / down projections under tensor parallelism): the main loop is a few microseconds and what
    // the launch pays for is the exposed epilogue of its single tile per CTA (0.8 us per 32 token columns).  Narrower
    // token tiles give more CTAs with shorter epilogues as long as everything still fits in one wave.
    const int nn = (a->N + BM_W - 1) / BM_W, kb = (a->K + BK - 1) / BK, sm = num_sms();
    auto tiles_of = [&](int t) { return ((a->M + t - 1) / t) * nn; };
    while (kb <= 32 && tn > 64 && tiles_of(tn) * 2 <= sm && tiles_of(tn / 2) <= sm) tn >>= 1;
  }
  pl.tn = tn;
  const int num_m = grouped ? a->grp_max_tiles : (a->M + tn - 1) / tn, num_n = (a->N + BM_W - 1) / BM_W;
  pl.tiles = num_m * num_n;
  const int num_kb = (a->K + BK - 1) / BK;
  const int sms = num_sms();
  int splits = grouped ? 1 : a->splits;
  if (splits <= 0) {
    splits = 1;
    if (pl.tiles * 2 <= sms && num_kb >= 8) {
      splits = sms / pl.tiles;
      if (splits > 8) splits = 8;
      if (splits > num_kb / 4) splits = num_kb / 4;
      if (splits < 1) splits = 1;
    }
  }
  if (splits > 8) splits = 8;
  if (splits > num_kb) splits = num_kb;
  while (splits & (splits - 1)) splits &= splits - 1;  // cluster sizes 1, 2, 4, 8
  while (splits > 1 && (splits - 1) * ((num_kb + splits - 1) / splits) >= num_kb) --splits;  // no empty split
  // an automatic split must fit in one wave of clusters
  if (a->splits <= 0 && !grouped)
    while (splits > 1 && pl.tiles > max_active_clusters(splits)) splits >>= 1;
  if (dual && tn == 256 && splits > 1) {
    // the parked fp32 partials of a 2 x 256-token tile do not fit in shared memory
    UbGemmArgs b = *a;
    b.tile_tokens = 128;
    return plan_gemm(&b);
  }
  pl.splits = splits;
  pl.tail_tiles = 0;
  pl.tail_splits = 1;
  pl.tail_units = 0;
  pl.sk = 0;
  // Two-phase schedule: when the last round of a persistent launch would keep fewer than half of the SMs busy, those
  // tiles run as a second launch with K split over clusters, so the tail costs 1/splits of a tile time.
  if (splits == 1 && !grouped && a->tail_split != 1 && pl.tiles > sms && num_kb >= 16) {
    const int r = pl.tiles % sms;
    if (r > 0 && r * 2 <= sms && !(dual && tn == 256)) {
      int ts = sms / r;
      if (ts > 8) ts = 8;
      while (ts & (ts - 1)) ts &= ts - 1;
      while (ts > 1 && (ts - 1) * ((num_kb + ts - 1) / ts) >= num_kb) ts >>= 1;   // no empty K slice
      if (ts >= 2) { pl.tail_tiles = r; pl.tail_splits = ts; }
    }
  }
  const int main_tiles = pl.tiles - pl.tail_tiles;
  pl.ctas = splits > 1 ? splits * pl.tiles : (main_tiles < sms ? main_tiles : sms) + pl.tail_tiles * pl.tail_splits;
  // 2-CTA tiles (256 weight rows per CTA pair): for token counts that fill a wide tile and enough tiles to keep the
  // SM pairs busy.  cta_pair: 0 auto, 1 never, 2 always (when the shape allows).
  pl.pair = 0;
  static int env_pair = -1;
  if (env_pair < 0) {
    const char* e = getenv("UB_GEMM_2CTA");
    env_pair = e ? atoi(e) : 0;          // same meaning as cta_pair; the argument wins when it is not 0
  }
  const int want = a->cta_pair != 0 ? a->cta_pair : env_pair;
  if (want != 1 && !grouped && a->splits <= 1 && a->M >= 64 && a->N >= 2 * BM_W) {
    int tn2 = a->tile_tokens > 0 ? a->tile_tokens : 256;
    if (tn2 < 64) tn2 = 64;
    if (tn2 > 256) tn2 = 256;
    while (tn2 > 64 && tn2 / 2 >= a->M) tn2 >>= 1;
    const int tiles2 = ((a->M + tn2 - 1) / tn2) * ((a->N + 2 * BM_W - 1) / (2 * BM_W));
    const bool enough = tiles2 * 4 >= (sms / 2) * 3;       // at least 3/4 of the SM pairs get a tile
    // What bounds these kernels at a few hundred tokens is the rate at which one SM can fill its shared memory
    // (measured: about 40 B/clk per SM, TMA without multicast).  Per k-block a 128 x 256 tile pulls 48 KB into one SM,
    // a CTA pair 32 KB into each of two SMs for twice the math, so pairs win as soon as the tokens fill a 256-wide
    // tile; gated GEMMs (two weight tiles per token tile) gain from 256 tokens up, plain ones from 384.
    const bool gains = dual ? a->M >= 256 : a->M >= 384;
    // pair tiles that cover at most half of the SM pairs: split K over 2 or 4 pairs per tile (clusters of 4 / 8 CTAs)
    int s2 = 1;
    if (!dual && tn2 >= 128 && a->M >= 384) {
      s2 = (sms / 2) / tiles2;
      if (s2 > 4) s2 = 4;
      if (s2 < 1) s2 = 1;
      while (s2 & (s2 - 1)) s2 &= s2 - 1;
      while (s2 > 1 && (num_kb < 16 * s2 || (s2 - 1) * ((num_kb + s2 - 1) / s2) >= num_kb)) s2 >>= 1;
      while (s2 > 1 && tiles2 > max_active_clusters(2 * s2)) s2 >>= 1;      // one wave of clusters of 2 * s2 CTAs
    }
    // tiles beyond one round of the SM pairs: the 1-CTA schedule splits its thin last round over K, pairs cannot
    const int pairs_now = max_active_clusters(2);
    // ... but a pair tile moves a third less data into shared memory per FLOP, so the pairs still win unless the last
    // round wastes more than 0.4 of the launch (1020 x 6144 x 4096: 96 pair tiles in two rounds, 56.7 us against 63.6 us)
    const int rounds2 = (tiles2 + pairs_now - 1) / pairs_now;
    const bool ragged = tiles2 > pairs_now && (tiles2 % pairs_now) != 0 &&
                        (rounds2 * pairs_now - tiles2) * 10 > rounds2 * pairs_now * 4;
    const int want_s = a->pair_splits > 0 ? a->pair_splits : s2;
    // short K in a single wave: the narrow 1-CTA tiles chosen above (more CTAs, shorter exposed epilogues) win
    const bool short_single = !dual && num_kb <= 32 && tiles2 <= pairs_now;
    // Stream-K: teams of pairs take equal shares of the (weight row, k-block) units instead of whole tiles, so a thin
    // last round or a round that leaves pairs idle costs nothing; the price is one fp32 partial per pair through L2.
    // Plain GEMMs only (a gated pair tile fills TMEM with its two accumulators, so the partial's read-out would stall
    // the MMAs; its thin last round goes to the two-phase schedule below), and only where it removes a round: parking
    // and re-reading a partial costs every pair about as much as 20 k-blocks, so single-round launches with idle
    // pairs gain nothing (1020 x 4096 x 14336: 90.8 -> 90.3 us, 640 x 4096 x 4096: 32.5 -> 33.1 us), while
    // 1020 x 6144 x 4096 (96 tiles = 74 + 22) goes from 57.1 to 45.6 us.
    static int env_sk = -1;
    if (env_sk < 0) { const char* e = getenv("UB_GEMM_STREAMK"); env_sk = (e != nullptr && e[0] == '0') ? 0 : 1; }
    bool sk_ok = false;
    if (env_sk && !tl_no_sk && !dual && want_s <= 1 && a->tile_tokens <= 0 && a->tail_split != 1 && a->rs_world == 0 &&
        pairs_now <= SK_PAIRS_MAX && pairs_now > 0) {
      const int num_m2 = (a->M + tn2 - 1) / tn2, num_n2 = (a->N + 2 * BM_W - 1) / (2 * BM_W);
      const int teams = pairs_now / num_m2;                  // a team = one pair per token tile, in lockstep over K
      if (teams >= 2) {
        const long long total = (long long)num_n2 * num_kb;
        const int now_units = rounds2 * num_kb;
        const int sk_units = (int)((total + teams - 1) / teams);
        sk_ok = rounds2 >= 2 && sk_units >= 16 && (now_units - sk_units) * 4 >= now_units;
      }
    }
    if (want == 2 || (a->tile_tokens <= 0 && !short_single &&
                      ((gains && (enough || sk_ok) && !(ragged && !dual && !sk_ok)) || want_s > 1))) {
      pl.pair = 1;
      pl.tn = tn2;
      pl.tiles = tiles2;
      pl.tail_tiles = 0;
      pl.tail_splits = 1;
      pl.splits = (!dual && tn2 >= 128 && want_s > 1) ? want_s : 1;
      pl.ctas = pl.splits > 1 ? 2 * pl.splits * tiles2 : 2 * (tiles2 < pairs_now ? tiles2 : pairs_now);
      // Two-phase schedule for gated GEMMs on pairs: the full rounds run as one persistent launch, the weight rows of a
      // thin last round as a second launch of 1-CTA tiles (128 tokens) with K split over a cluster, because a pair
      // tile of 2 x 256 accumulator columns cannot park its partials (1020 x 14336 x 4096 gated: 224 pair tiles =
      // 3 x 74 + 2; 186.9 -> 164.3 us).  Plain GEMMs gain nothing from it: the split launch's fixed cost (cold
      // start, reduction through distributed shared memory, exposed epilogue) is a full round of their shorter tiles
      // (1020 x 6144 x 4096: 54.3 -> 60.2 us).
      if (sk_ok && pl.splits == 1 && want != 2) {
        pl.sk = 1;
        pl.ctas = 2 * pairs_now;
      }
      static int env_tail = -1;
      if (env_tail < 0) { const char* e = getenv("UB_GEMM_PAIR_TAIL"); env_tail = (e != nullptr && e[0] == '0') ? 0 : 1; }
      if (!pl.sk && env_tail && pl.splits == 1 && a->tile_tokens <= 0 && a->tail_split != 1 && a->rs_world == 0 &&
          tiles2 > pairs_now && num_kb >= 32) {
        const int num_m2 = (a->M + tn2 - 1) / tn2;
        const int main_t = (((tiles2 / pairs_now) * pairs_now) / num_m2) * num_m2;
        const int tail_t = tiles2 - main_t;
        if (main_t > 0 && tail_t > 0 && (main_t + pairs_now - 1) / pairs_now < rounds2) {
          if (dual && tn2 == 256) {
            const int num_m1 = (a->M + 127) / 128, num_n1 = (a->N + BM_W - 1) / BM_W;
            const int units = num_m1 * num_n1 - (main_t / num_m2) * 2 * num_m1;
            int ts = units > 0 ? sms / units : 0;
            if (ts > 8) ts = 8;
            while (ts & (ts - 1)) ts &= ts - 1;
            while (ts > 1 && (num_kb < 8 * ts || (ts - 1) * ((num_kb + ts - 1) / ts) >= num_kb)) ts >>= 1;
            while (ts > 1 && units > max_active_clusters(ts)) ts >>= 1;
            if (ts >= 2) {
              pl.tail_tiles = tail_t;
              pl.tail_splits = ts;
              pl.tail_units = units;
              pl.ctas = 2 * pairs_now + ts * units;
            }
          }
        }
      }
    }
  }
  return pl;
}

template <int TN, int STAGES, bool DUAL, bool SPLITK>
static int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, const GemmPlan& pl,
                       cudaStream_t stream) {
  using S = GemmSmem<TN, STAGES, DUAL, SPLITK>;
  static bool attr_set[UB_MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm_tn_kernel<TN, STAGES, DUAL, SPLITK>;
  if (dev < UB_MAX_DEVICES && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return -(int)e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = S::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  cfg.attrs = attr;
  cfg.numAttrs = 0;
  if (SPLITK) {
    cfg.gridDim = dim3(pl.splits, pl.tiles, 1);   // the caller passes a plan whose tiles/splits describe THIS launch
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pl.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.numAttrs = 1;
  } else {
    cfg.gridDim = dim3(pl.ctas, 1, 1);
  }
  cfg.numAttrs += pdl_attr(&attr[cfg.numAttrs]);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, tx, p);
  return e == cudaSuccess ? 0 : -(int)e;
}

template <int TN, int STAGES, bool DUAL, bool SPLITK>
static int launch_gemm_2cta(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, const GemmPlan& pl,
                            cudaStream_t stream) {
  using S = Gemm2Smem<TN, STAGES, DUAL, SPLITK>;
  static bool attr_set[UB_MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm_tn_2cta_kernel<TN, STAGES, DUAL, SPLITK>;
  if (dev < UB_MAX_DEVICES && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return -(int)e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.gridDim = SPLITK ? dim3(2 * pl.splits, pl.tiles, 1) : dim3(pl.ctas, 1, 1);
  cfg.dynamicSmemBytes = S::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = SPLITK ? 2 * pl.splits : 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1 + pdl_attr(&attr[1]);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, tx, p);
  return e == cudaSuccess ? 0 : -(int)e;
}

template <bool DUAL>
static int dispatch_2cta(int tn, const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, const GemmPlan& pl,
                         cudaStream_t st) {
  if (pl.splits > 1) {
    // split-K over pairs: plain GEMMs with 128 / 256-token tiles (the gated form would not fit its partials)
    if constexpr (!DUAL) {
      switch (tn) {
        case 128: return launch_gemm_2cta<128, 8, false, true>(tw, tx, p, pl, st);
        case 256: return launch_gemm_2cta<256, 6, false, true>(tw, tx, p, pl, st);
      }
    }
    return -4;
  }
  if constexpr (!DUAL) {
    switch (tn) {
      case 64: return launch_gemm_2cta<64, 10, false, false>(tw, tx, p, pl, st);
      case 128: return launch_gemm_2cta<128, 8, false, false>(tw, tx, p, pl, st);
      case 256: return launch_gemm_2cta<256, 6, false, false>(tw, tx, p, pl, st);
    }
  } else {
    switch (tn) {
      case 64: return launch_gemm_2cta<64, 5, true, false>(tw, tx, p, pl, st);
      case 128: return launch_gemm_2cta<128, 5, true, false>(tw, tx, p, pl, st);
      case 256: return launch_gemm_2cta<256, 4, true, false>(tw, tx, p, pl, st);
    }
  }
  return -4;
}

template <bool DUAL, bool SPLITK>
static int dispatch_tn(int tn, const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p,
                       const GemmPlan& pl, cudaStream_t st) {
  // Stage counts fill the 227 KB of one resident CTA per SM.
  if constexpr (!DUAL) {
    switch (tn) {
      case 16: return launch_gemm<16, 10, false, SPLITK>(tw, tx, p, pl, st);
      case 32: return launch_gemm<32, 9, false, SPLITK>(tw, tx, p, pl, st);
      case 64: return launch_gemm<64, 8, false, SPLITK>(tw, tx, p, pl, st);
      case 128: return launch_gemm<128, 6, false, SPLITK>(tw, tx, p, pl, st);
      case 256: return launch_gemm<256, 4, false, SPLITK>(tw, tx, p, pl, st);
    }
  } else {
    switch (tn) {
      case 16: return launch_gemm<16, 6, true, SPLITK>(tw, tx, p, pl, st);
      case 32: return launch_gemm<32, 5, true, SPLITK>(tw, tx, p, pl, st);
      case 64: return launch_gemm<64, 5, true, SPLITK>(tw, tx, p, pl, st);
      case 128: return launch_gemm<128, 4, true, SPLITK>(tw, tx, p, pl, st);
      case 256:
        // 2 x 256 accumulator columns fill TMEM: single-buffered, and too large to park for split-K.
        if constexpr (!SPLITK) return launch_gemm<256, 3, true, false>(tw, tx, p, pl, st);
        else return -5;
    }
  }
  return -4;
}

}  // namespace ub

extern "C" int ub_gemm_num_ctas(const UbGemmArgs* a) {
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return 0;
  return ub::plan_gemm(a).ctas;
}

extern "C" int ub_gemv_supported(const UbGemmArgs* a);
extern "C" int ub_gemv(const UbGemmArgs* a, void* stream);

extern "C" int ub_gemm_tn(const UbGemmArgs* a, void* stream_v) {
  using namespace ub;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return 0;
  {
    // up to 16 tokens: the weight-streaming kernel (csrc/gemm/gemv.cu); UB_GEMV=0 keeps the tcgen05 tiles
    static int gemv = -1;
    if (gemv < 0) { const char* e = getenv("UB_GEMV"); gemv = (e != nullptr && e[0] == '0') ? 0 : 1; }
    if (gemv && a->M <= 16 && a->tile_tokens <= 0 && a->splits <= 0 && a->cta_pair == 0 && ub_gemv_supported(a))
      return ub_gemv(a, stream_v);
  }
  if (a->K % 8 != 0 || a->ldx % 8 != 0 || a->ldw % 8 != 0) return -2;  // TMA strides must be 16-byte multiples
  if ((reinterpret_cast<uintptr_t>(a->x) & 15) || (reinterpret_cast<uintptr_t>(a->w) & 15)) return -3;
  const bool dual = a->dual != 0;
  GemmPlan pl = plan_gemm(a);
  GemmParams p;
  p.sk_on = 0;
  p.sk_ws = nullptr;
  p.sk_flags = nullptr;
  if (pl.sk) {
    if (sk_workspace(stream, &p.sk_ws, &p.sk_flags)) {
      p.sk_on = 1;
    } else {
      tl_no_sk = true;
      pl = plan_gemm(a);
      tl_no_sk = false;
    }
  }
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.out = reinterpret_cast<__nv_bfloat16*>(a->out);
  p.ldo = a->ldo;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a->bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a->residual);
  p.ldr = a->ldr;
  p.act = a->act;
  p.up_row_off = a->up_row_off;
  p.out_f32 = a->out_f32;
  p.out_scale = a->out_scale == 0.f ? 1.f : a->out_scale;
  p.err = a->err;
  p.splits = pl.splits;
  p.tile_begin = 0;
  p.tile_end = 0;
  {
    static int dbg = -1;
    if (dbg < 0) { const char* e = getenv("UB_GEMM_DEBUG"); dbg = e ? atoi(e) : 0; }
    p.dbg = dbg;
  }
  p.grp_tiles = reinterpret_cast<const int4*>(a->grp_tiles);
  p.grp_max_tiles = a->grp_max_tiles;
  p.grp_w_rows = a->grp_w_rows;
  if (p.grp_tiles != nullptr && (a->tile_tokens <= 0 || a->grp_max_tiles <= 0 || a->grp_w_rows <= 0 || a->rs_world > 0 ||
                                 a->ag_world > 0 || a->bias != nullptr))
    return -6;  // grouped mode: fixed token tile, no bias, no fused collectives
  p.rs_world = a->rs_world; p.rs_rank = a->rs_rank; p.rs_rows_per_rank = a->rs_rows_per_rank;
  p.ag_world = a->ag_world; p.ag_rows_per_rank = a->ag_rows_per_rank;
  p.ag_flags = a->ag_flags; p.ag_epoch = a->ag_epoch; p.ag_signals_per_use = a->ag_signals_per_use;
  for (int i = 0; i < UB_MAX_RANKS; ++i) {
    p.rs_peer_out[i] = reinterpret_cast<__nv_bfloat16*>(a->rs_peer_out[i]);
    p.rs_peer_flag[i] = a->rs_peer_flag[i];
  }
  p.rs_local_count = a->rs_local_count;
  p.rs_total = (uint32_t)pl.ctas;          // every CTA of this GEMM (both launches of a two-phase schedule) arrives once
  if (p.rs_world > 0 && p.rs_local_count == nullptr) return -8;
  CUtensorMap tw, tx;
  const long long w_rows = (dual || a->grp_tiles != nullptr) ? (long long)a->w_rows_total : (long long)a->N;
  int rc = make_tmap_bf16_2d(&tw, a->w, w_rows, a->K, a->ldw, BM_W, BK);
  if (rc != 0) return rc;
  rc = make_tmap_bf16_2d(&tx, a->x, a->M, a->K, a->ldx, pl.pair ? pl.tn / 2 : pl.tn, BK);
  if (rc != 0) return rc;
  if (pl.pair && pl.tail_tiles == 0)
    return dual ? dispatch_2cta<true>(pl.tn, tw, tx, p, pl, stream) : dispatch_2cta<false>(pl.tn, tw, tx, p, pl, stream);
  if (pl.pair) {
    // phase 1: the full rounds on CTA pairs, persistent
    GemmPlan main_pl = pl;
    main_pl.tiles = pl.tiles - pl.tail_tiles;
    main_pl.splits = 1;
    const int pairs_now = max_active_clusters(2);
    main_pl.ctas = 2 * (main_pl.tiles < pairs_now ? main_pl.tiles : pairs_now);
    p.splits = 1;
    p.tile_begin = 0;
    p.tile_end = main_pl.tiles;
    if (!dual) return -4;                      // the planner makes this plan for gated GEMMs only
    rc = dispatch_2cta<true>(pl.tn, tw, tx, p, main_pl, stream);
    if (rc != 0) return rc;
    // phase 2: the thin last round, K split
    GemmPlan tail_pl = pl;
    tail_pl.splits = pl.tail_splits;
    p.splits = pl.tail_splits;
    // gated: the tail's weight rows as 1-CTA tiles of 128 tokens (pair row r = 1-CTA weight tiles 2r and 2r + 1)
    CUtensorMap tx1;
    rc = make_tmap_bf16_2d(&tx1, a->x, a->M, a->K, a->ldx, 128, BK);
    if (rc != 0) return rc;
    const int num_m1 = (a->M + 127) / 128, num_n1 = (a->N + BM_W - 1) / BM_W;
    tail_pl.pair = 0;
    tail_pl.tn = 128;
    tail_pl.tiles = pl.tail_units;
    p.tile_end = num_m1 * num_n1;
    p.tile_begin = p.tile_end - pl.tail_units;
    return dispatch_tn<true, true>(128, tw, tx1, p, tail_pl, stream);
  }
  if (pl.splits > 1) {
    return dual ? dispatch_tn<true, true>(pl.tn, tw, tx, p, pl, stream)
                : dispatch_tn<false, true>(pl.tn, tw, tx, p, pl, stream);
  }
  if (pl.tail_tiles == 0) {
    return dual ? dispatch_tn<true, false>(pl.tn, tw, tx, p, pl, stream)
                : dispatch_tn<false, false>(pl.tn, tw, tx, p, pl, stream);
  }
  // phase 1: full rounds, persistent
  GemmPlan main_pl = pl;
  main_pl.tiles = pl.tiles - pl.tail_tiles;
  const int sms = num_sms();
  main_pl.ctas = main_pl.tiles < sms ? main_pl.tiles : sms;
  p.tile_begin = 0;
  p.tile_end = main_pl.tiles;
  rc = dual ? dispatch_tn<true, false>(pl.tn, tw, tx, p, main_pl, stream)
            : dispatch_tn<false, false>(pl.tn, tw, tx, p, main_pl, stream);
  if (rc != 0) return rc;
  // phase 2: the leftover tiles, K split over clusters
  GemmPlan tail_pl = pl;
  tail_pl.tiles = pl.tail_tiles;
  tail_pl.splits = pl.tail_splits;
  p.tile_begin = main_pl.tiles;
  p.tile_end = pl.tiles;
  p.splits = pl.tail_splits;
  return dual ? dispatch_tn<true, true>(pl.tn, tw, tx, p, tail_pl, stream)
              : dispatch_tn<false, true>(pl.tn, tw, tx, p, tail_pl, stream);
}

// Lowers every stream-K flag of the current device (after a launch that gave up in a bounded wait and may have left
// some raised).  Ordered on `stream`.
extern "C" int ub_gemm_streamk_reset(void* stream_v) {
  using namespace ub;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= UB_MAX_DEVICES) return 0;
  std::lock_guard<std::mutex> lock(g_sk_mu);
  if (g_sk[dev].flags == nullptr) return 0;
  cudaError_t e = cudaMemsetAsync(g_sk[dev].flags, 0, SK_LANES * SK_LANE_FLAGS * sizeof(uint32_t),
                                  reinterpret_cast<cudaStream_t>(stream_v));
  return e == cudaSuccess ? 0 : -(int)e;
}

// Copies the timeline table of the last 1-CTA launches (UB_GEMM_DEBUG bit 4) to `out` ([512][12] uint64, nanoseconds).
extern "C" int ub_gemm_debug_timeline(unsigned long long* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, ub::g_gemm_ts, sizeof(unsigned long long) * ub::TS_CTAS * 12);
  return e == cudaSuccess ? 0 : -(int)e;
}
