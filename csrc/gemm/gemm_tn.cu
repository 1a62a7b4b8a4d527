// K1/K2/F1/F3: bf16 "TN" GEMM on 5th-gen tensor cores:  out[M, N] = epilogue(x[M, K] @ w[N, K]^T).
//
// Design (sm_100a only):
//  * Weights stay in the on-disk HF layout [out_features, in_features]; both operands are K-major.
//  * The weight tile is ALWAYS the 128-row MMA "A" operand and the token tile is the MMA "N"
//    operand (16..256 tokens).  A decode batch of 16 tokens and a prefill chunk of 8192 tokens
//    run the same kernel; only the token-tile width changes.  The accumulator in TMEM therefore
//    holds out^T: TMEM lane = output feature, TMEM column = token.
//  * Warp roles: warp 0 = TMA producer, warp 1 = tcgen05.mma issuer and TMEM owner,
//    warps 2..5 = epilogue (TMEM -> registers -> smem transpose -> 16-byte global stores).
//  * DUAL mode (K2): two weight tiles (gate rows, up rows) share one token tile and fill two
//    accumulators; the epilogue writes act(gate) * up, so SwiGLU/GeGLU never touches HBM.
//  * Collective fusion.  F1 (GEMM + reduce-scatter): the epilogue stores each output row straight
//    into the symmetric receive buffer of the rank that owns that token (peer pointer, plain
//    16-byte stores over NVLink), then bumps a counter on every peer.  F3 (all-gather + GEMM):
//    the TMA producer waits (bounded) on the per-source counters before it loads token rows that
//    another rank pushed into this rank's gather buffer.
//  * Every wait is bounded; a timeout sets the error word and the kernel drains and frees TMEM.
//
// Replaces in the reference: ops_fn::matmul (crates/runtime/src/tensor_core.rs:843-892), the
// QMatMul call sites (models_v2/llama.rs:1184-1195) and fused_swiglu (tensor_core.rs:1385-1396).
#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"

namespace ub {

constexpr int BM_W = 128;  // weight rows per tile (MMA M)
constexpr int BK = 64;     // K elements per stage (one 128-byte swizzle atom of bf16)
constexpr int UMMA_K = 16;

struct GemmParams {
  int M, N, K;
  __nv_bfloat16* out;
  long long ldo;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null
  long long ldr;
  int act;          // UB_ACT_*
  int up_row_off;   // DUAL: row offset of the "up" half inside w
  int out_f32;      // 1: out is float* (ldo in floats), no residual/bias fusion restrictions
  float out_scale;  // multiplies the result before bias/residual (1.0 = none)
  int* err;
  // F1: reduce-scatter push.  rs_world == 0 disables.
  int rs_world, rs_rank, rs_rows_per_rank;
  __nv_bfloat16* rs_peer_out[UB_MAX_RANKS];  // each: [world][rows_per_rank][ldo]
  uint32_t* rs_peer_flag[UB_MAX_RANKS];      // counter to bump on each peer
  // F3: all-gather wait.  ag_world == 0 disables.
  int ag_world, ag_rows_per_rank;
  const uint32_t* ag_flags;     // [world] counters in local memory, one per source rank
  const uint32_t* ag_epoch;     // device word: number of completed uses + 1
  uint32_t ag_signals_per_use;  // counter increments per source rank per use
};

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case UB_ACT_SILU: return v / (1.f + __expf(-v));
    case UB_ACT_GELU: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    case UB_ACT_GELU_TANH: {
      float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
      return 0.5f * v * (1.f + tanhf(u));
    }
    case UB_ACT_RELU: return fmaxf(v, 0.f);
    case UB_ACT_RELU2: { float r = fmaxf(v, 0.f); return r * r; }
    case UB_ACT_QUICK_GELU: return v / (1.f + __expf(-1.702f * v));
    default: return v;
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

template <int TN, int STAGES, bool DUAL>
struct GemmSmem {
  static constexpr int A_BYTES = BM_W * BK * 2;  // 16 KB
  static constexpr int B_BYTES = TN * BK * 2;
  static constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * A_BYTES + B_BYTES;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int STAGING_BYTES = TN * BM_W * 4;  // worst case fp32 staging
  static constexpr int DATA_BYTES = TILE_BYTES > STAGING_BYTES ? TILE_BYTES : STAGING_BYTES;
  static constexpr int TOTAL = DATA_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

template <int TN, int STAGES, bool DUAL>
__global__ void __launch_bounds__(192, (GemmSmem<TN, STAGES, DUAL>::TOTAL <= 112 * 1024) ? 2 : 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const GemmParams p) {
  using S = GemmSmem<TN, STAGES, DUAL>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::DATA_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * TN;     // first token of this tile
  const int n0 = blockIdx.y * BM_W;   // first output feature of this tile
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS_NEEDED = (DUAL ? 2 : 1) * TN;
  constexpr uint32_t TMEM_COLS = TMEM_COLS_NEEDED < 32 ? 32 : TMEM_COLS_NEEDED;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full_bar, 1);
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

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      if (p.ag_world > 0) {
        // Token rows [m0, m0+TN) were pushed by the ranks that own them; wait for those sources.
        const uint32_t want = (*p.ag_epoch) * p.ag_signals_per_use;
        int r_lo = m0 / p.ag_rows_per_rank;
        int m_hi = min(m0 + TN, p.M) - 1;
        int r_hi = m_hi / p.ag_rows_per_rank;
        if (r_hi >= p.ag_world) r_hi = p.ag_world - 1;
        const uint64_t t0 = globaltimer_ns();
        for (int r = r_lo; r <= r_hi; ++r) {
          uint32_t it = 0;
          while (int32_t(ld_acquire_sys_u32(p.ag_flags + r) - want) < 0) {
            if ((++it & 31u) == 0 && (globaltimer_ns() - t0 > UB_WAIT_NS)) {
              *abort_flag = 1;
              set_err(p.err, ERR_FLAG_TIMEOUT, r);
              break;
            }
          }
        }
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.err, 100 + s)) break;  // stop issuing copies
        uint8_t* st = smem + s * S::STAGE_BYTES;
        mbar_arrive_expect_tx(&full_bar[s], S::STAGE_BYTES);
        tma_load_2d_hint(st, &tmap_w, &full_bar[s], kb * BK, n0, pol_w);
        if (DUAL) tma_load_2d_hint(st + S::A_BYTES, &tmap_w, &full_bar[s], kb * BK, n0 + p.up_row_off, pol_w);
        tma_load_2d_hint(st + (DUAL ? 2 : 1) * S::A_BYTES, &tmap_x, &full_bar[s], kb * BK, m0, pol_x);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM_W, TN, 0, 0);
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&full_bar[s], ph, abort_flag, p.err, 200 + s)) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * S::STAGE_BYTES);
        const uint32_t b_addr = a_addr + (DUAL ? 2 : 1) * S::A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t bdesc = make_smem_desc_sw128(b_addr + k * UMMA_K * 2, 16, 1024);
          const uint64_t adesc = make_smem_desc_sw128(a_addr + k * UMMA_K * 2, 16, 1024);
          const uint32_t acc = (kb | k) != 0 ? 1u : 0u;
          umma_bf16_ss(tmem_base, adesc, bdesc, idesc, acc);
          if (DUAL) {
            const uint64_t a2desc = make_smem_desc_sw128(a_addr + S::A_BYTES + k * UMMA_K * 2, 16, 1024);
            umma_bf16_ss(tmem_base + TN, a2desc, bdesc, idesc, acc);
          }
        }
        umma_commit(&empty_bar[s]);  // stage is free once these MMAs have read it
      }
      umma_commit(tmem_full_bar);
    }
  } else {
    // ------------------------------ epilogue (warps 2..5) ------------------------------
    const int q = warp & 3;           // TMEM lane quarter this warp may read
    const int et = q * 32 + lane;     // 0..127 : output feature inside the tile == TMEM lane
    const int tid_e = threadIdx.x - 64;
    mbar_wait(tmem_full_bar, 0, abort_flag, p.err, 300);
    tc_fence_after();
    const int n = n0 + et;
    float bias_v = 0.f;
    if (p.bias != nullptr && n < p.N) bias_v = __bfloat162float(p.bias[n]);
    // Staging tile in smem (aliases the pipeline stages, which are idle now): [TN][128] of bf16 or fp32.
    __nv_bfloat16* stage_bf = reinterpret_cast<__nv_bfloat16*>(smem);
    float* stage_f = reinterpret_cast<float*>(smem);
    const uint32_t lane_addr = tmem_base + (uint32_t(q * 32) << 16);
    constexpr int CH = TN >= 32 ? 32 : 16;
#pragma unroll 1
    for (int c = 0; c < TN / CH; ++c) {
      uint32_t r[CH];
      uint32_t r2[CH];
      if constexpr (CH == 32) {
        tmem_ld_32x32(lane_addr + c * CH, r);
        if (DUAL) tmem_ld_32x32(lane_addr + TN + c * CH, r2);
      } else {
        tmem_ld_32x16(lane_addr + c * CH, r);
        if (DUAL) tmem_ld_32x16(lane_addr + TN + c * CH, r2);
      }
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        float v = __uint_as_float(r[j]) * p.out_scale;
        if (DUAL) {
          v = apply_act(v, p.act) * (__uint_as_float(r2[j]) * p.out_scale);
        } else {
          v += bias_v;
          v = apply_act(v, p.act);
        }
        const int tok = c * CH + j;
        if (p.out_f32) stage_f[tok * BM_W + et] = v;
        else stage_bf[tok * BM_W + et] = __float2bfloat16(v);
      }
    }
    tc_fence_before();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // Coalesced write-out: each token row of the tile is 128 features.
    if (p.out_f32) {
      float* outf = reinterpret_cast<float*>(p.out);
      for (int idx = tid_e; idx < TN * 32; idx += 128) {
        const int tok = idx >> 5, c4 = idx & 31;
        const int m = m0 + tok, nn = n0 + c4 * 4;
        if (m < p.M && nn < p.N) {
          float4 v = *reinterpret_cast<const float4*>(stage_f + tok * BM_W + c4 * 4);
          float* dst = outf + (long long)m * p.ldo + nn;
          if (nn + 4 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
            *reinterpret_cast<float4*>(dst) = v;
          } else {
            const float vv[4] = {v.x, v.y, v.z, v.w};
            for (int e = 0; e < 4 && nn + e < p.N; ++e) dst[e] = vv[e];
          }
        }
      }
    } else {
      const bool vec_ok = (p.N % 8 == 0) && (p.ldo % 8 == 0) &&
                          ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                          (p.residual == nullptr ||
                           ((p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0)));
      for (int idx = tid_e; idx < TN * 16; idx += 128) {
        const int tok = idx >> 4, c8 = idx & 15;
        const int m = m0 + tok, nn = n0 + c8 * 8;
        if (m >= p.M || nn >= p.N) continue;
        uint4 v = *reinterpret_cast<const uint4*>(stage_bf + tok * BM_W + c8 * 8);
        __nv_bfloat16* dst_base = p.out;
        long long row = m;
        if (p.rs_world > 0) {
          int owner = m / p.rs_rows_per_rank;
          if (owner >= p.rs_world) owner = p.rs_world - 1;
          dst_base = p.rs_peer_out[owner];
          row = (long long)p.rs_rank * p.rs_rows_per_rank + (m - owner * p.rs_rows_per_rank);
        }
        __nv_bfloat16* dst = dst_base + row * p.ldo + nn;
        if (vec_ok) {
          if (p.residual != nullptr) {
            const uint4 rr = *reinterpret_cast<const uint4*>(p.residual + (long long)m * p.ldr + nn);
            const uint32_t* a = reinterpret_cast<const uint32_t*>(&v);
            const uint32_t* b = reinterpret_cast<const uint32_t*>(&rr);
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              o[e] = pack_bf16x2(bf16_lo(a[e]) + bf16_lo(b[e]), bf16_hi(a[e]) + bf16_hi(b[e]));
            v = make_uint4(o[0], o[1], o[2], o[3]);
          }
          *reinterpret_cast<uint4*>(dst) = v;
        } else {
          const __nv_bfloat16* sv = reinterpret_cast<const __nv_bfloat16*>(&v);
          for (int e = 0; e < 8 && nn + e < p.N; ++e) {
            float f = __bfloat162float(sv[e]);
            if (p.residual != nullptr) f += __bfloat162float(p.residual[(long long)m * p.ldr + nn + e]);
            dst[e] = __float2bfloat16(f);
          }
        }
      }
    }
    if (p.rs_world > 0) {
      // Publish: every storing thread fences to system scope, then one thread per peer bumps its counter.
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (tid_e < p.rs_world) red_release_sys_add_u32(p.rs_peer_flag[tid_e], 1u);
    }
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

// 2-D bf16 tensor map, rows x cols (cols contiguous), box = box_rows x 64 columns, 128-byte swizzle.
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld_elems,
                      int box_rows, int box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld_elems * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

template <int TN, int STAGES, bool DUAL>
static int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, cudaStream_t stream) {
  using S = GemmSmem<TN, STAGES, DUAL>;
  static bool attr_set[UB_MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < UB_MAX_DEVICES && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tn_kernel<TN, STAGES, DUAL>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return -(int)e;
    attr_set[dev] = true;
  }
  dim3 grid((p.M + TN - 1) / TN, (p.N + BM_W - 1) / BM_W, 1);
  gemm_tn_kernel<TN, STAGES, DUAL><<<grid, 192, S::TOTAL, stream>>>(tw, tx, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

}  // namespace ub

extern "C" int ub_gemm_tn(const UbGemmArgs* a, void* stream_v) {
  using namespace ub;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return 0;
  if (a->K % 8 != 0 || a->ldx % 8 != 0 || a->ldw % 8 != 0) return -2;  // TMA strides must be 16-byte multiples
  if ((reinterpret_cast<uintptr_t>(a->x) & 15) || (reinterpret_cast<uintptr_t>(a->w) & 15)) return -3;
  const bool dual = a->dual != 0;
  int tn = a->tile_tokens;
  if (tn <= 0) {
    tn = 16;
    while (tn < a->M && tn < 256) tn <<= 1;
  }
  GemmParams p;
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
  p.rs_world = a->rs_world; p.rs_rank = a->rs_rank; p.rs_rows_per_rank = a->rs_rows_per_rank;
  p.ag_world = a->ag_world; p.ag_rows_per_rank = a->ag_rows_per_rank;
  p.ag_flags = a->ag_flags; p.ag_epoch = a->ag_epoch; p.ag_signals_per_use = a->ag_signals_per_use;
  for (int i = 0; i < UB_MAX_RANKS; ++i) {
    p.rs_peer_out[i] = reinterpret_cast<__nv_bfloat16*>(a->rs_peer_out[i]);
    p.rs_peer_flag[i] = a->rs_peer_flag[i];
  }
  CUtensorMap tw, tx;
  const long long w_rows = dual ? (long long)a->w_rows_total : (long long)a->N;
  int rc = make_tmap_bf16_2d(&tw, a->w, w_rows, a->K, a->ldw, BM_W, BK);
  if (rc != 0) return rc;
  rc = make_tmap_bf16_2d(&tx, a->x, a->M, a->K, a->ldx, tn, BK);
  if (rc != 0) return rc;
  if (!dual) {
    switch (tn) {
      // Stage counts: token tiles up to 128 keep two CTAs resident per SM (one CTA's epilogue hides
      // behind the other's main loop); the 256-token tile owns the SM.
      case 16: return launch_gemm<16, 6, false>(tw, tx, p, stream);
      case 32: return launch_gemm<32, 5, false>(tw, tx, p, stream);
      case 64: return launch_gemm<64, 4, false>(tw, tx, p, stream);
      case 128: return launch_gemm<128, 3, false>(tw, tx, p, stream);
      case 256: return launch_gemm<256, 4, false>(tw, tx, p, stream);
    }
  } else {
    switch (tn) {
      case 16: return launch_gemm<16, 3, true>(tw, tx, p, stream);
      case 32: return launch_gemm<32, 3, true>(tw, tx, p, stream);
      case 64: return launch_gemm<64, 5, true>(tw, tx, p, stream);
      case 128: return launch_gemm<128, 4, true>(tw, tx, p, stream);
      case 256: return launch_gemm<256, 3, true>(tw, tx, p, stream);
    }
  }
  return -4;
}
