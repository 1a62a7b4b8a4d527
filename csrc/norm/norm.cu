// K5: RMSNorm / LayerNorm with fused residual add, plus the two collective roles it plays in the
// tensor-parallel pipeline:
//   * F1 consumer: the input may be `rs_world` partial slots pushed by the GEMM+reduce-scatter
//     epilogues of all ranks; the kernel waits (bounded) on the local counter, sums the slots in
//     fp32 in a fixed order (deterministic) and continues as usual.
//   * F3 producer: the normalised row is also stored into every peer's all-gather buffer (plain
//     16-byte peer stores over NVLink) and a per-source counter is bumped on each peer.
// One CTA per token row; the row is staged in shared memory as fp32.
//
// Replaces in the reference: ops_fn::layer_norm / rms_norm / fused_residual_rms_norm
// (crates/runtime/src/tensor_core.rs:973-1008, 1130-1143, 1398-1423) and the AVX2/NEON rms_norm
// (crates/runtime/src/simd/arch/avx2.rs:155-201).
#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"

namespace ub {

struct NormParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* weight;
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;
  __nv_bfloat16* residual_out;
  int* err;
  int T, H;
  float eps;
  int kind, weight_offset_one;
  int rs_world;
  const uint32_t* rs_flag;
  const uint32_t* epoch;
  uint32_t rs_signals_per_use;
  int ag_world, ag_rank;
  __nv_bfloat16* ag_peer_out[UB_MAX_RANKS];
  uint32_t* ag_peer_flag[UB_MAX_RANKS];
  uint32_t* reset_flags;   // local counters that no kernel is using right now; zeroed by block 0 before it signals
  int reset_count;
  uint32_t* ag_local_count;   // local arrival counter of the row CTAs (see publish_to_peers)
  int rs_multimem;            // x is a multicast address: rows are read with multimem.ld_reduce (sum over all ranks)
  __nv_bfloat16* ag_mc_out;   // multicast address of the gather buffer: one multimem.st per 16 bytes instead of peer stores
};

// 8 bf16 values, each the sum (fp32 accumulation inside the switch) of the values at this offset on every rank
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
// 16 bytes to the same offset on every rank
__device__ __forceinline__ void multimem_st_16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// CH > 0: H is a multiple of 8 and at most 2048 * CH, every thread keeps its (at most CH) 16-byte chunks of the row in
// registers between the two passes; CH == 0: any H, the row is staged in shared memory as fp32.
template <int CH>
__global__ void __launch_bounds__(256) norm_kernel(const NormParams p) {
  pdl_launch_dependents();     // the next kernel may start its private set-up now
  pdl_wait();                  // nothing global is touched before the previous kernel has completed
  extern __shared__ float row[];  // [H] (CH == 0 only)
  float fr[CH > 0 ? CH : 1][8];
  __shared__ float red[32];
  __shared__ int wait_failed;
  const int t = blockIdx.x;
  const int H = p.H;
  const bool vec = (H % 8 == 0);

  if (blockIdx.x == 0 && threadIdx.x < p.reset_count) {
    // Flag hygiene: counters are reset to zero between uses by a kernel that is ordered (through the
    // data dependencies of the layer pipeline) after their last reader and before their next writer.
    p.reset_flags[threadIdx.x] = 0u;
    __threadfence_system();
  }
  if (p.rs_world > 0) {
    if (threadIdx.x == 0) {
      wait_failed = 0;
      const uint32_t want = p.rs_signals_per_use;
      const uint64_t t0 = wait_ticks();
      uint32_t it = 0, v;
      while (true) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.rs_flag) : "memory");
        if (int32_t(v - want) >= 0) break;
        if ((++it & 31u) == 0 && wait_expired(t0, p.err)) {
          set_err(p.err, ERR_FLAG_TIMEOUT, 1000 + t);
          wait_failed = 1;
          break;
        }
      }
    }
    __syncthreads();
  }

  const int nslots = (p.rs_world > 0 && !p.rs_multimem) ? p.rs_world : 1;
  const long long slot_stride = (long long)p.T * H;
  float ssum = 0.f, ssq = 0.f;
  if (vec) {
    auto load_chunk = [&](int c, float* keep) {
      float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      // all slots' loads are issued before the first sum (a loop over a run-time slot count issued them one latency
      // after the other: 13 us of a 19 us launch at 8 slots); slots are summed in rank order, as before
      uint4 sv[UB_MAX_RANKS];
#pragma unroll
      for (int s = 0; s < UB_MAX_RANKS; ++s) {
        if (s < nslots) {
          // L2-only load: with rs_world > 0 these rows were written by peers and L1 may hold a stale line
          sv[s] = p.rs_multimem ? multimem_ld_reduce_bf16x8(p.x + (long long)t * H + c * 8)
                                : __ldcg(reinterpret_cast<const uint4*>(p.x + s * slot_stride + (long long)t * H + c * 8));
        }
      }
#pragma unroll
      for (int s = 0; s < UB_MAX_RANKS; ++s) {
        if (s < nslots) {
          const uint32_t* a = reinterpret_cast<const uint32_t*>(&sv[s]);
#pragma unroll
          for (int e = 0; e < 4; ++e) { f[2 * e] += bf16_lo(a[e]); f[2 * e + 1] += bf16_hi(a[e]); }
        }
      }
      if (p.residual != nullptr) {
        const uint4 v = *reinterpret_cast<const uint4*>(p.residual + (long long)t * H + c * 8);
        const uint32_t* a = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) { f[2 * e] += bf16_lo(a[e]); f[2 * e + 1] += bf16_hi(a[e]); }
      }
      if (p.residual_out != nullptr) {
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          o[e] = pack_bf16x2(f[2 * e], f[2 * e + 1]);
          // normalise the value that is actually stored so that later layers see a consistent residual
          f[2 * e] = bf16_lo(o[e]); f[2 * e + 1] = bf16_hi(o[e]);
        }
        *reinterpret_cast<uint4*>(p.residual_out + (long long)t * H + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) { keep[e] = f[e]; ssum += f[e]; ssq += f[e] * f[e]; }
    };
    if constexpr (CH > 0) {
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        const int c = threadIdx.x + k * 256;
        if (c < H / 8) load_chunk(c, fr[k]);
      }
    } else {
      for (int c = threadIdx.x; c < H / 8; c += blockDim.x) load_chunk(c, row + c * 8);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float f = 0.f;
      for (int s = 0; s < nslots; ++s) f += __bfloat162float(p.x[s * slot_stride + (long long)t * H + i]);
      if (p.residual != nullptr) f += __bfloat162float(p.residual[(long long)t * H + i]);
      if (p.residual_out != nullptr) {
        __nv_bfloat16 b = __float2bfloat16(f);
        p.residual_out[(long long)t * H + i] = b;
        f = __bfloat162float(b);
      }
      row[i] = f; ssum += f; ssq += f * f;
    }
  }
  float mean = 0.f, rstd;
  if (p.kind == 1) {
    mean = block_sum(ssum, red) / H;
    // two-pass variance for accuracy
    float sv = 0.f;
    if constexpr (CH > 0) {
#pragma unroll
      for (int k = 0; k < CH; ++k)
        if (threadIdx.x + k * 256 < H / 8) {
#pragma unroll
          for (int e = 0; e < 8; ++e) { const float d = fr[k][e] - mean; sv += d * d; }
        }
    } else {
      for (int i = threadIdx.x; i < H; i += blockDim.x) { float d = row[i] - mean; sv += d * d; }
    }
    rstd = rsqrtf(block_sum(sv, red) / H + p.eps);
  } else {
    rstd = rsqrtf(block_sum(ssq, red) / H + p.eps);
  }

  const float woff = p.weight_offset_one ? 1.f : 0.f;
  if (vec) {
    auto store_chunk = [&](int c, const float* kept) {
      float w[8], b[8];
      if (p.weight != nullptr) {
        const uint4 v = *reinterpret_cast<const uint4*>(p.weight + c * 8);
        const uint32_t* a = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) { w[2 * e] = bf16_lo(a[e]) + woff; w[2 * e + 1] = bf16_hi(a[e]) + woff; }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = 1.f;
      }
      if (p.bias != nullptr) {
        const uint4 v = *reinterpret_cast<const uint4*>(p.bias + c * 8);
        const uint32_t* a = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) { b[2 * e] = bf16_lo(a[e]); b[2 * e + 1] = bf16_hi(a[e]); }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) b[e] = 0.f;
      }
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float y0 = (kept[2 * e] - mean) * rstd * w[2 * e] + b[2 * e];
        const float y1 = (kept[2 * e + 1] - mean) * rstd * w[2 * e + 1] + b[2 * e + 1];
        o[e] = pack_bf16x2(y0, y1);
      }
      const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
      if (p.out != nullptr) *reinterpret_cast<uint4*>(p.out + (long long)t * H + c * 8) = ov;
      if (p.ag_world > 0) {
        const long long grow = (long long)p.ag_rank * p.T + t;
        if (p.ag_mc_out != nullptr) {
          multimem_st_16(p.ag_mc_out + grow * H + c * 8, ov);
        } else {
          for (int r = 0; r < p.ag_world; ++r)
            *reinterpret_cast<uint4*>(p.ag_peer_out[r] + grow * H + c * 8) = ov;
        }
      }
    };
    if constexpr (CH > 0) {
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        const int c = threadIdx.x + k * 256;
        if (c < H / 8) store_chunk(c, fr[k]);
      }
    } else {
      for (int c = threadIdx.x; c < H / 8; c += blockDim.x) store_chunk(c, row + c * 8);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float w = p.weight != nullptr ? __bfloat162float(p.weight[i]) + woff : 1.f;
      const float b = p.bias != nullptr ? __bfloat162float(p.bias[i]) : 0.f;
      const __nv_bfloat16 y = __float2bfloat16((row[i] - mean) * rstd * w + b);
      if (p.out != nullptr) p.out[(long long)t * H + i] = y;
      if (p.ag_world > 0) {
        const long long grow = (long long)p.ag_rank * p.T + t;
        for (int r = 0; r < p.ag_world; ++r) p.ag_peer_out[r][grow * H + i] = y;
      }
    }
  }
  if (p.ag_world > 0) {
    // the row CTAs arrive locally; the last one tells every peer that ALL rows of this rank are there
    __syncthreads();
    if (threadIdx.x == 0) publish_to_peers(p.ag_local_count, gridDim.x, p.ag_peer_flag, p.ag_world);
  }
}

__global__ void bump_epoch_kernel(uint32_t* e) { *e = *e + 1; }

__global__ void wait_flag_kernel(const uint32_t* flags, uint32_t value, int* err) {
  const uint32_t* flag = flags + threadIdx.x;   // one thread per counter
  const uint64_t t0 = wait_ticks();
  uint32_t it = 0, v;
  while (true) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (int32_t(v - value) >= 0) return;
    if ((++it & 31u) == 0 && wait_expired(t0, err)) {
      set_err(err, ERR_FLAG_TIMEOUT, 2000);
      return;
    }
  }
}

}  // namespace ub

extern "C" int ub_norm(const UbNormArgs* a, void* stream_v) {
  using namespace ub;
  if (a->T <= 0 || a->H <= 0) return 0;
  if ((size_t)a->H * 4 > 160 * 1024) return -2;
  NormParams p;
  p.x = (const __nv_bfloat16*)a->x; p.residual = (const __nv_bfloat16*)a->residual;
  p.weight = (const __nv_bfloat16*)a->weight; p.bias = (const __nv_bfloat16*)a->bias;
  p.out = (__nv_bfloat16*)a->out; p.residual_out = (__nv_bfloat16*)a->residual_out;
  p.err = a->err; p.T = a->T; p.H = a->H; p.eps = a->eps; p.kind = a->kind;
  p.weight_offset_one = a->weight_offset_one;
  p.rs_world = a->rs_world; p.rs_flag = a->rs_flag; p.epoch = a->epoch;
  p.rs_signals_per_use = a->rs_signals_per_use;
  p.ag_world = a->ag_world; p.ag_rank = a->ag_rank;
  p.reset_flags = a->reset_flags; p.reset_count = a->reset_count;
  p.ag_local_count = a->ag_local_count;
  if (p.ag_world > 0 && p.ag_local_count == nullptr) return -8;
  p.rs_multimem = a->rs_multimem;
  p.ag_mc_out = (__nv_bfloat16*)a->ag_mc_out;
  if ((p.rs_multimem || p.ag_mc_out != nullptr) && a->H % 8 != 0) return -9;   // the multicast paths are 16-byte vector only
  for (int i = 0; i < UB_MAX_RANKS; ++i) {
    p.ag_peer_out[i] = (__nv_bfloat16*)a->ag_peer_out[i];
    p.ag_peer_flag[i] = a->ag_peer_flag[i];
  }
  cudaError_t e;
  if (a->H % 8 == 0 && a->H <= 2048 * 2) {
    e = ub::launch_pdl(norm_kernel<2>, dim3(a->T), dim3(256), (size_t)0, (cudaStream_t)stream_v, p);
  } else if (a->H % 8 == 0 && a->H <= 2048 * 4) {
    e = ub::launch_pdl(norm_kernel<4>, dim3(a->T), dim3(256), (size_t)0, (cudaStream_t)stream_v, p);
  } else {
    const size_t smem = (size_t)a->H * 4;
    static bool attr_set[UB_MAX_DEVICES] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && dev < UB_MAX_DEVICES && !attr_set[dev]) {
      cudaFuncSetAttribute(norm_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      attr_set[dev] = true;
    }
    e = ub::launch_pdl(norm_kernel<0>, dim3(a->T), dim3(256), smem, (cudaStream_t)stream_v, p);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int ub_bump_epoch(uint32_t* epoch, void* stream_v) {
  ub::bump_epoch_kernel<<<1, 1, 0, (cudaStream_t)stream_v>>>(epoch);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int ub_wait_flags(const uint32_t* flags, int n, uint32_t value, int* err, void* stream_v) {
  if (n < 1 || n > 32) return -2;
  ub::wait_flag_kernel<<<1, n, 0, (cudaStream_t)stream_v>>>(flags, value, err);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int ub_wait_flag(const uint32_t* flag, uint32_t value, int* err, void* stream_v) {
  ub::wait_flag_kernel<<<1, 1, 0, (cudaStream_t)stream_v>>>(flag, value, err);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
