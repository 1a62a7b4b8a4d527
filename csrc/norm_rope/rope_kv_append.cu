// K6: per-head RMSNorm (optional, QK-norm models) + rotary embedding of q and k + append of the
// rotated k and of v into the paged KV cache, in one pass over the QKV GEMM output.
// Cache layout: [num_blocks, Hkv, block_size, D] bf16 for K and for V, so one (block, head) page
// is a contiguous block_size x D tile that attention kernels can fetch with bulk copies.
// One CTA per token, one warp per head (round-robin).  cos/sin are computed on the fly from the
// position (no table in HBM); partial rotary, linear position scaling and Llama-3 frequency
// scaling are parameters.  Slots are bounds-checked: a bad slot sets the error word and is skipped.
//
// Replaces in the reference: apply_rope / apply_rope_with_offset (crates/runtime/src/models_v2/
// llama.rs:761-883), LayerKVCache::append (crates/runtime/src/kv_cache.rs:91-134) and the scalar /
// NEON apply_rope (crates/runtime/src/simd/arch/scalar.rs:112-153).
#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"

namespace ub {

__device__ __forceinline__ float rope_inv_freq(int i, const UbRopeArgs& a) {
  // i = pair index in [0, rd/2)
  float inv = exp2f(-(2.f * i / a.rotary_dim) * log2f(a.theta));
  if (a.l3_factor > 0.f) {
    const float two_pi = 6.283185307179586f;
    const float wavelen = two_pi / inv;
    const float low_wl = a.l3_orig_ctx / a.l3_low_freq_factor;
    const float high_wl = a.l3_orig_ctx / a.l3_high_freq_factor;
    if (wavelen > low_wl) {
      inv = inv / a.l3_factor;
    } else if (wavelen >= high_wl) {
      const float smooth = (a.l3_orig_ctx / wavelen - a.l3_low_freq_factor) /
                           (a.l3_high_freq_factor - a.l3_low_freq_factor);
      inv = (1.f - smooth) * inv / a.l3_factor + smooth * inv;
    }
  }
  return inv;
}

__global__ void __launch_bounds__(128) rope_kv_append_kernel(const UbRopeArgs a) {
  pdl_launch_dependents();
  pdl_wait();          // no global access before the previous kernel has completed
  extern __shared__ float sm[];  // [4 warps][D] staging (QK-norm / interleaved path), then [rotary_dim] cos | sin
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = a.D;
  float* hv = sm + warp * D;
  const int nheads = a.Hq + 2 * a.Hkv;
  __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(a.qkv) + (long long)t * nheads * D;
  const float pos = (float)a.positions[t] * a.pos_scale;
  const long long slot = a.slot_mapping != nullptr ? (long long)a.slot_mapping[t] : -1;
  bool slot_ok = slot >= 0;
  if (slot >= a.num_slots) {
    slot_ok = false;
    if (threadIdx.x == 0) set_err(a.err, ERR_BOUNDS, t);
  }
  const int half = a.rotary_dim / 2;
  // the angles depend on the token and the pair only: once per CTA, shared by all heads
  float* cs = sm + 4 * D;           // cos [half] then sin [half]
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf(pos * rope_inv_freq(i, a), &s, &c);
    cs[i] = c;
    cs[half + i] = s;
  }
  __syncthreads();
  const long long blk = slot_ok ? slot / a.block_size : 0, off = slot_ok ? slot % a.block_size : 0;
  const bool fast = !a.interleaved && a.q_norm_w == nullptr && a.k_norm_w == nullptr && (half % 2 == 0) && (D % 8 == 0);

  if (fast) {
    // Flat over (head, two adjacent pairs): consecutive threads touch consecutive 4-byte words of a head, and a thread's
    // loads of several items are issued before the first of them is used.
    constexpr int U = 4;
    const int ppl = half / 2;                       // items per rotated head
    const int nrot = a.Hq + a.Hkv;
    const int items = nrot * ppl;
    __nv_bfloat16* kc = reinterpret_cast<__nv_bfloat16*>(a.k_cache) + ((blk * a.Hkv) * a.block_size + off) * D;
    const long long khead = (long long)a.block_size * D;      // cache stride between KV heads of one block
    for (int it0 = threadIdx.x; it0 < items; it0 += U * blockDim.x) {
      uint32_t lo[U], hi[U];
      int hh[U], ii[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int it = it0 + u * blockDim.x;
        hh[u] = -1;
        if (it < items) {
          hh[u] = it / ppl;
          ii[u] = 2 * (it - hh[u] * ppl);
          const __nv_bfloat16* src = base + (long long)hh[u] * D;
          lo[u] = *reinterpret_cast<const uint32_t*>(src + ii[u]);
          hi[u] = *reinterpret_cast<const uint32_t*>(src + ii[u] + half);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (hh[u] < 0) continue;
        const int i = ii[u];
        const float c0 = cs[i], c1 = cs[i + 1], s0 = cs[half + i], s1 = cs[half + i + 1];
        const float x0 = bf16_lo(lo[u]), x1 = bf16_hi(lo[u]), y0 = bf16_lo(hi[u]), y1 = bf16_hi(hi[u]);
        const uint32_t olo = pack_bf16x2(x0 * c0 - y0 * s0, x1 * c1 - y1 * s1);
        const uint32_t ohi = pack_bf16x2(y0 * c0 + x0 * s0, y1 * c1 + x1 * s1);
        __nv_bfloat16* src = base + (long long)hh[u] * D;
        *reinterpret_cast<uint32_t*>(src + i) = olo;
        *reinterpret_cast<uint32_t*>(src + i + half) = ohi;
        if (hh[u] >= a.Hq && slot_ok) {
          __nv_bfloat16* kd = kc + (hh[u] - a.Hq) * khead;
          *reinterpret_cast<uint32_t*>(kd + i) = olo;
          *reinterpret_cast<uint32_t*>(kd + i + half) = ohi;
        }
      }
    }
    if (slot_ok) {
      // partial rotary: the unrotated tail of every K head goes to the cache as it is
      const int tail = (D - a.rotary_dim) / 2;
      for (int it = threadIdx.x; it < a.Hkv * tail; it += blockDim.x) {
        const int hk = it / tail, i = a.rotary_dim + 2 * (it - hk * tail);
        *reinterpret_cast<uint32_t*>(kc + hk * khead + i) =
            *reinterpret_cast<const uint32_t*>(base + (long long)(a.Hq + hk) * D + i);
      }
      // V heads: straight 16-byte copies
      __nv_bfloat16* vcd = reinterpret_cast<__nv_bfloat16*>(a.v_cache) + ((blk * a.Hkv) * a.block_size + off) * D;
      const int cpr = D / 8;
      for (int it = threadIdx.x; it < a.Hkv * cpr; it += blockDim.x) {
        const int hk = it / cpr, c = it - hk * cpr;
        reinterpret_cast<uint4*>(vcd + hk * khead)[c] =
            reinterpret_cast<const uint4*>(base + (long long)(a.Hq + a.Hkv + hk) * D)[c];
      }
    }
    return;
  }

  for (int h = warp; h < nheads; h += 4) {
    const bool is_q = h < a.Hq;
    const bool is_k = !is_q && h < a.Hq + a.Hkv;
    __nv_bfloat16* src = base + (long long)h * D;
    if (!is_q && !is_k) {
      // V head: straight copy into the cache
      if (slot_ok) {
        const int hk = h - a.Hq - a.Hkv;
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.v_cache) + ((blk * a.Hkv + hk) * a.block_size + off) * D;
        if (D % 8 == 0) {
          for (int i = lane; i < D / 8; i += 32) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
        } else {
          for (int i = lane; i < D; i += 32) dst[i] = src[i];
        }
      }
      continue;
    }
    __nv_bfloat16* kdst = nullptr;
    if (is_k && slot_ok) {
      const int hk = h - a.Hq;
      kdst = reinterpret_cast<__nv_bfloat16*>(a.k_cache) + ((blk * a.Hkv + hk) * a.block_size + off) * D;
    }
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
      const float v = __bfloat162float(src[i]);
      hv[i] = v;
      ss += v * v;
    }
    const __nv_bfloat16* nw = is_q ? reinterpret_cast<const __nv_bfloat16*>(a.q_norm_w)
                                   : reinterpret_cast<const __nv_bfloat16*>(a.k_norm_w);
    if (nw != nullptr) {
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / D + a.norm_eps);
      __syncwarp();
      for (int i = lane; i < D; i += 32) hv[i] = hv[i] * rstd * __bfloat162float(nw[i]);
    }
    __syncwarp();
    if (half > 0) {
      for (int i = lane; i < half; i += 32) {
        const float c = cs[i], s = cs[half + i];
        const int i0 = a.interleaved ? 2 * i : i;
        const int i1 = a.interleaved ? 2 * i + 1 : i + half;
        const float x0 = hv[i0], x1 = hv[i1];
        hv[i0] = x0 * c - x1 * s;
        hv[i1] = x1 * c + x0 * s;
      }
      __syncwarp();
    }
    for (int i = lane; i < D; i += 32) {
      const __nv_bfloat16 b = __float2bfloat16(hv[i]);
      src[i] = b;
      if (kdst != nullptr) kdst[i] = b;
    }
    __syncwarp();
  }
}

}  // namespace ub

extern "C" int ub_rope_kv_append(const UbRopeArgs* a, void* stream_v) {
  if (a->T <= 0) return 0;
  if (a->D > 512 || (a->rotary_dim & 1) || a->rotary_dim > a->D) return -2;
  ub::launch_pdl(ub::rope_kv_append_kernel, dim3(a->T), dim3(128), (4 * a->D + a->rotary_dim) * sizeof(float), (cudaStream_t)stream_v, *a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
