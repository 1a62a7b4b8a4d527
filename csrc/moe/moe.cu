// K7: MoE routing (router GEMV + top-k + softmax), expert sort with the token-tile table that drives the grouped
// GEMM, row gather and weighted combine.
//
// What the reference does (crates/runtime/src/model_core.rs:796-905, MoELayer::forward): a dense [T,E] router
// matmul, softmax, per-token top-k on the host, then a Python-style loop "for each token, for each selected expert,
// run that expert's MLP on one row".  Here the tokens are sorted by expert once and each expert's rows run as
// tensor-core tiles of one grouped GEMM launch (csrc/gemm/gemm_tn.cu, grouped mode).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"

namespace ub {

constexpr int MOE_MAX_E = 256;
constexpr int MOE_MAX_K = 16;

// One CTA of 128 threads per token: logits (from x and the router matrix, or given), top-k, weights.
__global__ void __launch_bounds__(128) moe_route_kernel(const UbMoeRouteArgs a) {
  __shared__ float logit[MOE_MAX_E];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int E = a.E, K = a.K;
  if (a.router_w != nullptr) {
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x) + (long long)t * a.H;
    const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(a.router_w);
    for (int e = warp; e < E; e += 4) {
      const __nv_bfloat16* we = w + (long long)e * a.H;
      float acc = 0.f;
      for (int h = lane * 8; h < a.H; h += 256) {
        const uint4 xv = *reinterpret_cast<const uint4*>(x + h);
        const uint4 wv = __ldg(reinterpret_cast<const uint4*>(we + h));
        const uint32_t* xs = reinterpret_cast<const uint32_t*>(&xv);
        const uint32_t* ws = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc += bf16_lo(xs[j]) * bf16_lo(ws[j]) + bf16_hi(xs[j]) * bf16_hi(ws[j]);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      // the reference model keeps router logits in the activation dtype: round like a bf16 linear layer would
      if (lane == 0) logit[e] = a.round_logits_bf16 ? __bfloat162float(__float2bfloat16(acc)) : acc;
    }
  } else {
    for (int e = threadIdx.x; e < E; e += 128)
      logit[e] = a.logits_f32 ? reinterpret_cast<const float*>(a.logits)[(long long)t * E + e]
                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.logits)[(long long)t * E + e]);
  }
  __syncthreads();
  if (warp != 0) return;
  // Softmax statistics over all experts (used when the weights are not renormalised over the selection).
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, logit[e]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float den = 0.f;
  for (int e = lane; e < E; e += 32) den += __expf(logit[e] - mx);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
  uint32_t taken = 0;  // bit j: expert lane + 32*j already selected
  float sel_l[MOE_MAX_K];
  int sel_e[MOE_MAX_K];
  for (int k = 0; k < K; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane, j = 0; e < E; e += 32, ++j) {
      if (taken >> j & 1u) continue;
      const float v = logit[e];
      if (v > best || (v == best && e < bi)) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (bi < E && (bi & 31) == lane) taken |= 1u << (bi >> 5);
    sel_l[k] = best;
    sel_e[k] = bi < E ? bi : 0;
  }
  if (lane == 0) {
    float s = 0.f;
    for (int k = 0; k < K; ++k) { sel_l[k] = __expf(sel_l[k] - mx); s += sel_l[k]; }
    const float inv = a.norm_topk ? 1.f / s : 1.f / den;
    for (int k = 0; k < K; ++k) {
      a.topk_ids[(long long)t * K + k] = sel_e[k];
      a.topk_w[(long long)t * K + k] = sel_l[k] * inv * a.weight_scale;
    }
  }
}

// One CTA: counts, exclusive offsets, slot assignment and the token-tile table of the grouped GEMM.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const UbMoeRouteArgs a) {
  __shared__ int cnt[MOE_MAX_E], off[MOE_MAX_E + 1], cur[MOE_MAX_E];
  const int E = a.num_local_experts > 0 ? a.num_local_experts : a.E, n = a.T * a.K;
  for (int e = threadIdx.x; e < E; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
  __syncthreads();
  // Expert parallelism: only experts [expert_lo, expert_lo + E) live on this rank; the rest get no slot.
  const int lo = a.expert_lo;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = a.topk_ids[i] - lo;
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0, tile = 0;
    int4* tiles = reinterpret_cast<int4*>(a.tiles);
    for (int e = 0; e < E; ++e) {
      off[e] = acc;
      if (tiles != nullptr) {
        for (int r = 0; r < cnt[e] && tile < a.max_tiles; r += a.tile_tokens, ++tile)
          tiles[tile] = make_int4(e, acc + r, acc + cnt[e], 0);
      }
      acc += cnt[e];
    }
    off[E] = acc;
    if (tiles != nullptr)
      for (; tile < a.max_tiles; ++tile) tiles[tile] = make_int4(-1, 0, 0, 0);
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    a.expert_offsets[e] = off[e];
    if (e < E) a.expert_counts[e] = cnt[e];
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = a.topk_ids[i] - lo;
    if (e < 0 || e >= E) { a.row_slot[i] = -1; continue; }
    const int slot = off[e] + atomicAdd(&cur[e], 1);
    a.sorted_rows[slot] = i;
    a.row_slot[i] = slot;
  }
  for (int i = off[E] + threadIdx.x; i < n; i += blockDim.x) a.sorted_rows[i] = -1;   // unused tail
}

// out[slot, :] = x[sorted_rows[slot] / K, :]
__global__ void __launch_bounds__(256) moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted_rows,
                                                         __nv_bfloat16* __restrict__ out, int rows, int K, int H) {
  const int vec = H / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)rows * vec;
       i += (long long)gridDim.x * blockDim.x) {
    const int slot = int(i / vec), c = int(i % vec);
    const int sr = sorted_rows[slot];
    if (sr < 0) continue;                      // slot not used on this rank
    const int src = sr / K;
    reinterpret_cast<uint4*>(out + (long long)slot * H)[c] = __ldg(reinterpret_cast<const uint4*>(x + (long long)src * H) + c);
  }
}

// out[t, :] = residual[t, :] + sum_k w[t,k] * y[row_slot[t*K+k], :]
struct CombinePush {
  int world, rank, rows_per_rank;            // world == 0: plain store to `out`
  __nv_bfloat16* peer_out[UB_MAX_RANKS];     // each: [world][rows_per_rank][H] receive slots
  uint32_t* peer_flag[UB_MAX_RANKS];
  uint32_t* local_count;                     // local arrival counter of the CTAs (see publish_to_peers)
};

__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ row_slot,
                                                          const float* __restrict__ topk_w, const __nv_bfloat16* __restrict__ residual,
                                                          __nv_bfloat16* __restrict__ out, int T, int K, int H, const CombinePush push) {
  const int vec = H / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)T * vec;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = int(i / vec), c = int(i % vec);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (residual != nullptr) {
      const uint4 r = __ldg(reinterpret_cast<const uint4*>(residual + (long long)t * H) + c);
      const uint32_t* rs = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[2 * j] = bf16_lo(rs[j]); acc[2 * j + 1] = bf16_hi(rs[j]); }
    }
    for (int k = 0; k < K; ++k) {
      const float w = topk_w[(long long)t * K + k];
      const int slot = row_slot[(long long)t * K + k];
      if (slot < 0) continue;                  // expert lives on another rank
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(y + (long long)slot * H) + c);
      const uint32_t* vs = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[2 * j] += w * bf16_lo(vs[j]); acc[2 * j + 1] += w * bf16_hi(vs[j]); }
    }
    __nv_bfloat16* dst = out + (long long)t * H;
    if (push.world > 0 && push.peer_out[0] != nullptr) {
      // F6: the partial row goes straight into the receive slot of the rank that owns token t
      // (with null peer pointers it stays in `out`, this rank's own partial buffer, which the owners read summed
      // through the multicast address)
      int owner = t / push.rows_per_rank;
      if (owner >= push.world) owner = push.world - 1;
      dst = push.peer_out[owner] + ((long long)push.rank * push.rows_per_rank + (t - owner * push.rows_per_rank)) * H;
    }
    reinterpret_cast<uint4*>(dst)[c] =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
  if (push.world > 0) {
    // publish: the CTAs arrive on the local counter; the last one bumps every peer's counter once
    __syncthreads();
    if (threadIdx.x == 0) publish_to_peers(push.local_count, gridDim.x, push.peer_flag, push.world);
  }
}


// ------------------------------------------------------------------------------------------------------------
// F5 / F6: sparse expert-parallel dispatch and combine over peer memory.
//
// Every rank owns R = T / world consecutive token rows (the rows its norm kernel has just produced), routes THEM
// (1 / world of the router work), and sends each (token, choice) pair's row only to the rank that holds the chosen
// expert: T * K / world rows leave a rank instead of (world - 1) * T / world for the all-gather, and T * K / world
// come back instead of T.  No count exchange precedes the rows: rank `src` owns the fixed region
// [src * cap, (src + 1) * cap), cap = R * K, of every destination's receive buffer, fills it front to back in expert
// order, and writes how many rows of each local expert it sent into a small header.  One arrival per source tells
// the destination that region and header are complete (publish_to_peers); the destination's build kernel turns the
// world x experts_local count table into expert-contiguous row order, the tile table of the grouped GEMM and the
// return address of every row.  The combine scales each expert output by its routing weight and stores it into
// slot [choice k][row] of the token owner's combine area, one writer per (token, k), so the owner's norm kernel sums
// K slots in a fixed order.  Replaces the host loop over tokens and experts at
// crates/runtime/src/models_v2/mixtral.rs:639-662 / model_core.rs:796-905.
// ------------------------------------------------------------------------------------------------------------

// One CTA: pairs per global expert, and each pair's position inside its destination's region.
__global__ void __launch_bounds__(1024) moe_dispatch_sort_kernel(const UbMoeDispatchArgs a) {
  __shared__ int cnt[MOE_MAX_E], off[MOE_MAX_E], cur[MOE_MAX_E];
  const int n = a.R * a.K;
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = a.topk_ids[i];
    if (e >= 0 && e < a.E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x < a.world) {
    // experts [d * experts_local, (d + 1) * experts_local) live on rank d: offsets restart at every destination
    const int d = threadIdx.x;
    int acc = 0;
    for (int el = 0; el < a.experts_local; ++el) {
      off[d * a.experts_local + el] = acc;
      acc += cnt[d * a.experts_local + el];
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) a.send_counts[e] = cnt[e];
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = a.topk_ids[i];
    a.send_slot[i] = (e >= 0 && e < a.E) ? off[e] + atomicAdd(&cur[e], 1) : -1;
  }
}

// Rows, their metadata and the count header go to the destinations; the last CTA signals every rank once.
__global__ void __launch_bounds__(256) moe_dispatch_push_kernel(const UbMoeDispatchArgs a) {
  const int vec = a.H / 8;
  const long long work = (long long)a.R * a.K * vec;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < work; i += (long long)gridDim.x * blockDim.x) {
    const int pair = int(i / vec), c = int(i % vec);
    const int slot = a.send_slot[pair];
    if (slot < 0 || slot >= a.cap) continue;
    const int e = a.topk_ids[pair];
    const int d = e / a.experts_local;
    const long long row = (long long)a.rank * a.cap + slot;
    const uint4 v = *reinterpret_cast<const uint4*>(x + (long long)(pair / a.K) * a.H + c * 8);
    reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.peer_rows[d]) + row * a.H)[c] = v;
    if (c == 0) {
      // global pair id (token * K + k), local expert, routing weight
      const int gp = (a.rank * a.R + pair / a.K) * a.K + pair % a.K;
      reinterpret_cast<int4*>(a.peer_meta[d])[row] = make_int4(gp, e - d * a.experts_local, __float_as_int(a.topk_w[pair]), 0);
    }
  }
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
      const int d = e / a.experts_local;
      a.peer_counts[d][a.rank * a.experts_local + (e - d * a.experts_local)] = a.send_counts[e];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) publish_to_peers(a.local_count, gridDim.x, a.peer_flag, a.world);
}

// One CTA on the receiving rank: wait (bounded) for the arrival of every source, then expert-contiguous order.
__global__ void __launch_bounds__(1024) moe_recv_build_kernel(const UbMoeRecvArgs a) {
  __shared__ int cnt[MOE_MAX_E];     // [world][experts_local]; world * experts_local = E <= MOE_MAX_E (host check)
  __shared__ int base[MOE_MAX_E];    // first compacted slot of (source, expert)
  __shared__ int srcoff[MOE_MAX_E];  // first row of the expert inside the source's region
  __shared__ int nsrc[UB_MAX_RANKS];
  __shared__ int total_s;
  const int W = a.world, EL = a.experts_local;
  if (threadIdx.x == 0) {
    const uint32_t round = *a.round + 1;                // exchanges are counted; the flag is never reset
    const uint32_t want = round * (uint32_t)W;
    const uint64_t t0 = wait_ticks();
    uint32_t it = 0, v;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.flag) : "memory");
      if (int32_t(v - want) >= 0) break;
      if ((++it & 31u) == 0 && wait_expired(t0, a.err)) {
        set_err(a.err, ERR_FLAG_TIMEOUT, 5000);
        break;
      }
    }
    *a.round = round;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < W * EL; i += blockDim.x) {
    int c = __ldcg(a.counts + i);                       // written by peers: L2 only
    if (c < 0 || c > a.cap) { set_err(a.err, ERR_BOUNDS, 5100 + i); c = 0; }
    cnt[i] = c;
  }
  __syncthreads();
  if (threadIdx.x < W) {
    int acc = 0;
    for (int el = 0; el < EL; ++el) { srcoff[threadIdx.x * EL + el] = acc; acc += cnt[threadIdx.x * EL + el]; }
    if (acc > a.cap) { set_err(a.err, ERR_BOUNDS, 5200 + threadIdx.x); acc = 0; }
    nsrc[threadIdx.x] = acc;
  }
  if (threadIdx.x == 0) {
    int acc = 0, tile = 0;
    int4* tiles = reinterpret_cast<int4*>(a.tiles);
    for (int el = 0; el < EL; ++el) {
      const int start = acc;
      for (int s = 0; s < W; ++s) { base[s * EL + el] = acc; acc += cnt[s * EL + el]; }
      a.expert_offsets[el] = start;
      a.expert_counts[el] = acc - start;
      for (int r = start; r < acc && tile < a.max_tiles; r += a.tile_tokens, ++tile) tiles[tile] = make_int4(el, r, acc, 0);
    }
    a.expert_offsets[EL] = acc;
    for (; tile < a.max_tiles; ++tile) tiles[tile] = make_int4(-1, 0, 0, 0);
    total_s = acc;
  }
  __syncthreads();
  const int4* meta = reinterpret_cast<const int4*>(a.meta);
  int4* slot_meta = reinterpret_cast<int4*>(a.slot_meta);
  for (int i = threadIdx.x; i < W * a.cap; i += blockDim.x) {
    const int s = i / a.cap, j = i - s * a.cap;
    if (j >= nsrc[s]) continue;
    const int4 m = __ldcg(meta + i);
    const int el = m.y;
    if (el < 0 || el >= EL || j < srcoff[s * EL + el] || j - srcoff[s * EL + el] >= cnt[s * EL + el]) {
      set_err(a.err, ERR_BOUNDS, 5300 + s);
      continue;
    }
    const int slot = base[s * EL + el] + (j - srcoff[s * EL + el]);
    a.sorted_rows[slot] = i;
    slot_meta[slot] = make_int4(m.x, s, m.z, 0);
  }
  for (int i = total_s + threadIdx.x; i < W * a.cap; i += blockDim.x) a.sorted_rows[i] = -1;
}

// Expert outputs go home: y[slot] * weight -> slot [k][token row] of the owner's combine area.
__global__ void __launch_bounds__(256) moe_combine_push_kernel(const UbMoeReturnArgs a) {
  const int vec = a.H / 8;
  const int total = a.expert_offsets[a.experts_local];
  const __nv_bfloat16* y = reinterpret_cast<const __nv_bfloat16*>(a.y);
  const int4* slot_meta = reinterpret_cast<const int4*>(a.slot_meta);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)total * vec;
       i += (long long)gridDim.x * blockDim.x) {
    const int slot = int(i / vec), c = int(i % vec);
    const int4 m = slot_meta[slot];
    const int owner = m.y, tok = m.x / a.K, k = m.x - tok * a.K;
    const int row = tok - owner * a.R;
    if (owner < 0 || owner >= a.world || row < 0 || row >= a.R) {
      if (c == 0) set_err(a.err, ERR_BOUNDS, 5400);
      continue;
    }
    const float w = __int_as_float(m.z);
    const uint4 v = *reinterpret_cast<const uint4*>(y + (long long)slot * a.H + c * 8);
    const uint32_t* vs = reinterpret_cast<const uint32_t*>(&v);
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = pack_bf16x2(w * bf16_lo(vs[j]), w * bf16_hi(vs[j]));
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.peer_comb[owner]) + ((long long)k * a.R + row) * a.H;
    reinterpret_cast<uint4*>(dst)[c] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  __syncthreads();
  if (threadIdx.x == 0) publish_to_peers(a.local_count, gridDim.x, a.peer_flag, a.world);
}

}  // namespace ub

extern "C" int ub_moe_route(const UbMoeRouteArgs* a, void* stream_v) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  if (a->T <= 0) return 0;
  if (a->E <= 0 || a->E > ub::MOE_MAX_E || a->K <= 0 || a->K > ub::MOE_MAX_K || a->K > a->E) return -2;
  if (a->router_w != nullptr && (a->H % 8 != 0 || a->x == nullptr)) return -3;
  if (a->tiles != nullptr && (a->tile_tokens <= 0 || a->max_tiles <= 0)) return -4;
  UbMoeRouteArgs b = *a;
  if (b.weight_scale == 0.f) b.weight_scale = 1.f;
  ub::moe_route_kernel<<<a->T, 128, 0, st>>>(b);
  ub::moe_sort_kernel<<<1, 1024, 0, st>>>(b);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int ub_moe_gather(const void* x, const int* sorted_rows, void* out, int rows, int K, int H, void* stream_v) {
  if (rows <= 0) return 0;
  if (H % 8 != 0) return -2;
  const long long work = (long long)rows * (H / 8);
  int blocks = int((work + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  ub::moe_gather_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), sorted_rows, reinterpret_cast<__nv_bfloat16*>(out), rows, K, H);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

static int combine_blocks(int T, int H) {
  const long long work = (long long)T * (H / 8);
  int blocks = int((work + 255) / 256);
  return blocks > 148 * 4 ? 148 * 4 : blocks;
}

extern "C" int ub_moe_combine_num_ctas(int T, int H) { return T <= 0 ? 0 : combine_blocks(T, H); }

extern "C" int ub_moe_combine(const void* y, const int* row_slot, const float* topk_w, const void* residual, void* out, int T,
                              int K, int H, void* stream_v) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return -2;
  ub::CombinePush push = {};
  ub::moe_combine_kernel<<<combine_blocks(T, H), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const __nv_bfloat16*>(y), row_slot, topk_w, reinterpret_cast<const __nv_bfloat16*>(residual),
      reinterpret_cast<__nv_bfloat16*>(out), T, K, H, push);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// F6: combine + reduce-scatter.  Every CTA (ub_moe_combine_num_ctas of them) signals every peer once.
extern "C" int ub_moe_combine_rs(const void* y, const int* row_slot, const float* topk_w, int T, int K, int H, int world, int rank,
                                 int rows_per_rank, void* const* peer_out, uint32_t* const* peer_flag, uint32_t* local_count,
                                 void* local_out, void* stream_v) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || world <= 0 || world > UB_MAX_RANKS || rows_per_rank <= 0 || local_count == nullptr) return -2;
  if (peer_out[0] == nullptr && local_out == nullptr) return -3;
  ub::CombinePush push = {};
  push.world = world; push.rank = rank; push.rows_per_rank = rows_per_rank;
  push.local_count = local_count;
  for (int i = 0; i < world; ++i) {
    push.peer_out[i] = reinterpret_cast<__nv_bfloat16*>(peer_out[i]);
    push.peer_flag[i] = peer_flag[i];
  }
  ub::moe_combine_kernel<<<combine_blocks(T, H), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      reinterpret_cast<const __nv_bfloat16*>(y), row_slot, topk_w, nullptr, reinterpret_cast<__nv_bfloat16*>(local_out), T, K, H,
      push);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// F5: route-local dispatch.  Two launches (sort, push); grid of the push as reported by ub_moe_dispatch_num_ctas.
static int dispatch_blocks(int R, int K, int H) {
  const long long work = (long long)R * K * (H / 8);
  int blocks = int((work + 255) / 256);
  return blocks > 148 * 4 ? 148 * 4 : (blocks < 1 ? 1 : blocks);
}
extern "C" int ub_moe_dispatch(const UbMoeDispatchArgs* a, void* stream_v) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  if (a->R <= 0) return 0;
  if (a->H % 8 != 0 || a->E <= 0 || a->E > ub::MOE_MAX_E || a->world <= 0 || a->world > UB_MAX_RANKS ||
      a->experts_local * a->world != a->E || a->cap < a->R * a->K || a->local_count == nullptr)
    return -2;
  ub::moe_dispatch_sort_kernel<<<1, 1024, 0, st>>>(*a);
  ub::moe_dispatch_push_kernel<<<dispatch_blocks(a->R, a->K, a->H), 256, 0, st>>>(*a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int ub_moe_recv_build(const UbMoeRecvArgs* a, void* stream_v) {
  if (a->world <= 0 || a->world > UB_MAX_RANKS || a->experts_local <= 0 ||
      a->world * a->experts_local > ub::MOE_MAX_E || a->tile_tokens <= 0 || a->max_tiles <= 0 ||
      a->round == nullptr || a->flag == nullptr)
    return -2;
  ub::moe_recv_build_kernel<<<1, 1024, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// F6: sparse combine.  max_slots bounds the grid (the true row count is read on the device).
extern "C" int ub_moe_combine_push(const UbMoeReturnArgs* a, int max_slots, void* stream_v) {
  if (a->H % 8 != 0 || a->world <= 0 || a->world > UB_MAX_RANKS || a->local_count == nullptr || a->R <= 0 || a->K <= 0) return -2;
  ub::moe_combine_push_kernel<<<dispatch_blocks(max_slots, 1, a->H), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
