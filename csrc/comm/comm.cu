// C1 helpers: small-message one-shot all-reduce over NVSwitch peer memory (F1s).
//
// Every rank stores its vector into slot [parity][rank] of every peer's symmetric receive buffer with plain
// 16-byte peer stores, then tells the peers, then waits (bounded) until all `world` ranks' data for this exchange
// has arrived and sums the slots in rank order (bitwise identical on every rank).  Latency-optimal for messages up
// to a few hundred KB (each rank sends (world-1) * n bytes); larger tensors go through the GEMM-fused
// reduce-scatter / all-gather path.
//
// The vector is cut into one chunk per CTA (the same cut on every rank, the grid depends on n only); CTA c pushes
// chunk c, bumps counter [c] on every peer and waits for its own counter [c] to show `world` more arrivals, so a
// chunk is reduced as soon as ITS pieces are there and the remote atomics spread over up to 64 addresses.
// Counters are monotonic.  A launch uses as many CTAs as its size asks for, so every CTA keeps its own count of the
// exchanges it took part in (a local word per CTA) and expects `world` arrivals more per exchange on ITS counter; the
// number of the exchange itself (a local word that the last CTA to finish advances, so the launch can sit in a CUDA
// graph) only selects the slot.  Slots alternate by the parity of that number e: a fast rank
// may start exchange e + 1 while a slow one still sums exchange e, but it cannot reach e + 2 before the slow rank
// has pushed e + 1, which that rank does only after it has finished reading e.
// The reference has no collective of any kind.
#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"

namespace ub {

__global__ void __launch_bounds__(256) allreduce_oneshot_kernel(const UbAllReduceArgs a) {
  const long long nv = a.n / 8;  // n is a multiple of 8 (checked on the host)
  const long long per = (nv + gridDim.x - 1) / gridDim.x;
  const long long c0 = (long long)blockIdx.x * per, c1 = min(nv, c0 + per);
  __shared__ uint32_t round_s;
  __shared__ int failed;
  if (threadIdx.x == 0) {
    round_s = *a.round + 1;       // the word is advanced by the last CTA of this launch, after everyone has read it
    failed = 0;
  }
  __syncthreads();
  const uint32_t round = round_s;
  const long long slot = (long long)(round & 1u) * a.world * a.max_n;
  const __nv_bfloat16* in = reinterpret_cast<const __nv_bfloat16*>(a.in);
  // 1. push this CTA's chunk into every rank's slot [parity][rank]
  for (long long c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
    const uint4 v = *reinterpret_cast<const uint4*>(in + c * 8);
    for (int r = 0; r < a.world; ++r) {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.peer_slots[r]) + slot + (long long)a.rank * a.max_n + c * 8;
      *reinterpret_cast<uint4*>(dst) = v;
    }
  }
  __threadfence_system();       // every thread's own peer stores are performed before the CTA meets
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    for (int r = 0; r < a.world; ++r)
      asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(a.peer_flags[r] + blockIdx.x), "r"(1u) : "memory");
    // 2. wait for the same chunk of all ranks: `world` arrivals more than after this CTA's previous exchange
    const uint32_t mine = a.cta_rounds[blockIdx.x] + 1;
    a.cta_rounds[blockIdx.x] = mine;
    const uint32_t want = mine * (uint32_t)a.world;
    const uint64_t t0 = wait_ticks();
    uint32_t it = 0, v;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.my_flags + blockIdx.x) : "memory");
      if (int32_t(v - want) >= 0) break;
      if ((++it & 31u) == 0 && wait_expired(t0, a.err)) {
        set_err(a.err, ERR_FLAG_TIMEOUT, 3000 + blockIdx.x);
        failed = 1;
        break;
      }
    }
  }
  __syncthreads();
  // 3. reduce in rank order
  const __nv_bfloat16* slots = reinterpret_cast<const __nv_bfloat16*>(a.my_slots) + slot;
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.out);
  for (long long c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < a.world; ++r) {
      const uint4 v = ld_sys_u128(slots + (long long)r * a.max_n + c * 8);     // peers wrote it: read at the point of coherence
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) { f[2 * e] += bf16_lo(w[e]); f[2 * e + 1] += bf16_hi(w[e]); }
    }
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = pack_bf16x2(f[2 * e], f[2 * e + 1]);
    *reinterpret_cast<uint4*>(out + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  // 4. the last CTA to get here advances the exchange number for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t old = atomicAdd(a.done_count, 1u);
    if (old + 1 == gridDim.x) {
      *a.done_count = 0u;
      *a.round = round;
    }
  }
}

}  // namespace ub

extern "C" int ub_allreduce_oneshot_ctas(long long n) {
  // The grid must be co-resident (CTAs of different ranks wait on one another): stay well under one wave.
  long long g = (n / 8 + 1023) / 1024;       // at least 16 KB per CTA
  if (g > UB_AR_MAX_CTAS) g = UB_AR_MAX_CTAS;
  return g < 1 ? 1 : (int)g;
}

extern "C" int ub_allreduce_oneshot(const UbAllReduceArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  if (a->n % 8 != 0 || a->world < 1 || a->world > UB_MAX_RANKS || a->round == nullptr || a->done_count == nullptr ||
      a->cta_rounds == nullptr || a->max_n < a->n || a->max_n % 8 != 0)
    return -2;
  ub::allreduce_oneshot_kernel<<<(unsigned)ub_allreduce_oneshot_ctas(a->n), 256, 0, (cudaStream_t)stream_v>>>(*a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// ----------------------------------------------------------------------------------------------
// F4s: one-shot all-gather of (value, id) pairs, the exchange of vocabulary-parallel top-k / top-p sampling.  Every
// rank holds, per sampled row, the k best (scaled logit, global id) pairs of its vocabulary shard; after the exchange
// every rank has all world * k pairs of every row, in rank order, and draws the same token from them.  The rows are cut
// into one chunk per CTA (the same cut on every rank); CTA c stores its chunk into slot [parity][row][rank] of every
// rank, bumps counter [c] on every rank, waits (bounded) for `world` arrivals on its own counter [c] and copies the
// chunk's gathered pairs into the caller's buffers.  Parity and exchange number as in the all-reduce above.
// ----------------------------------------------------------------------------------------------
namespace ub {

__global__ void __launch_bounds__(256) pair_gather_oneshot_kernel(const UbPairGatherArgs a) {
  const int per = (a.rows + gridDim.x - 1) / gridDim.x;
  const int r0 = blockIdx.x * per, r1 = min(a.rows, r0 + per);
  __shared__ uint32_t round_s;
  if (threadIdx.x == 0) round_s = *a.round + 1;
  __syncthreads();
  const uint32_t round = round_s;
  const long long slot = (long long)(round & 1u) * a.cap * a.world;
  const int k = a.k, W = a.world;
  // 1. this CTA's rows into slot [parity][row][rank][0..k) of every rank
  for (long long i = (long long)r0 * k + threadIdx.x; i < (long long)r1 * k; i += blockDim.x) {
    const long long row = i / k;
    const int j = int(i - row * k);
    const float v = a.vals[i];
    const int id = a.ids[i];
    const long long dst = slot + (row * W + a.rank) * k + j;
    for (int r = 0; r < W; ++r) {
      reinterpret_cast<float*>(a.peer_vals[r])[dst] = v;
      reinterpret_cast<int*>(a.peer_ids[r])[dst] = id;
    }
  }
  __threadfence_system();       // every thread's own peer stores are performed before the CTA meets ...
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");     // ... and before the arrival that thread 0 sends for all of them
    for (int r = 0; r < W; ++r)
      asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(a.peer_flags[r] + blockIdx.x), "r"(1u) : "memory");
    const uint32_t mine = a.cta_rounds[blockIdx.x] + 1;       // exchanges this CTA index has taken part in (grids vary)
    a.cta_rounds[blockIdx.x] = mine;
    const uint32_t want = mine * (uint32_t)W;
    const uint64_t t0 = wait_ticks();
    uint32_t it = 0, v;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.my_flags + blockIdx.x) : "memory");
      if (int32_t(v - want) >= 0) break;
      if ((++it & 31u) == 0 && wait_expired(t0, a.err)) {
        set_err(a.err, ERR_FLAG_TIMEOUT, 6000 + blockIdx.x);
        break;
      }
    }
  }
  __syncthreads();
  // 2. the gathered pairs of this CTA's rows -> [row][world * k]
  for (long long i = (long long)r0 * W * k + threadIdx.x; i < (long long)r1 * W * k; i += blockDim.x) {
    a.out_vals[i] = ld_sys_f32(a.my_vals + slot + i);      // peers wrote it: read at the point of coherence
    a.out_ids[i] = (int)ld_sys_u32(a.my_ids + slot + i);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t old = atomicAdd(a.done_count, 1u);
    if (old + 1 == gridDim.x) {
      *a.done_count = 0u;
      *a.round = round;
    }
  }
}

}  // namespace ub

extern "C" int ub_pair_gather_oneshot(const UbPairGatherArgs* a, void* stream_v) {
  if (a->rows <= 0) return 0;
  if (a->k <= 0 || a->world < 1 || a->world > UB_MAX_RANKS || (long long)a->rows * a->k > a->cap || a->round == nullptr ||
      a->done_count == nullptr || a->cta_rounds == nullptr)
    return -2;
  // The grid must be co-resident (CTAs of different ranks wait on one another): at most UB_AR_MAX_CTAS.
  int g = (int)(((long long)a->rows * a->k + 4095) / 4096);
  if (g > UB_AR_MAX_CTAS) g = UB_AR_MAX_CTAS;
  if (g > a->rows) g = a->rows;
  if (g < 1) g = 1;
  ub::pair_gather_oneshot_kernel<<<g, 256, 0, (cudaStream_t)stream_v>>>(*a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// ----------------------------------------------------------------------------------------------
// F4: vocabulary-parallel greedy merge.  Every rank holds, per sampled row, the best (value, id) of its
// vocabulary shard.  One single-block kernel pushes the pairs into every peer's slot [parity][rank],
// bumps the peers' counters, waits (bounded) until all `world` ranks have arrived for this exchange and
// picks the global winner (highest value, lowest id on ties) -- the same answer on every rank.
// The exchange number lives in a device word that the kernel itself increments, so the launch can sit in
// a CUDA graph; slots alternate by its parity because a fast rank may start exchange n+1 while a slow
// one still reads exchange n.
// ----------------------------------------------------------------------------------------------
namespace ub {

__global__ void __launch_bounds__(256) tp_argmax_merge_kernel(const UbArgmaxMergeArgs a) {
  __shared__ uint32_t round_s;
  __shared__ int failed;
  if (threadIdx.x == 0) {
    round_s = *a.round + 1;
    *a.round = round_s;
    failed = 0;
  }
  __syncthreads();
  const uint32_t round = round_s;
  const int par = round & 1u;
  const long long slot = ((long long)par * a.world + a.rank) * a.max_rows;
  for (int i = threadIdx.x; i < a.rows; i += blockDim.x) {
    const float v = a.vals[i];
    const int id = a.ids[i];
    for (int r = 0; r < a.world; ++r) {
      reinterpret_cast<float*>(a.peer_vals[r])[slot + i] = v;
      reinterpret_cast<int*>(a.peer_ids[r])[slot + i] = id;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < a.world)
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(a.peer_flags[threadIdx.x]), "r"(1u) : "memory");
  if (threadIdx.x == 0) {
    const uint32_t want = round * (uint32_t)a.world;
    const uint64_t t0 = wait_ticks();
    uint32_t it = 0, v;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.my_flag) : "memory");
      if (int32_t(v - want) >= 0) break;
      if ((++it & 31u) == 0 && wait_expired(t0, a.err)) {
        set_err(a.err, ERR_FLAG_TIMEOUT, 4000);
        failed = 1;
        break;
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < a.rows; i += blockDim.x) {
    float bv = -3.4e38f;
    int bi = 0x7fffffff;
    for (int r = 0; r < a.world; ++r) {
      const long long s = ((long long)par * a.world + r) * a.max_rows + i;
      const float v = ld_sys_f32(a.my_vals + s);      // peers wrote it: read at the point of coherence
      const int id = (int)ld_sys_u32(a.my_ids + s);
      if (v > bv || (v == bv && id < bi)) { bv = v; bi = id; }
    }
    a.out_ids[i] = bi;
  }
}

}  // namespace ub

extern "C" int ub_tp_argmax_merge(const UbArgmaxMergeArgs* a, void* stream_v) {
  if (a->rows <= 0) return 0;
  if (a->rows > a->max_rows || a->world < 1 || a->world > UB_MAX_RANKS) return -2;
  ub::tp_argmax_merge_kernel<<<1, 256, 0, (cudaStream_t)stream_v>>>(*a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
