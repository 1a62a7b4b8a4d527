// Thin inline-PTX wrappers for the Blackwell (sm_100a) execution model:
// mbarrier, TMA (cp.async.bulk.tensor, never with cluster multicast), tcgen05
// (TMEM alloc / mma / commit / ld) and the error-word convention shared by all
// kernels in this library.
//
// Error convention: every wait in device code is bounded.  When a wait gives up
// it records a code in a caller-provided global `int* err` (first writer wins)
// and the kernel carries on to its normal exit so that TMEM is released and the
// context stays usable.  Results of such a launch are garbage; the host checks
// the word after the step.
#pragma once
#include "launch.cuh"
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ub {

enum ErrCode : int {
  ERR_NONE = 0,
  ERR_MBAR_TIMEOUT = 1,   // an mbarrier phase never completed
  ERR_FLAG_TIMEOUT = 2,   // a peer / producer flag never reached its value
  ERR_BOUNDS = 3,         // an index (block table entry, slot, token id) was out of range
  ERR_BAD_ARG = 4,
};

__device__ __forceinline__ void set_err(int* err, int code, int detail = 0) {
  if (err != nullptr) {
    if (atomicCAS(err, 0, code) == 0) err[1] = detail;
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Time base of the bounded waits: SM cycles / 2 ("ticks").  The SM cycle counter is read instead of %globaltimer:
// the global timer is a slow off-SM read, and a wait that polls it (even once per call) costs more than the event it
// waits for.  Only differences inside one thread are used.  A tick is 1.0 ns at 2.0 GHz and 1.5 ns at 1.3 GHz, so a
// limit stated in ticks is a time between those bounds -- all a give-up deadline needs.
__device__ __forceinline__ uint64_t wait_ticks() {
  return (uint64_t)clock64() >> 1;
}

// Loads of data that a PEER GPU has written into this GPU's memory, issued after the arrival counter has been
// acquired: relaxed at system scope, i.e. served from the point of coherence.  (A weak ld.global.cg after another
// thread's acquire returned stale zeros from a line that had been cached before the peer's stores landed.)
__device__ __forceinline__ uint32_t ld_sys_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_sys_f32(const void* p) { return __uint_as_float(ld_sys_u32(p)); }
__device__ __forceinline__ uint4 ld_sys_u128(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  `abort_flag` is a CTA-shared int: once any wait of this CTA has
// timed out, later waits give up at once so a broken launch drains quickly.
#ifndef UB_WAIT_TICKS
#define UB_WAIT_TICKS 1500000000ull  // 1.5 s at 2 GHz, 2.3 s at 1.3 GHz
#endif
// True when a bounded wait that started at t0 should give up: its deadline has passed, or an error is already
// recorded in the device error word (by an earlier kernel of the step or another CTA) -- then nothing this launch
// produces will be used, and sitting out one more deadline per wait would only make a broken step take minutes.
__device__ __forceinline__ bool wait_expired(uint64_t t0, const int* err) {
  if (err != nullptr && *reinterpret_cast<const volatile int*>(err) != 0) return true;
  return wait_ticks() - t0 > UB_WAIT_TICKS;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err,
                                          int detail) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  const uint64_t t0 = wait_ticks();
  uint32_t it = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 63u) == 0) {
      if (*abort_flag) return false;
      if (wait_expired(t0, err)) break;
    }
  }
  *abort_flag = 1;
  set_err(err, ERR_MBAR_TIMEOUT, detail);
  return false;
}

// ----------------------------------------------------------------------------
// TMA (tiled bulk tensor copies; no multicast anywhere in this library)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
// x is the innermost (contiguous) coordinate: x * elemsize must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, "
      "%4}], [%2], %5;" ::"r"(smem_u32(smem_dst)),
      "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
// Ask L2 to fetch a tile (no shared memory, no barrier): hides DRAM latency behind a shallow smem pipeline.
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* m, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(m), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ----------------------------------------------------------------------------
// tcgen05 / TMEM
// ----------------------------------------------------------------------------
// One full warp allocates `ncols` (power of two, >= 32) TMEM columns; the base
// address is written to *smem_slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread.
__device__ __forceinline__ void umma_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]: A is read from tensor memory (row = lane, K packed two bf16 per 32-bit column,
// so one K = 16 step is 8 columns); A must be K-major.
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives (count 1) on the mbarrier when all previously issued MMAs of this thread are complete.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
// Bit layout: [4,6) c_format (1 = f32), [7,10) a_format (1 = bf16), [10,13) b_format,
// bit 15 a_major, bit 16 b_major (0 = K-major, 1 = MN-major), [17,23) N>>3, [24,29) M>>4.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(a_mn_major) << 15) | (uint32_t(b_mn_major) << 16) |
         (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle.  Fields are in 16-byte units:
// [0,14) start address, [16,30) leading byte offset, [32,46) stride byte offset,
// [46,48) version = 1, [61,64) layout type (2 = SWIZZLE_128B).
// K-major operand  : rows of 128 B (64 bf16 of K), 8-row groups 1024 B apart -> SBO = 1024, LBO unused (1).
// MN-major operand : rows of 128 B (64 bf16 of M/N) indexed by K; 8-K groups SBO apart, 64-wide MN blocks LBO apart.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr >> 4) & 0x3FFF);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

// The descriptor of the same layout `bytes` further into shared memory (bytes % 16 == 0; the 14-bit address field must
// not overflow, i.e. the operand stays inside the 256 KB window).  One add instead of rebuilding the descriptor keeps
// the scalar instruction chain of the MMA-issuing thread short (measured: no effect on the kernels' times, because the
// issue of an MMA waits for the tensor pipe anyway; kept for the shorter code).
__device__ __forceinline__ uint64_t smem_desc_advance(uint64_t desc, uint32_t bytes) { return desc + uint64_t(bytes >> 4); }

// TMEM -> registers: 32 lanes x 32 consecutive 32-bit columns; thread i of the warp reads lane (base_lane + i).
// A warp may only touch lanes [32 * (warp_id % 4), +32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Registers -> TMEM, same shape and lane rule as tmem_ld_32x32.
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------
// Publishing peer stores of a whole launch with ONE arrival per peer
// ----------------------------------------------------------------------------
// Every CTA of a producing launch stores rows into peers' memory.  Instead of each CTA bumping a counter on every
// peer (ctas x world remote atomics on one hot address per peer and use), the CTAs arrive on a counter in LOCAL
// memory and the last one to arrive bumps each peer's counter once.  Called by ONE thread per CTA, after a CTA-wide
// barrier that follows the CTA's peer stores (the barrier orders the other threads' stores before this thread's
// system-scope fence; the acquire-release chain through the local counter orders the other CTAs' stores before the
// last CTA's remote arrivals).  The last CTA zeroes the local counter again, so the next launch in the stream can
// reuse it; `total` is the number of CTAs that call this for one use (it may span two launches).
__device__ __forceinline__ void publish_to_peers(uint32_t* local_count, uint32_t total, uint32_t* const* peer_flag, int world) {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
  uint32_t old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(local_count) : "memory");
  if (old + 1 == total) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(local_count), "r"(0u) : "memory");
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    for (int r = 0; r < world; ++r)
      asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(peer_flag[r]), "r"(1u) : "memory");
  }
}

// ----------------------------------------------------------------------------
// Small numeric helpers
// ----------------------------------------------------------------------------
// Two fp32 values per instruction (fma.rn.f32x2 / add.f32x2 / mul.f32x2 on a 64-bit register pair) and a three-input
// maximum: epilogues and softmax loops are bound by the instruction issue of a few warps, and these halve their
// arithmetic instructions.
__device__ __forceinline__ uint64_t pack_f32x2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace ub
