// K4, short key ranges: persistent paged decode attention with the copies of the NEXT work item in flight while the
// current one is finished.
//
// The second pass of the cascade (every sequence attends to its own 128..256 keys behind a shared prefix) gives each
// (sequence, kv head) work item only two to four 64-key tiles.  In attn_decode_mma.cu one CTA serves one item, so its
// life is a chain of dependent latencies -- sequence length, block-table entries, keys / values, merge partial -- and
// the kernel reaches 0.4 of the copy bandwidth.  Here a CTA walks over many items; while it computes the last tile
// of an item and runs that item's epilogue, the first tile of the next item is already being copied, and the next
// item's length, block-table entries, query rows and merge partial were requested one item earlier.
//
// Keys and values arrive by TMA (template flag): a 16-byte cp.async per thread keeps only a few tens of KB in flight
// per SM -- about 20 GB/s per SM at HBM latency, which is what both decode kernels measured -- while one bulk tensor
// copy moves a whole 16-key page half (2 KB) and many of them can be outstanding.  The boxes land in the 128-byte
// swizzled layout (two planes of 64 head-dim columns), which ldmatrix reads without bank conflicts.
//
// Same math and layouts as attn_decode_mma.cu (warp-level m16n8k16 MMAs, the GQA group as the 16 MMA rows, 64-key
// tiles gathered page by page with cp.async into XOR-swizzled shared memory, four warps with 16 keys each and their
// own online-softmax state).  Restrictions: no sliding window, no ALiBi, no KV splits (the caller falls back to the
// one-item-per-CTA kernel otherwise).
//
// Replaces in the reference: the cached attention path of LlamaAttention::forward_with_cache
// (crates/runtime/src/models_v2/llama.rs:1027-1156) where q_len == 1.
#include <cuda.h>
#include <math_constants.h>
#include <stdlib.h>
#include <string.h>

#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"

namespace ub {
namespace dper {

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr int KT = 64;       // keys per tile (16 per warp)
constexpr int ROWS = 16;     // query heads per CTA (MMA M)
constexpr int NST = 2;       // ring stages: one tile in use, one in flight
constexpr int BT_MAX = 128;  // block-table entries kept in shared memory per item (one per thread)

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
__device__ __forceinline__ float ex2a(float x) {        // 2^x, approximate; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// [rows][D] bf16 tile with 16-byte chunks XOR-swizzled by (row & 7)
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

// TMA layout of a [KT][D] tile: planes of 64 columns, rows of 128 bytes, 16-byte chunks XOR-swizzled by (row & 7)
template <int D, bool TMA>
__device__ __forceinline__ uint32_t kv_off(int row, int chunk) {
  if (TMA) return (uint32_t)((chunk >> 3) * (KT * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
  return tile_off<D>(row, chunk);
}

template <int D>
struct Smem {
  static constexpr int STAGE_BYTES = 2 * KT * D * 2;                 // K tile then V tile
  static constexpr int RED_BYTES = 4 * ROWS * D * 4;                 // per-warp partial outputs (fp32): fits one stage
  static_assert(RED_BYTES <= STAGE_BYTES, "the reduction buffer overlays one ring stage");
  static constexpr int Q_OFF = NST * STAGE_BYTES;                    // 2 x [16][D] bf16, swizzled
  static constexpr int ML_OFF = Q_OFF + 2 * ROWS * D * 2;            // [4][16][2] floats
  static constexpr int BT_OFF = ML_OFF + 4 * ROWS * 2 * 4;           // 2 x BT_MAX block-table entries
  static constexpr int ROW_OFF = BT_OFF + 2 * BT_MAX * 4;            // [16 rows][8] floats: epilogue coefficients per row
  static constexpr int BAR_OFF = ROW_OFF + ROWS * 8 * 4;             // NST mbarriers + abort flag
  static constexpr int USED = BAR_OFF + NST * 8 + 16;
  static constexpr int ALIGN_SLACK = 1024;                           // TMA only: the swizzled boxes want 1024-byte aligned stages
};

// What the copy of a tile and the arithmetic on it need to know about a work item.
struct Item {
  int seq, kvh, gc;
  int kv_len, kv_lo, kv_hi, tile_origin, n_tiles, page0;
};

template <int D, bool TMA>
__global__ void __launch_bounds__(128, 3)
attn_decode_persist_kernel(const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv,
                           const UbAttnArgs a, const int gchunks, const int n_items) {
  constexpr int CPR = D / 8;                 // 16-byte chunks per row
  constexpr int QPT = ROWS * CPR / 128;      // query chunks per thread
  constexpr int PRE = 4;                     // merge-partial elements per thread kept in registers (GQA group of 4)
  using S = Smem<D>;
  extern __shared__ __align__(128) uint8_t dsm_raw[];
  uint8_t* dsm = TMA ? reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dsm_raw) + 1023) & ~uintptr_t(1023)) : dsm_raw;
  float (*red_ml)[ROWS][2] = reinterpret_cast<float (*)[ROWS][2]>(dsm + S::ML_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(dsm + S::BAR_OFF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + NST);

  pdl_launch_dependents();
  pdl_wait();          // no global access before the previous kernel has completed

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Gtot = a.Hq / a.Hkv;
  const int per_seq = a.Hkv * gchunks;
  const int bs_shift = 31 - __clz(a.block_size);
  const int kv_lo = max(a.kv_start, 0);                       // no window, no splits: the same for every item
  const int tile_origin = kv_lo & ~(a.block_size - 1);
  const int page0 = tile_origin >> bs_shift;
  const int pages_per_tile = KT >> bs_shift;
  const int chunks_per_page = CPR << bs_shift;
  const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(a.k_cache);
  const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(a.v_cache);
  const __nv_bfloat16* mo = reinterpret_cast<const __nv_bfloat16*>(a.merge_o);
  const float sc = a.scale * LOG2E;

  // ---- the next item's metadata: requested one item ahead, held in registers until it is committed to shared memory
  int nx_len = 0, nx_bt = -1;
  uint4 nx_q[QPT];
  float nx_la[PRE], nx_oa[PRE];
  auto decode_item = [&](int item, int& seq, int& kvh, int& gc) {
    seq = item / per_seq;
    const int rem = item - seq * per_seq;
    kvh = rem / gchunks;
    gc = rem - kvh * gchunks;
  };
  auto request = [&](int item) {
    int seq, kvh, gc;
    decode_item(item, seq, kvh, gc);
    const int h0 = kvh * Gtot + gc * ROWS;
    const int gn = min(ROWS, Gtot - gc * ROWS);
    nx_len = a.seq_lens[seq];
    const int bi = page0 + (int)threadIdx.x;
    nx_bt = bi < a.max_blocks_per_seq ? a.block_tables[(long long)seq * a.max_blocks_per_seq + bi] : -1;
    const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(a.q) + (long long)seq * a.q_stride;
#pragma unroll
    for (int k = 0; k < QPT; ++k) {
      const int i = threadIdx.x + k * 128, r = i / CPR, c = i % CPR;
      nx_q[k] = make_uint4(0, 0, 0, 0);
      if (r < gn) nx_q[k] = *reinterpret_cast<const uint4*>(qp + (long long)(h0 + r) * D + c * 8);
    }
#pragma unroll
    for (int k = 0; k < PRE; ++k) {
      const int i = threadIdx.x + k * 128;
      nx_la[k] = 0.f;
      nx_oa[k] = 0.f;
      if (mo != nullptr && i < gn * D) {
        const int h = h0 + i / D;
        nx_la[k] = a.merge_lse[(long long)seq * a.Hq + h];
        nx_oa[k] = __bfloat162float(mo[((long long)seq * a.Hq + h) * D + i % D]);
      }
    }
  };
  // writes the requested block-table entries and query rows into buffer `buf`, returns the item's key range
  auto commit = [&](int item, int buf) {
    int* bt_sm = reinterpret_cast<int*>(dsm + S::BT_OFF) + buf * BT_MAX;
    uint8_t* q_sm = dsm + S::Q_OFF + buf * ROWS * D * 2;
    bt_sm[threadIdx.x] = nx_bt;
#pragma unroll
    for (int k = 0; k < QPT; ++k) {
      const int i = threadIdx.x + k * 128, r = i / CPR, c = i % CPR;
      *reinterpret_cast<uint4*>(q_sm + tile_off<D>(r, c)) = nx_q[k];
    }
    Item it;
    decode_item(item, it.seq, it.kvh, it.gc);
    it.kv_len = nx_len;
    it.kv_lo = kv_lo;
    it.kv_hi = nx_len;
    it.tile_origin = tile_origin;
    it.page0 = page0;
    const int nt = it.kv_hi > tile_origin ? (it.kv_hi - tile_origin + KT - 1) / KT : 0;
    it.n_tiles = max(nt, 1);               // an empty range still runs one (fully masked, zero-filled) tile
    return it;
  };
  // copies tile t of an item into ring stage `stage`: whole pages, 16-byte chunks at consecutive addresses
  auto issue_tile = [&](const Item& it, int buf, int t, int stage) {
    const int* bt_sm = reinterpret_cast<const int*>(dsm + S::BT_OFF) + buf * BT_MAX;
    uint8_t* st = dsm + stage * S::STAGE_BYTES;
    const int t0 = it.tile_origin + t * KT;
    if (TMA) {
      // thread 0 arms the stage's barrier with the bytes of the pages that exist; lane 0 of every warp copies the
      // pages pg = warp, warp + 4, ... (one box per page and plane), so no single warp carries all the issue work.
      // A copy may complete before the barrier is armed: the phase cannot end while thread 0's arrival is pending.
      // first global row of page pg in the cache view, or -1 when the page is past the end of the sequence
      auto page_row = [&](int pg) {
        const int pos0 = t0 + (pg << bs_shift);
        if (pos0 >= it.kv_hi) return -1;
        const int bi = pos0 >> bs_shift;
        int blk = -1;
        if (bi < a.max_blocks_per_seq)
          blk = (bi - it.page0) < BT_MAX ? bt_sm[bi - it.page0] : a.block_tables[(long long)it.seq * a.max_blocks_per_seq + bi];
        if (blk < 0 || blk >= a.num_blocks) { set_err(a.err, ERR_BOUNDS, it.seq); return -1; }
        return (blk * a.Hkv + it.kvh) << bs_shift;
      };
      if (threadIdx.x == 0) {
        uint32_t bytes = 0;
        for (int pg = 0; pg < pages_per_tile; ++pg)
          if (page_row(pg) >= 0) bytes += 2u * (uint32_t)a.block_size * D * 2u;
        mbar_arrive_expect_tx(&bars[stage], bytes);
      }
      if (lane == 0) {
        for (int pg = warp; pg < pages_per_tile; pg += 4) {
          const int row = page_row(pg);
          if (row < 0) continue;
          uint8_t* dk = st + (pg << bs_shift) * 128;
          uint8_t* dv = dk + KT * D * 2;
#pragma unroll
          for (int pl = 0; pl < D / 64; ++pl) {
            tma_load_2d(dk + pl * KT * 128, &tmk, &bars[stage], pl * 64, row);
            tma_load_2d(dv + pl * KT * 128, &tmv, &bars[stage], pl * 64, row);
          }
        }
      }
      return;
    }
    for (int pg = 0; pg < pages_per_tile; ++pg) {
      const int pos0 = t0 + (pg << bs_shift);
      const int nvalid = min(max(it.kv_hi - pos0, 0), a.block_size);       // keys of this page that exist
      long long base = 0;
      if (nvalid > 0) {
        const int bi = pos0 >> bs_shift;
        int blk = -1;
        if (bi < a.max_blocks_per_seq)
          blk = (bi - it.page0) < BT_MAX ? bt_sm[bi - it.page0] : a.block_tables[(long long)it.seq * a.max_blocks_per_seq + bi];
        if (blk < 0 || blk >= a.num_blocks) set_err(a.err, ERR_BOUNDS, it.seq);
        else base = (((long long)blk * a.Hkv + it.kvh) << bs_shift) * D;
      }
      for (int c = threadIdx.x; c < chunks_per_page; c += 128) {
        const int tr = c / CPR;
        const int r = (pg << bs_shift) + tr;
        const bool ok = tr < nvalid;
        const uint32_t dst = tile_off<D>(r, c % CPR);
        cp_async16(st + dst, kc + base + c * 8, ok);
        cp_async16(st + KT * D * 2 + dst, vc + base + c * 8, ok);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  int item = blockIdx.x;
  if (item >= n_items) return;
  if (TMA) {
    if (threadIdx.x == 0) {
      *abort_flag = 0;
      for (int i = 0; i < NST; ++i) mbar_init(&bars[i], 1);
      fence_mbar_init();
    }
    // rows that no copy ever fills (pages past the end of a sequence) are multiplied by zero probabilities: they have
    // to hold finite values
    for (int i = threadIdx.x; i < NST * S::STAGE_BYTES / 16; i += 128) reinterpret_cast<uint4*>(dsm)[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async_smem();
  }
  request(item);
  Item cur = commit(item, 0);
  float cur_la[PRE], cur_oa[PRE];
#pragma unroll
  for (int k = 0; k < PRE; ++k) { cur_la[k] = nx_la[k]; cur_oa[k] = nx_oa[k]; }
  __syncthreads();                                   // block-table entries and query rows of the first item are visible
  int g = 0;                                         // flat tile counter over all items of this CTA: ring stage = g % NST
  int buf = 0;
  issue_tile(cur, buf, 0, 0);

  const int ra = lane >> 2, rb = ra + 8;             // this thread's MMA rows (query heads of the group)
  while (true) {
    const int next_item = item + (int)gridDim.x;
    const bool has_next = next_item < n_items;
    if (has_next) request(next_item);                // its loads run under the wait for this item's first tile
    const int h0 = cur.kvh * Gtot + cur.gc * ROWS;
    const int gn = min(ROWS, Gtot - cur.gc * ROWS);
    const uint8_t* q_sm = dsm + S::Q_OFF + buf * ROWS * D * 2;
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
      const int c = ks * 2 + (lane >> 4);
      ldsm_x4(smem_u32(q_sm + tile_off<D>(r, c)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_a = -CUDART_INF_F, m_b = -CUDART_INF_F, l_a = 0.f, l_b = 0.f;
    Item nxt = cur;

    for (int t = 0; t < cur.n_tiles; ++t, ++g) {
      bool landed = true;
      if (TMA) {
        landed = mbar_wait(&bars[g % NST], (g / NST) & 1, abort_flag, a.err, 700 + (g % NST));
        fence_proxy_async_smem();          // this thread's earlier generic writes to the stage refilled next (reduction
                                           // buffer) are ordered before the bulk copy issued after the barrier
      } else {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      // flat tile g is visible; everyone is done with tile g - 1 and with the previous item's reduction buffer, which
      // lived in the stage filled next.  A wait that gave up ends the CTA for all threads together.
      if (__syncthreads_or(!landed)) {
        for (int i = 0; i < 64; ++i) __nanosleep(20000);   // let bulk copies in flight land before the CTA's smem is reused
        return;
      }
      if (t == 0 && has_next) {
        nxt = commit(next_item, buf ^ 1);
        __syncthreads();                   // the next item's block-table entries are visible before its first copy
      }
      if (t + 1 < cur.n_tiles) issue_tile(cur, buf, t + 1, (g + 1) % NST);
      else if (has_next) issue_tile(nxt, buf ^ 1, 0, (g + 1) % NST);
      else if (!TMA) asm volatile("cp.async.commit_group;" ::: "memory");

      const uint8_t* kb = dsm + (g % NST) * S::STAGE_BYTES;
      const uint8_t* vb = kb + KT * D * 2;
      const int tw0 = warp * 16;           // this warp's 16 keys inside the tile
      const int t0 = cur.tile_origin + t * KT + tw0;
      if (t0 >= cur.kv_hi || t0 + 16 <= cur.kv_lo) continue;   // warp-uniform: nothing visible in this warp's slice

      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int mi = lane >> 3;
        const int r = tw0 + (mi >> 1) * 8 + (lane & 7);
        const int c = ks * 2 + (mi & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(kb + kv_off<D, TMA>(r, c)), b0, b1, b2, b3);
        mma_bf16(s[0], qf[ks], b0, b1);
        mma_bf16(s[1], qf[ks], b2, b3);
      }
      float mx_a = m_a, mx_b = m_b;
      if (t0 >= cur.kv_lo && t0 + 16 <= cur.kv_hi) {
        // interior slice: every key of this warp is visible, no per-key predicate
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          s[j][0] *= sc; s[j][1] *= sc; s[j][2] *= sc; s[j][3] *= sc;
          mx_a = fmaxf(mx_a, fmaxf(s[j][0], s[j][1]));
          mx_b = fmaxf(mx_b, fmaxf(s[j][2], s[j][3]));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int kpos = t0 + j * 8 + (lane & 3) * 2 + (e & 1);
            const float v = (kpos < cur.kv_hi && kpos >= cur.kv_lo) ? s[j][e] * sc : -CUDART_INF_F;
            s[j][e] = v;
            if (e >= 2) mx_b = fmaxf(mx_b, v); else mx_a = fmaxf(mx_a, v);
          }
        }
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      // 2^-inf = 0 covers masked keys and the first tile; a row with nothing visible so far keeps reference 0
      const float ref_a = (mx_a == -CUDART_INF_F) ? 0.f : mx_a, ref_b = (mx_b == -CUDART_INF_F) ? 0.f : mx_b;
      const float al_a = (mx_a == m_a) ? 1.f : ex2a(m_a - ref_a);
      const float al_b = (mx_b == m_b) ? 1.f : ex2a(m_b - ref_b);
      m_a = mx_a; m_b = mx_b;
      float ps_a = 0.f, ps_b = 0.f;
      uint32_t pf[4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float p0 = ex2a(s[j][0] - ref_a), p1 = ex2a(s[j][1] - ref_a);
        const float p2 = ex2a(s[j][2] - ref_b), p3 = ex2a(s[j][3] - ref_b);
        ps_a += p0 + p1; ps_b += p2 + p3;
        pf[j * 2 + 0] = pack_bf16x2(p0, p1);     // accumulator layout of two adjacent n8 tiles == A fragment of a k16 step
        pf[j * 2 + 1] = pack_bf16x2(p2, p3);
      }
      l_a = l_a * al_a + ps_a;
      l_b = l_b * al_b + ps_b;
      // the running maximum seldom moves after the first tiles: skip the rescale of the 64 accumulators then
      if (__any_sync(0xffffffffu, al_a != 1.f || al_b != 1.f)) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b; }
      }
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        const int mi = lane >> 3;
        const int r = tw0 + (mi & 1) * 8 + (lane & 7);
        const int c = dp * 2 + (mi >> 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(vb + kv_off<D, TMA>(r, c)), b0, b1, b2, b3);
        mma_bf16(o[dp * 2], pf, b0, b1);
        mma_bf16(o[dp * 2 + 1], pf, b2, b3);
      }
    }

    // ---- epilogue of the current item.  The stage of its last tile is free (the copy in flight, if any, fills the
    // other one): the four warps' partial outputs are combined there.
    __syncthreads();                           // every warp is done with the last tile
    float (*red_o)[ROWS][D] = reinterpret_cast<float (*)[ROWS][D]>(dsm + ((g + NST - 1) % NST) * S::STAGE_BYTES);
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
    // per-row scalars once per row (not once per output element): weights of the four warps' partials, already
    // divided by the row sum and, with a partial to merge, multiplied by this pass's share; the partial's share; LSE
    float (*row_s)[8] = reinterpret_cast<float (*)[8]>(dsm + S::ROW_OFF);
    if ((int)threadIdx.x < gn) {
      const int gq = threadIdx.x, h = h0 + gq;
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int w = 0; w < 4; ++w) mx = fmaxf(mx, red_ml[w][gq][0]);
      const float ref = (mx == -CUDART_INF_F) ? 0.f : mx;
      float scw[4], lt = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        scw[w] = ex2a(red_ml[w][gq][0] - ref);
        lt += red_ml[w][gq][1] * scw[w];
      }
      float mine = lt > 0.f ? 1.f / lt : 0.f;            // factor on this pass's unnormalised output
      float lse = lt > 0.f ? (mx + log2f(lt)) * LN2 : -CUDART_INF_F;
      float ca = 0.f;
      if (mo != nullptr) {
        // fold in the partial result over the other key set (shared prefix): weights exp(lse_x - max)
        float la;
        if (D == 128 && gq < PRE) la = gq == 0 ? cur_la[0] : gq == 1 ? cur_la[1] : gq == 2 ? cur_la[2] : cur_la[3];
        else la = a.merge_lse[(long long)cur.seq * a.Hq + h];
        const float mm = fmaxf(la, lse);
        const float wa = (la == -CUDART_INF_F) ? 0.f : __expf(la - mm);
        const float wb = (lse == -CUDART_INF_F) ? 0.f : __expf(lse - mm);
        const float den = wa + wb;
        ca = den > 0.f ? wa / den : 0.f;
        mine = den > 0.f ? mine * wb / den : 0.f;
        lse = den > 0.f ? mm + __logf(den) : -CUDART_INF_F;
      }
#pragma unroll
      for (int w = 0; w < 4; ++w) row_s[gq][w] = scw[w] * mine;
      row_s[gq][4] = ca;
      if (a.lse != nullptr) a.lse[(long long)cur.seq * a.Hq + h] = lse;
    }
    __syncthreads();
    for (int i = threadIdx.x, it = 0; i < gn * D; i += 128, ++it) {
      const int gq = i / D, d = i % D;
      float val = red_o[0][gq][d] * row_s[gq][0] + red_o[1][gq][d] * row_s[gq][1] + red_o[2][gq][d] * row_s[gq][2] +
                  red_o[3][gq][d] * row_s[gq][3];
      if (mo != nullptr) {
        float oa;
        if (it < PRE) oa = it == 0 ? cur_oa[0] : it == 1 ? cur_oa[1] : it == 2 ? cur_oa[2] : cur_oa[3];
        else oa = __bfloat162float(mo[((long long)cur.seq * a.Hq + h0 + gq) * D + d]);
        val += oa * row_s[gq][4];
      }
      reinterpret_cast<__nv_bfloat16*>(a.out)[(long long)cur.seq * a.o_stride + (long long)(h0 + gq) * D + d] = __float2bfloat16(val);
    }
    if (!has_next) break;
    // the reduction buffer is read above; the stage it lives in is refilled only after the barrier at the top of the
    // next item's first tile
    item = next_item;
    cur = nxt;
    buf ^= 1;
#pragma unroll
    for (int k = 0; k < PRE; ++k) { cur_la[k] = nx_la[k]; cur_oa[k] = nx_oa[k]; }
  }
  if (!TMA) asm volatile("cp.async.wait_group 0;" ::: "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// K / V cache viewed as rows of D columns (row = (block * Hkv + kv head) * block_size + slot); box = 64 columns x one page
static int encode_cache_map(CUtensorMap* out, const void* base, int D, long long rows, int block_size) {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)block_size};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

template <int D, bool TMA>
static int launch(const UbAttnArgs& a, cudaStream_t st) {
  constexpr int SMEM = Smem<D>::USED + (TMA ? Smem<D>::ALIGN_SLACK : 0);   // without the slack three CTAs fit on an SM
  static bool attr_set[UB_MAX_DEVICES] = {};
  static int sms[UB_MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= UB_MAX_DEVICES) return -1;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_persist_kernel<D, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return -(int)e;
    cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    attr_set[dev] = true;
  }
  const int Gtot = a.Hq / a.Hkv;
  const int gchunks = (Gtot + ROWS - 1) / ROWS;
  const int n_items = a.num_seqs * a.Hkv * gchunks;
  if (n_items <= 0) return 0;
  int grid = 3 * sms[dev];                       // three resident CTAs per SM
  if (grid > n_items) grid = n_items;
  CUtensorMap tmk, tmv;
  memset(&tmk, 0, sizeof(tmk));
  memset(&tmv, 0, sizeof(tmv));
  if (TMA) {
    const long long rows = (long long)a.num_blocks * a.Hkv * a.block_size;
    int rc = encode_cache_map(&tmk, a.k_cache, D, rows, a.block_size);
    if (rc == 0) rc = encode_cache_map(&tmv, a.v_cache, D, rows, a.block_size);
    if (rc != 0) return rc;
  }
  cudaError_t e = ub::launch_pdl(attn_decode_persist_kernel<D, TMA>, dim3(grid), dim3(128), (size_t)SMEM, st, tmk, tmv, a,
                                 gchunks, n_items);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

}  // namespace dper
}  // namespace ub

// Persistent decode attention for short key ranges.  Supported: head size 64 / 128, page sizes 8..64, no sliding
// window, no ALiBi, no KV splits; the caller checks with ub_attn_decode_persist_supported.
extern "C" int ub_attn_decode_persist_supported(const UbAttnArgs* a) {
  if (a->D != 64 && a->D != 128) return 0;
  if (a->block_size < 8 || a->block_size > 64 || (a->block_size & (a->block_size - 1))) return 0;
  if (a->Hkv <= 0 || a->Hq % a->Hkv != 0 || a->q_stride % 8 != 0) return 0;
  if (a->window > 0 || a->alibi_slopes != nullptr || a->splits != 1) return 0;
  if ((reinterpret_cast<uintptr_t>(a->q) & 15) || (reinterpret_cast<uintptr_t>(a->k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(a->v_cache) & 15))
    return 0;
  return 1;
}

extern "C" int ub_attn_decode_persist(const UbAttnArgs* a, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // UB_DECODE_TMA=1: keys / values through bulk tensor copies instead of per-thread cp.async.  Measured slower on the
  // serving step (82.9 vs 69.8 us per layer: all threads poll the stage barrier and one thread issues the boxes), so
  // cp.async is the default.
  static const bool tma = [] {
    const char* e = getenv("UB_DECODE_TMA");
    return e != nullptr && e[0] == '1';
  }();
  if (tma) return a->D == 64 ? ub::dper::launch<64, true>(*a, st) : ub::dper::launch<128, true>(*a, st);
  return a->D == 64 ? ub::dper::launch<64, false>(*a, st) : ub::dper::launch<128, false>(*a, st);
}
