// K3 on the 5th-generation tensor cores: paged prefill / shared-prefix attention with tcgen05.mma, accumulators
// in TMEM and all operands staged by TMA.
//
// Work unit: 128 packed query rows of one (sequence, kv head); a packed row is (token, head of the GQA group),
// so one K/V tile serves all G query heads of the group.  Per KV tile of 128 keys:
//   S = Q K^T          tcgen05.mma 128x128x128, S in TMEM (double-buffered, so the next tile's QK^T overlaps the
//                      softmax of this one)
//   P = exp2(S - m)    four softmax warps, one query row per thread (tcgen05.ld, no shuffles), P written as bf16
//                      into shared memory in the 128-byte-swizzled K-major layout the MMA reads
//   O_j = P V          tcgen05.mma with V as an MN-major operand straight from the page layout [key][d]
//   acc = acc * alpha + O_j   in registers of the softmax threads (read back from TMEM)
// K and V pages (16 keys x 128 d, 4 KB contiguous in the cache) are gathered through the block table with ONE TMA copy
// per page: the caches are described as 4-D tensors (64 d, 8 keys, 2 halves of d, groups of 8 keys) whose box
// {64, 8, 2, 2} lands in shared memory as [key group][d half][8 keys][128 B], i.e. as 128-byte-swizzled 8-row atoms with
// the two d halves of a key group side by side (group stride 2048 B, half stride 1024 B in the MMA descriptors).  With
// two copies per page (one per d half) the TMA unit was the limit: 32 copies per KV tile, tiles landing about 5 000
// cycles after their request and the MMA thread waiting 750 - 1 200 cycles per tile for them.  Q comes in through a
// 3-D tensor map (d, head, token) so that the packed-row order is produced by the copy itself.
//
// Handles head_dim 128, page size 16, causal (with offset, for chunked prefill and prefix-cache hits) or
// bidirectional masks, optional log-sum-exp output for merging partial results.  Sliding windows, ALiBi and other
// head sizes stay on the warp-MMA kernel (attn_prefill.cu).
//
// Replaces in the reference: ops_fn::flash_attention (crates/runtime/src/tensor_core.rs:1318-1383).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdlib.h>

#include "../common/ptx.cuh"
#include "../include/unillm_b200.h"

namespace ub {
namespace atc {

constexpr int BM = 128;           // packed query rows per CTA
constexpr int BN = 128;           // keys per tile
constexpr int HD = 128;           // head dim
constexpr int PAGE = 16;
constexpr int HALF_BYTES = BM * 128;            // one 64-column half of a 128-row operand: 16 KB
constexpr int TILE_BYTES = 2 * HALF_BYTES;      // 32 KB
constexpr int SMEM_Q = 0;
constexpr int SMEM_K = SMEM_Q + TILE_BYTES;         // 2 stages
constexpr int SMEM_V = SMEM_K + 2 * TILE_BYTES;     // 2 stages
constexpr int SMEM_P = SMEM_V + 2 * TILE_BYTES;
constexpr int SMEM_BAR = SMEM_P + TILE_BYTES;       // 192 KB of tiles, then barriers
constexpr int SMEM_XCH = SMEM_BAR + 256;            // row maxima exchanged between the two softmax warpgroups
constexpr int SMEM_TOTAL = SMEM_XCH + 3072 + 1024;  // 2 KB of maxima + 1 KB of row sums, + alignment slack
constexpr int THREADS = 320;                        // TMA warp, MMA warp, 2 x 4 softmax warps
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// UB_ATTN_DEBUG=1: CTA (0, 0, 0) records SM-cycle stamps per KV tile (up to 16 tiles): [tile][0..4] softmax warp 2 (S ready,
// S in registers, exponentials done, previous P V done, P published), [tile][5..9] MMA thread (K of the next tile landed,
// its Q K^T issued, V of this tile landed, P half 0 seen, P half 1 seen); read with ub_attn_debug_timeline.
__device__ unsigned long long g_attn_ts[16][10];

struct Params {
  int dbg;
  __nv_bfloat16* out;
  float* lse;
  const int* block_tables;
  const int* seq_lens;
  const int* q_start;
  int* err;
  int Hq, Hkv, G, max_blocks_per_seq, num_blocks;
  long long o_stride;
  float scale_log2;
  int causal;
  int kv_start;     // first key position to attend (suffix pass after a shared prefix); 0 = all
  const __nv_bfloat16* merge_o;   // optional partial over a disjoint key set, [T, Hq, HD] contiguous
  const float* merge_lse;         // its log-sum-exp, [T, Hq]
  // Key split: grid.z = num_seqs * kv_splits; CTA (seq, split) walks 1 / kv_splits of the visible KV tiles and writes
  // its partial (O rows bf16, log-sum-exp) into slot [split] of the workspace; attn_merge_splits_kernel folds them.
  int kv_splits;
  __nv_bfloat16* part_o;          // [kv_splits][total_q][Hq][HD]
  float* part_lse;                // [kv_splits][total_q][Hq]
  int total_q;
};

template <bool P_TMEM>
__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [3]
  uint64_t* k_empty = bars + 4;   // [3]
  uint64_t* v_full = bars + 7;    // [2]
  uint64_t* v_empty = bars + 9;   // [2]
  uint64_t* s_full = bars + 11;   // [2]
  uint64_t* s_empty = bars + 13;  // [2]
  uint64_t* p_full = bars + 15;   // [2] one per key half
  uint64_t* o_full = bars + 17;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  // K tiles: with P in tensor memory the shared-memory P buffer is free and serves as a third K stage, so the K copies
  // run two tiles ahead of their use (the copy of a tile is gathered from 16 boxes and completes with its slowest).
  constexpr int KST = P_TMEM ? 3 : 2;
  auto k_stage = [&](int st) { return smem + (st < 2 ? SMEM_K + st * TILE_BYTES : SMEM_P); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_wait();          // the sequence metadata read below may be written by earlier kernels of the stream
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = int(blockIdx.z) / p.kv_splits, split = int(blockIdx.z) % p.kv_splits, kh = blockIdx.y, G = p.G;
  const int TOK = BM / G;                                   // query tokens per tile
  const int q_begin = p.q_start[seq], q_end = p.q_start[seq + 1];
  const int q_len = q_end - q_begin;
  // causal: the last query tiles see the most keys; start them first so that the tail of the grid is made of short ones
  const int qtile = p.causal ? int(gridDim.x) - 1 - int(blockIdx.x) : int(blockIdx.x);
  const int t0 = q_begin + qtile * TOK;                     // first token of this tile (global token index)
  if (t0 >= q_end) return;                                  // whole CTA leaves together, nothing allocated yet
  const int kv_len = p.seq_lens[seq];
  const int t_last = min(t0 + TOK, q_end) - 1;
  int kv_hi = p.causal ? min(kv_len, kv_len - q_len + (t_last - q_begin) + 1) : kv_len;
  if (kv_hi < 0) kv_hi = 0;
  const int kv_lo = max(p.kv_start, 0);
  int tile0 = kv_lo / BN;                                   // first KV tile that holds a visible key
  int n_tiles = kv_hi > kv_lo ? (kv_hi + BN - 1) / BN - tile0 : 0;
  if (p.kv_splits > 1) {
    // this CTA's share of the tiles; the masks below stay relative to the whole range [kv_lo, limit)
    const int per = (n_tiles + p.kv_splits - 1) / p.kv_splits;
    tile0 += split * per;
    n_tiles = max(0, min(per, n_tiles - split * per));
  }

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      if (i == 0) { mbar_init(&k_full[2], 1); mbar_init(&k_empty[2], 1); }
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 256);
    }
    mbar_init(&p_full[0], 128);
    mbar_init(&p_full[1], 128);
    mbar_init(&o_full[0], 1);
    mbar_init(&o_full[1], 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();     // only now: this CTA holds its TMEM columns before any CTA of the next kernel can exist
  const uint32_t tmem_s = tmem_base;            // S buffers: columns [0,128) and [128,256)
  const uint32_t tmem_o = tmem_base + 256;      // two O accumulators, one per key half: columns [256,384) and [384,512)

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // The whole warp takes part: lanes 0..7 each own one 16-key page of the tile.  They read their block-table entry
    // one tile ahead (a dependent global load in front of every copy would otherwise serialise the pipeline) and each
    // issues the copies of its page, so a tile costs a handful of issue slots instead of 64 single-thread copies.
    if (n_tiles > 0) {
      if (lane == 0) {
        mbar_arrive_expect_tx(q_full, TILE_BYTES);
        tma_load_3d(smem + SMEM_Q, &tmap_q, q_full, 0, kh * G, t0);
        tma_load_3d(smem + SMEM_Q + HALF_BYTES, &tmap_q, q_full, 64, kh * G, t0);
      }
      const int* bt = p.block_tables + (long long)seq * p.max_blocks_per_seq;
      const int pages_valid = (kv_hi + PAGE - 1) / PAGE;
      constexpr int PPT = BN / PAGE;                       // pages per tile
      auto page_block = [&](int j) {
        int blk = 0;
        if (lane < PPT) {
          const int pi = (tile0 + j) * PPT + lane;
          blk = (pi < pages_valid && pi < p.max_blocks_per_seq) ? bt[pi] : 0;   // pages past the end: any finite page
          if (blk < 0 || blk >= p.num_blocks) { set_err(p.err, ERR_BOUNDS, blk); blk = 0; }
        }
        return blk;
      };
      // one tile of K or V: lane 0 waits for the stage and arms the barrier, lanes 0..7 copy one page each
      auto load_tile = [&](uint8_t* dst_tile, const CUtensorMap* map, uint64_t* full, uint64_t* empty, uint32_t ph, int blk,
                           int code) {
        int ok = 1;
        if (lane == 0) {
          ok = mbar_wait(empty, ph ^ 1, abort_flag, p.err, code) ? 1 : 0;
          if (ok) mbar_arrive_expect_tx(full, TILE_BYTES);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok && lane < PPT) {
          const int row = (blk * p.Hkv + kh) * PAGE;                 // first key row of the page: a multiple of 16
          tma_load_4d(dst_tile + lane * (PAGE * HD * 2), map, full, 0, 0, 0, row >> 3);
        }
        return ok != 0;
      };
      auto load_k = [&](int t, int blk) {
        const int st = t % KST;
        return load_tile(k_stage(st), &tmap_k, &k_full[st], &k_empty[st], (t / KST) & 1, blk, 500 + st);
      };
      auto load_v = [&](int t, int blk) {
        const int st = t & 1;
        return load_tile(smem + SMEM_V + st * TILE_BYTES, &tmap_v, &v_full[st], &v_empty[st], (t >> 1) & 1, blk, 510 + st);
      };
      // block ids of this lane's page in tiles j, j + 1 (and j + 2): K runs KST - 1 tiles ahead of V
      int blk_v = page_block(0);
      int blk_1 = n_tiles > 1 ? page_block(1) : 0;
      int blk_2 = (KST == 3 && n_tiles > 2) ? page_block(2) : 0;
      bool alive = load_k(0, blk_v);
      if (alive && KST == 3 && n_tiles > 1) alive = load_k(1, blk_1);
      for (int j = 0; j < n_tiles && alive; ++j) {
        const int jk = j + KST - 1;
        if (jk < n_tiles) alive = load_k(jk, KST == 3 ? blk_2 : blk_1);
        const int blk_next = (jk + 1 < n_tiles) ? page_block(jk + 1) : 0;
        if (alive) alive = load_v(j, blk_v);
        if (KST == 3) { blk_v = blk_1; blk_1 = blk_2; blk_2 = blk_next; } else { blk_v = blk_1; blk_1 = blk_next; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(BM, BN, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BM, HD, 0, 1);   // B = V is MN-major ([key][d], d contiguous)
      const uint32_t p_addr = smem_u32(smem + SMEM_P);
      // descriptors are built once and advanced by constants (the issue of the eight Q K^T MMAs takes about 700 cycles
      // either way: it proceeds at the pace of the tensor pipe)
      const uint64_t q_desc = make_smem_desc_sw128(smem_u32(smem + SMEM_Q), 16, 1024);
      const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(smem + SMEM_K), 16, 2048);
      const uint64_t k_desc2 = make_smem_desc_sw128(smem_u32(smem + SMEM_P), 16, 2048);
      const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(smem + SMEM_V), 1024, 2048);
      auto issue_qk = [&](int j) {
        const int st = j % KST;
        const uint64_t k_desc = st == 2 ? k_desc2 : smem_desc_advance(k_desc0, st * TILE_BYTES);
        const uint32_t d = tmem_s + (j & 1) * BN;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;        // Q: [d half][128 rows][128 B]
          const uint32_t koff = (k >> 2) * 1024 + (k & 3) * 32;             // K: [key group][d half][8 keys][128 B]
          umma_bf16_ss(d, smem_desc_advance(q_desc, off), smem_desc_advance(k_desc, koff), idesc_qk, k != 0);
        }
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, 520);
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag, p.err, 521);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
        umma_commit(&s_full[0]);
        umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const bool stamp = p.dbg && j < 16 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
        if (j + 1 < n_tiles) {
          const int jn = j + 1, sn = jn & 1;
          const uint32_t phn = (jn >> 1) & 1;
          if (!mbar_wait(&k_full[jn % KST], (jn / KST) & 1, abort_flag, p.err, 522)) { ok = false; break; }
          if (stamp) g_attn_ts[j][5] = clock64();
          // S buffer sn: its last readers were the softmax loads of tile j - 1 and, when P lives in TMEM, P V of
          // tile j - 1, which this thread issued before (the tensor pipe runs MMAs in issue order).
          if (!P_TMEM && !mbar_wait(&s_empty[sn], phn ^ 1, abort_flag, p.err, 523)) { ok = false; break; }
          tc_fence_after();
          issue_qk(jn);
          umma_commit(&s_full[sn]);
          umma_commit(&k_empty[jn % KST]);
        }
        if (stamp) g_attn_ts[j][6] = clock64();
        const int s = j & 1;
        if (!mbar_wait(&v_full[s], (j >> 1) & 1, abort_flag, p.err, 525)) { ok = false; break; }
        if (stamp) g_attn_ts[j][7] = clock64();
        const uint64_t v_desc = smem_desc_advance(v_desc0, s * TILE_BYTES);
        // The two key halves of the tile are independent softmax streams with their own accumulators: P_h V_h is
        // issued as soon as half h has delivered its probabilities.
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (!mbar_wait(&p_full[h], j & 1, abort_flag, p.err, 524 + 10 * h)) { ok = false; break; }
          if (stamp) g_attn_ts[j][8 + h] = clock64();
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int kk = h * 4 + k;                                    // 16-key step inside the tile
            // B = V, MN-major: 16 keys = one page = two 8-key groups (2048 B apart); the two 64-wide d blocks of a
            // group are 1024 B apart
            const uint64_t b_desc = smem_desc_advance(v_desc, kk * (PAGE * HD * 2));
            const uint32_t accumulate = (j > 0 || k != 0) ? 1u : 0u;     // O stays in TMEM over all KV tiles
            if (P_TMEM) {
              // A = P in tensor memory: packed bf16 pairs over the first 32 columns of this half's S columns
              umma_bf16_ts(tmem_o + h * HD, tmem_s + s * BN + h * 64 + k * 8, b_desc, idesc_pv, accumulate);
            } else {
              // A = P, K-major over keys: 64-key halves 16 KB apart, 16 keys = 32 B inside a 128-B row
              const uint64_t a_desc = make_smem_desc_sw128(p_addr + h * HALF_BYTES + k * 32, 16, 1024);
              umma_bf16_ss(tmem_o + h * HD, a_desc, b_desc, idesc_pv, accumulate);
            }
          }
          umma_commit(&o_full[h]);
        }
        if (!ok) break;
        umma_commit(&v_empty[s]);
      }
    }
  } else {
    // ------------------------------ softmax + output (warps 2..9) ------------------------------
    // Two warpgroups share every query row: warps 2..5 take keys [0, 64) of every tile, warps 6..9 keys [64, 128) (a
    // warp may read the TMEM lanes 32 * (warp % 4) .. + 32, at any column).  The halves are two independent
    // flash-attention streams over disjoint key sets: own exponent reference, own row sum, own O accumulator in
    // TMEM, own barriers to the MMA warp -- nothing is exchanged per tile, so the two softmax warps of a scheduler
    // drift freely and fill each other's stalls.  The streams are merged once, at the end.
    const int half = (warp - 2) >> 2;
    const int qd = warp & 3;                    // TMEM lane quarter this warp may read
    const int row = qd * 32 + lane;             // packed query row == TMEM lane
    const uint32_t lane_off = uint32_t(qd * 32) << 16;
    const int tok = t0 + row / G, head = kh * G + row % G;
    const bool row_valid = tok < q_end;
    int limit = kv_len;
    if (p.causal) limit = min(kv_len, kv_len - q_len + (tok - q_begin) + 1);
    if (!row_valid || limit < 0) limit = 0;
    // m is the exponent reference of this half row (log2 domain).  It follows the running maximum lazily: it moves
    // only when a tile's maximum exceeds it by more than 8, so probabilities stay below 2^8 and the O rows in TMEM
    // are rescaled rarely.  The final O / l does not depend on the reference.
    float m = -CUDART_INF_F, l = 0.f;
    uint8_t* p_row = smem + SMEM_P + row * 128 + half * HALF_BYTES;
    const uint32_t o_mine = tmem_o + half * HD + lane_off, o_other = tmem_o + (half ^ 1) * HD + lane_off;
    // every wait is agreed on by the whole warp: the TMEM loads and stores below are warp-wide instructions
    auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, p.err, code)) != 0;
    };
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j & 1;
      ok = ok && wait_all(&s_full[b], (j >> 1) & 1, 530);
      const bool stamp = p.dbg && warp == 2 && lane == 0 && j < 16 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
      if (stamp) g_attn_ts[j][0] = clock64();
      tc_fence_after();
      const uint32_t s_addr = tmem_s + b * BN + half * 64 + lane_off;      // this half's 64 S columns
      const int key0 = (tile0 + j) * BN + half * 64;
      // Tiles that lie completely inside [kv_lo, limit) need no per-key predicate (all but the first and last ones).
      const bool full = key0 >= kv_lo && key0 + 64 <= limit;
      uint32_t sv[2][32];
      tmem_ld_32x32(s_addr, sv[0]);
      tmem_ld_32x32(s_addr + 32, sv[1]);
      tmem_ld_wait();
      if (stamp) g_attn_ts[j][1] = clock64();
      if (!P_TMEM) {
        tc_fence_before();
        mbar_arrive(&s_empty[b]);
      }
      // independent chains per reduction: a warp has to cover its own ALU latency
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
      if (full) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
      } else {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int k = key0 + c * 32 + i;
            if (k < limit && k >= kv_lo) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[c][i]));
          }
      }
      const float m_tile = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      float alpha = 1.f;
      if (m_tile > m + 8.f) {                       // also the first visible tile (m == -inf)
        alpha = (m == -CUDART_INF_F) ? 0.f : ex2_approx(m - m_tile);
        m = m_tile;
      }
      const float m_use = (m == -CUDART_INF_F) ? 0.f : m;   // nothing visible so far: every p is masked to 0
      if (!P_TMEM && j > 0) {
        // this half of the single P buffer in shared memory is free once P_h V_h of the previous tile has completed
        ok = ok && wait_all(&o_full[half], (j - 1) & 1, 531);
      }
      uint64_t ps2[2] = {0ull, 0ull};                  // two chains of two packed row sums
      const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2), nm2 = pack_f32x2(-m_use, -m_use);
      uint32_t packed[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[c][2 * i]), __uint_as_float(sv[c][2 * i + 1])), sc2, nm2), x0, x1);
          float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
          if (!full) {
            const int k0 = key0 + c * 32 + 2 * i;
            if (!(k0 < limit && k0 >= kv_lo)) p0 = 0.f;
            if (!(k0 + 1 < limit && k0 + 1 >= kv_lo)) p1 = 0.f;
          }
          ps2[i & 1] = add_f32x2(ps2[i & 1], pack_f32x2(p0, p1));
          packed[c * 16 + i] = pack_bf16x2(p0, p1);
        }
      }
      float ps4[4];
      unpack_f32x2(ps2[0], ps4[0], ps4[1]);
      unpack_f32x2(ps2[1], ps4[2], ps4[3]);
      if (stamp) g_attn_ts[j][2] = clock64() + (packed[0] & 0u);      // after the exponentials (data dependence keeps it there)
      if (P_TMEM) {
        // 64 keys = 32 packed columns, written over the head of this half's own S columns (already in registers)
        tmem_st_32x32(s_addr, packed);
        // O_h may only be touched (and the next P_h V_h issued) after P_h V_h of the previous tile; by now it has
        // had the whole softmax of this tile to finish
        if (j > 0) ok = ok && wait_all(&o_full[half], (j - 1) & 1, 531);
      } else {
        // 64 keys = one 64-key half of the K-major P tile: 8 chunks of 16 B, swizzled by the row
#pragma unroll
        for (int q8 = 0; q8 < 8; ++q8) {
          *reinterpret_cast<uint4*>(p_row + ((q8 ^ (row & 7)) << 4)) =
              make_uint4(packed[4 * q8], packed[4 * q8 + 1], packed[4 * q8 + 2], packed[4 * q8 + 3]);
        }
      }
      l = l * alpha + ((ps4[0] + ps4[1]) + (ps4[2] + ps4[3]));
      // rescale this half's O rows when the reference moved (warp-uniform decision: the TMEM accesses are warp-wide)
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(o_mine + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32(o_mine + c * 32, r);
        }
      }
      if (stamp) g_attn_ts[j][3] = clock64();
      tmem_st_wait();
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&p_full[half]);
      if (stamp) g_attn_ts[j][4] = clock64();
    }
    // Merge of the two streams.  MMAs complete in issue order, so once this half's last P V has completed the other
    // half's barrier is at most one phase behind and its parity wait cannot alias.
    if (n_tiles > 0) {
      ok = ok && wait_all(&o_full[half], (n_tiles - 1) & 1, 532);
      ok = ok && wait_all(&o_full[half ^ 1], (n_tiles - 1) & 1, 533);
    }
    tc_fence_after();
    float* xch = reinterpret_cast<float*>(smem + SMEM_XCH);       // [2 halves][128 rows][m, l]
    xch[(half * 128 + row) * 2] = m;
    xch[(half * 128 + row) * 2 + 1] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    const float m_o = xch[((half ^ 1) * 128 + row) * 2], l_o = xch[((half ^ 1) * 128 + row) * 2 + 1];
    const float mm_ = fmaxf(m, m_o);
    const float w_mine = (m == -CUDART_INF_F) ? 0.f : ex2_approx(m - mm_);
    const float w_other = (m_o == -CUDART_INF_F) ? 0.f : ex2_approx(m_o - mm_);
    const float lt = l * w_mine + l_o * w_other;                  // row sum over all keys, reference mm_
    if (ok) {
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      float lse_v = lt > 0.f ? (mm_ * LN2 + logf(lt)) : -CUDART_INF_F;
      float ca = 0.f, cb = inv;
      const __nv_bfloat16* src = nullptr;
      if (p.merge_o != nullptr && row_valid) {
        // fold in the partial result over the other key set (shared prefix): weights exp(lse_x - max)
        const float la = p.merge_lse[(long long)tok * p.Hq + head];
        const float mx_ = fmaxf(la, lse_v);
        const float wa = (la == -CUDART_INF_F) ? 0.f : __expf(la - mx_);
        const float wb = (lse_v == -CUDART_INF_F) ? 0.f : __expf(lse_v - mx_);
        const float den = wa + wb;
        ca = den > 0.f ? wa / den : 0.f;
        cb = den > 0.f ? inv * wb / den : 0.f;
        src = p.merge_o + ((long long)tok * p.Hq + head) * HD;
        lse_v = den > 0.f ? mx_ + logf(den) : -CUDART_INF_F;
      }
      const float c_mine = (l > 0.f) ? cb * w_mine : 0.f, c_other = (l_o > 0.f) ? cb * w_other : 0.f;
      __nv_bfloat16* dst = p.out + (long long)tok * p.o_stride + (long long)head * HD;
      if (p.kv_splits > 1) dst = p.part_o + (((long long)split * p.total_q + tok) * p.Hq + head) * HD;
      // each half writes 64 of the 128 output columns, reading them from both accumulators
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        const int d0 = half * 64 + c * 32;
        uint32_t r[32], r2[32];
        tmem_ld_32x32(o_mine + d0, r);            // an accumulator that never saw a visible key is not used: l == 0
        tmem_ld_32x32(o_other + d0, r2);
        tmem_ld_wait();
        if (row_valid) {
          float o[32];
#pragma unroll
          for (int i = 0; i < 32; ++i)
            o[i] = (c_mine != 0.f ? __uint_as_float(r[i]) * c_mine : 0.f) + (c_other != 0.f ? __uint_as_float(r2[i]) * c_other : 0.f);
          if (src != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              const uint4 raw = *reinterpret_cast<const uint4*>(src + d0 + i);
              const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                o[i + 2 * e] += bf16_lo(w[e]) * ca;
                o[i + 2 * e + 1] += bf16_hi(w[e]) * ca;
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            *reinterpret_cast<uint4*>(dst + d0 + i) =
                make_uint4(pack_bf16x2(o[i], o[i + 1]), pack_bf16x2(o[i + 2], o[i + 3]),
                           pack_bf16x2(o[i + 4], o[i + 5]), pack_bf16x2(o[i + 6], o[i + 7]));
          }
        }
        __syncwarp();
      }
      if (p.kv_splits > 1) {
        if (row_valid && half == 0) p.part_lse[((long long)split * p.total_q + tok) * p.Hq + head] = lse_v;
      } else if (p.lse != nullptr && row_valid && half == 0) {
        p.lse[(long long)tok * p.Hq + head] = lse_v;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(20000);   // let bulk copies in flight land before smem is reused
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Folds the partials of a key-split launch: one warp per (token, head) row, 4 head-dim values per lane.
// out = sum_s w_s O_s with w_s = exp(lse_s - max) / sum, lse = max + log(sum); a split that saw no key has lse = -inf.
__global__ void __launch_bounds__(256) attn_merge_splits_kernel(const __nv_bfloat16* __restrict__ part_o,
                                                                 const float* __restrict__ part_lse, int splits,
                                                                 long long rows, int Hq, __nv_bfloat16* __restrict__ out,
                                                                 long long o_stride, float* __restrict__ lse) {
  pdl_wait();
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float mx = -CUDART_INF_F;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part_lse[(long long)s * rows + row]);
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, den = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float l = part_lse[(long long)s * rows + row];
    if (l == -CUDART_INF_F) continue;
    const float w = __expf(l - mx);
    den += w;
    const uint2 raw = *reinterpret_cast<const uint2*>(part_o + ((long long)s * rows + row) * HD + lane * 4);
    acc[0] += bf16_lo(raw.x) * w; acc[1] += bf16_hi(raw.x) * w;
    acc[2] += bf16_lo(raw.y) * w; acc[3] += bf16_hi(raw.y) * w;
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  const long long tok = row / Hq;
  const int head = int(row % Hq);
  *reinterpret_cast<uint2*>(out + tok * o_stride + (long long)head * HD + lane * 4) =
      make_uint2(pack_bf16x2(acc[0] * inv, acc[1] * inv), pack_bf16x2(acc[2] * inv, acc[3] * inv));
  if (lse != nullptr && lane == 0) lse[row] = den > 0.f ? mx + logf(den) : -CUDART_INF_F;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

static int encode(CUtensorMap* out, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
                  const cuuint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides_bytes, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

}  // namespace atc
}  // namespace ub

// 1 when the tensor-core kernel can run this problem.
extern "C" int ub_attn_prefill_tc_supported(const UbAttnArgs* a) {
  if (a->D != 128 || a->block_size != 16 || a->window > 0 || a->alibi_slopes != nullptr) return 0;
  if (a->Hkv <= 0 || a->Hq % a->Hkv != 0) return 0;
  const int G = a->Hq / a->Hkv;
  if (G > 128 || 128 % G != 0) return 0;
  if (a->q_stride % 8 != 0 || a->o_stride % 8 != 0) return 0;
  if ((reinterpret_cast<uintptr_t>(a->q) & 15) || (reinterpret_cast<uintptr_t>(a->out) & 15) ||
      (reinterpret_cast<uintptr_t>(a->k_cache) & 15) || (reinterpret_cast<uintptr_t>(a->v_cache) & 15))
    return 0;
  if (a->total_q <= 0) return 0;
  return 1;
}

extern "C" int ub_attn_prefill_tc(const UbAttnArgs* a, void* stream_v) {
  using namespace ub;
  using namespace ub::atc;
  if (a->num_seqs <= 0 || a->max_q_len <= 0) return 0;
  if (!ub_attn_prefill_tc_supported(a)) return -4;
  const int G = a->Hq / a->Hkv;
  const int TOK = BM / G;
  CUtensorMap tq, tk, tv;
  {
    // Q viewed as (d, head, token): box = 64 d x G heads x TOK tokens -> rows ordered (token, head in group)
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)a->Hq, (cuuint64_t)a->total_q};
    cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)a->q_stride * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)TOK};
    int rc = encode(&tq, a->q, 3, dims, strides, box);
    if (rc != 0) return rc;
  }
  {
    // K / V caches: key row r = (block * Hkv + kv head) * 16 + slot is 256 B; viewed as (64 d, 8 keys, 2 d halves, r / 8)
    // so that one box {64, 8, 2, 2} is a whole page, delivered as swizzled 8-key atoms with the d halves side by side
    cuuint64_t dims[4] = {64, 8, 2, (cuuint64_t)a->num_blocks * a->Hkv * PAGE / 8};
    cuuint64_t strides[3] = {(cuuint64_t)HD * 2, 128, (cuuint64_t)HD * 2 * 8};
    cuuint32_t box[4] = {64, 8, 2, 2};
    int rc = encode(&tk, a->k_cache, 4, dims, strides, box);
    if (rc != 0) return rc;
    rc = encode(&tv, a->v_cache, 4, dims, strides, box);
    if (rc != 0) return rc;
  }
  Params p;
  {
    static int dbg = -1;
    if (dbg < 0) { const char* e = getenv("UB_ATTN_DEBUG"); dbg = e ? atoi(e) : 0; }
    p.dbg = dbg;
  }
  p.out = reinterpret_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.block_tables = a->block_tables;
  p.seq_lens = a->seq_lens;
  p.q_start = a->q_start;
  p.err = a->err;
  p.Hq = a->Hq; p.Hkv = a->Hkv; p.G = G;
  p.max_blocks_per_seq = a->max_blocks_per_seq;
  p.num_blocks = a->num_blocks;
  p.o_stride = a->o_stride;
  p.scale_log2 = a->scale * LOG2E;
  p.causal = a->causal;
  p.kv_start = a->kv_start;
  p.merge_o = reinterpret_cast<const __nv_bfloat16*>(a->merge_o);
  p.merge_lse = a->merge_lse;
  // Key split (a->splits > 1): the caller provides the workspace in a->scratch, laid out as the log-sum-exps
  // [splits][total_q][Hq] fp32 (rounded up to 16 bytes) followed by the partial rows [splits][total_q][Hq][128] bf16.
  int S = a->splits > 1 ? a->splits : 1;
  if (S > 16) S = 16;
  if (S > 1 && (a->scratch == nullptr || a->merge_o != nullptr)) return -7;
  p.kv_splits = S;
  p.total_q = a->total_q;
  p.part_lse = a->scratch;
  {
    const long long lse_floats = ((long long)S * a->total_q * a->Hq + 3) / 4 * 4;
    p.part_o = S > 1 ? reinterpret_cast<__nv_bfloat16*>(a->scratch + lse_floats) : nullptr;
  }
  // P (the probabilities fed to the second MMA) lives in tensor memory by default; UB_ATTN_TC_P=smem stages it in
  // shared memory instead (the A operand then comes through a shared-memory descriptor).
  static const bool p_tmem = [] {
    const char* e = getenv("UB_ATTN_TC_P");
    return !(e != nullptr && e[0] == 's');
  }();
  static bool attr_set[UB_MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < UB_MAX_DEVICES && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_prefill_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) return -(int)e;
    attr_set[dev] = true;
  }
  dim3 grid((a->max_q_len + TOK - 1) / TOK, a->Hkv, a->num_seqs * S);
  if (p_tmem)
    launch_pdl(attn_prefill_tc_kernel<true>, grid, dim3(THREADS), (size_t)SMEM_TOTAL, reinterpret_cast<cudaStream_t>(stream_v), tq, tk, tv, p);
  else
    launch_pdl(attn_prefill_tc_kernel<false>, grid, dim3(THREADS), (size_t)SMEM_TOTAL, reinterpret_cast<cudaStream_t>(stream_v), tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return -(int)e;
  if (S > 1) {
    const long long rows = (long long)a->total_q * a->Hq;
    launch_pdl(attn_merge_splits_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), (size_t)0,
               reinterpret_cast<cudaStream_t>(stream_v), (const __nv_bfloat16*)p.part_o, (const float*)p.part_lse, S, rows,
               a->Hq, p.out, (long long)a->o_stride, a->lse);
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? 0 : -(int)e;
}

// Copies the per-tile stamps of the last launch made under UB_ATTN_DEBUG=1 to `out` ([16][10] uint64, SM cycles).
extern "C" int ub_attn_debug_timeline(unsigned long long* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, ub::atc::g_attn_ts, sizeof(unsigned long long) * 16 * 10);
  return e == cudaSuccess ? 0 : -(int)e;
}
