/* C ABI of libunillm_b200_cuda.so: every entry point takes raw device pointers and a CUDA
 * stream (as void*), launches asynchronously on that stream and returns 0 on success or a
 * negative code.  No entry point allocates device memory unless its comment says so.
 * The Python package binds these with ctypes (unillm_b200/ops/_native.py); the structs below
 * are mirrored there field by field. */
#ifndef UNILLM_B200_H_
#define UNILLM_B200_H_
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define UB_MAX_RANKS 8
#define UB_MAX_DEVICES 16

enum UbAct {
  UB_ACT_NONE = 0,
  UB_ACT_SILU = 1,
  UB_ACT_GELU = 2,
  UB_ACT_GELU_TANH = 3,
  UB_ACT_RELU = 4,
  UB_ACT_RELU2 = 5,
  UB_ACT_QUICK_GELU = 6,
  UB_ACT_SIGMOID = 7,
  UB_ACT_TANH = 8,
  UB_ACT_SOFTPLUS = 9,
  UB_ACT_EXP = 10,
};

/* ---------------- K1 / K2 / F1 / F3 : tcgen05 GEMM  out[M,N] = epi(x[M,K] @ w[N,K]^T) ---------------- */
typedef struct UbGemmArgs {
  const void* x;        /* bf16 [M, ldx]  */
  const void* w;        /* bf16 [N or w_rows_total, ldw] */
  void* out;            /* bf16 (or fp32 when out_f32) [M, ldo] */
  const void* bias;     /* bf16 [N] or NULL */
  const void* residual; /* bf16 [M, ldr] or NULL: added to the result */
  int* err;             /* int[2] device error word or NULL */
  int M, N, K;
  long long ldx, ldw, ldo, ldr;
  int act;              /* UbAct applied to the result (dual: to the gate half) */
  int dual;             /* 1: out = act(x w_gate^T) * (x w_up^T); gate rows [0,N), up rows [up_row_off, +N) */
  int up_row_off;
  int w_rows_total;     /* dual: number of rows of w (e.g. 2*N) */
  int out_f32;
  float out_scale;      /* 0 or 1 = none */
  int tile_tokens;      /* 0 = auto; else 16/32/64/128/256 */
  int splits;           /* 0 = auto; 1 = no split-K; 2/4/8 = cluster size of the split-K reduction */
  /* F1: push rows to the rank that owns the token instead of writing `out`. */
  int rs_world, rs_rank, rs_rows_per_rank;
  void* rs_peer_out[UB_MAX_RANKS];
  uint32_t* rs_peer_flag[UB_MAX_RANKS];
  /* F3: wait for token rows gathered from other ranks. */
  int ag_world, ag_rows_per_rank;
  const uint32_t* ag_flags;
  const uint32_t* ag_epoch;
  uint32_t ag_signals_per_use;
  /* K13 grouped mode (MoE): x is the expert-sorted activation matrix [M, K]; w stacks the experts' weights
     row-wise ([num_experts * grp_w_rows, K], w_rows_total = that row count).  grp_tiles is the int4 table written
     by ub_moe_route for token tile `tile_tokens`: {expert or -1, first row, end row, 0}.  NULL disables. */
  const void* grp_tiles;
  int grp_max_tiles;
  int grp_w_rows;
  int tail_split;       /* 0 = auto (split K of a thin last round over clusters in a second launch), 1 = never */
  int cta_pair;         /* 0 = auto, 1 = never, 2 = always: tiles of 256 weight rows on pairs of CTAs (cta_group::2) */
  int pair_splits;      /* 0 = auto; 1 / 2 / 4: K slices (pairs per tile) when the CTA-pair kernel is used */
  /* F1: a zeroed u32 in LOCAL memory on which the CTAs of this GEMM arrive; the last one bumps every rs_peer_flag
     once (one arrival per source rank and use at the consumer).  Required when rs_world > 0. */
  uint32_t* rs_local_count;
} UbGemmArgs;
int ub_gemm_tn(const UbGemmArgs* args, void* stream);
/* Number of CTAs the launch for `args` will use; each CTA signals every peer once in F1 mode. */
int ub_gemm_num_ctas(const UbGemmArgs* args);
/* Shared-memory fill-rate probe (csrc/common/fill_probe.cu): one CTA per SM brings `steps` 16 KB tiles of the bf16 matrix
 * buf[rows][K] into shared memory; mode 0 linear bulk copies, 1 tensor-map tiles of the row-major matrix, 2 tensor-map
 * tiles stored contiguously.  cycles: int64 per SM.  Returns the number of CTAs, negative on error. */
int ub_fill_probe(const void* buf, int rows, int K, int mode, int steps, int* err, long long* cycles, void* stream);
/* Lowers the flags of the GEMM's stream-K workspace on the current device; call after a launch reported a timed-out
 * wait in the error word (a flag raised for a consumer that gave up would otherwise be taken for the next launch's). */
int ub_gemm_streamk_reset(void* stream);

/* ---------------- K5 : normalisation ---------------- */
typedef struct UbNormArgs {
  const void* x;         /* bf16 [T, H] */
  const void* residual;  /* bf16 [T, H] or NULL; when set h = x + residual is normalised */
  const void* weight;    /* bf16 [H] or NULL */
  const void* bias;      /* bf16 [H] or NULL (LayerNorm only) */
  void* out;             /* bf16 [T, H] normalised */
  void* residual_out;    /* bf16 [T, H] or NULL: receives h */
  int* err;
  int T, H;
  float eps;
  int kind;              /* 0 = RMSNorm, 1 = LayerNorm (mean-subtracting) */
  int weight_offset_one; /* Gemma: scale by (1 + w) */
  /* F1 consumer: sum `rs_world` partial slots [world][T][H] before the residual add (x is then the slot base). */
  int rs_world;
  const uint32_t* rs_flag;       /* local counter bumped by producers */
  const uint32_t* epoch;         /* unused */
  uint32_t rs_signals_per_use;
  /* F3 producer: also push the normalised row into every peer's gather buffer at row (ag_rank*T + t). */
  int ag_world, ag_rank;
  void* ag_peer_out[UB_MAX_RANKS];
  uint32_t* ag_peer_flag[UB_MAX_RANKS]; /* peer's counter for source `ag_rank` */
  /* up to 32 consecutive local counters that are idle during this kernel: block 0 zeroes them first */
  uint32_t* reset_flags;
  int reset_count;
  /* F3 producer: a zeroed u32 in LOCAL memory on which the row CTAs arrive; the last one bumps every ag_peer_flag
     once (the consumer waits for one arrival per source rank).  Required when ag_world > 0. */
  uint32_t* ag_local_count;
  /* NVSwitch multicast variants (addresses inside the multicast mapping of a symmetric heap, see csrc/comm/symm_heap.cu):
     rs_multimem = 1: x is the MULTICAST address of this rank's rows inside a [world * T, H] buffer in which every rank
     holds its own partial result at the same offset; the rows are read with multimem.ld_reduce (summed in the switch,
     fp32 accumulation) instead of summing rs_world local slots.
     ag_mc_out != NULL: the normalised row goes to row (ag_rank * T + t) of this multicast address with ONE multimem.st
     (the switch replicates it to every rank) instead of ag_world peer stores; ag_peer_out is then unused. */
  int rs_multimem;
  void* ag_mc_out;
} UbNormArgs;
int ub_norm(const UbNormArgs* args, void* stream);

/* ---------------- K6 : (q/k head RMSNorm) + RoPE + paged KV append ---------------- */
typedef struct UbRopeArgs {
  void* qkv;                 /* bf16 [T, (Hq + 2 Hkv) * D]; q and k are rotated in place */
  const int* positions;      /* [T] */
  const int* slot_mapping;   /* [T] flat slot = block * block_size + offset, or -1 to skip the append */
  void* k_cache;             /* bf16 [num_blocks, Hkv, block_size, D] */
  void* v_cache;
  const void* q_norm_w;      /* bf16 [D] or NULL */
  const void* k_norm_w;      /* bf16 [D] or NULL */
  int* err;
  int T, Hq, Hkv, D;
  int rotary_dim;            /* <= D, even; 0 disables rotation */
  int block_size;
  long long num_slots;       /* num_blocks * block_size, for the bounds check */
  float theta;
  float pos_scale;           /* linear RoPE scaling: position * pos_scale (1 = none) */
  float norm_eps;
  int interleaved;           /* 0 = half-split pairs (i, i + rd/2); 1 = adjacent pairs (2i, 2i+1) */
  /* Llama-3 style frequency scaling; factor <= 0 disables */
  float l3_factor, l3_low_freq_factor, l3_high_freq_factor, l3_orig_ctx;
} UbRopeArgs;
int ub_rope_kv_append(const UbRopeArgs* args, void* stream);

/* ---------------- K3 / K4 : paged attention ---------------- */
typedef struct UbAttnArgs {
  const void* q;             /* bf16 [T, Hq, D] with row stride q_stride elements */
  const void* k_cache;       /* bf16 [num_blocks, Hkv, block_size, D] */
  const void* v_cache;
  void* out;                 /* bf16 [T, Hq, D] row stride o_stride */
  float* lse;                /* fp32 [T, Hq] or NULL (natural-log sum-exp of scaled scores) */
  const int* block_tables;   /* [num_seqs, max_blocks_per_seq] */
  const int* seq_lens;       /* [num_seqs] kv length visible to the LAST query token of the sequence */
  const int* q_start;        /* [num_seqs + 1] prefix sums of query tokens (prefill); NULL for decode (1 per seq) */
  const float* alibi_slopes; /* [Hq] or NULL */
  float* scratch;            /* decode split-KV partials: [num_seqs, Hq, splits, D + 2] fp32, or NULL when splits == 1 */
  int* err;
  int num_seqs, Hq, Hkv, D;
  int block_size, max_blocks_per_seq, num_blocks;
  long long q_stride, o_stride;
  float scale;
  int causal;                /* prefill: 1 = causal (query i sees kv <= kv_len - q_len + i), 0 = bidirectional */
  int window;                /* > 0: sliding window (query sees at most `window` latest keys) */
  int splits;                /* decode: number of KV splits per sequence */
  int kv_start;              /* first kv position to attend (suffix attention after a shared prefix); 0 = all */
  int total_q;               /* prefill: total query tokens */
  int max_q_len;             /* prefill: max query tokens in one sequence (grid sizing) */
  /* Optional partial result over a DISJOINT key set (e.g. a shared prefix), merged into the output by the kernel
     itself: merge_o bf16 [T, Hq, D] contiguous and merge_lse fp32 [T, Hq].  Supported by the tensor-core prefill kernel
     and the warp-MMA decode kernel with splits == 1; other paths answer -7. */
  const void* merge_o;
  const float* merge_lse;
} UbAttnArgs;
int ub_attn_decode(const UbAttnArgs* args, void* stream);
int ub_attn_prefill(const UbAttnArgs* args, void* stream);
/* merge two partial attention results (o_a, lse_a) and (o_b, lse_b) -> out; rows = T*Hq, D columns */
int ub_attn_merge(const void* o_a, const float* lse_a, const void* o_b, const float* lse_b, void* out, float* lse_out,
                  long long rows, int D, void* stream);

/* ---------------- K8 : sampling ---------------- */
typedef struct UbSampleArgs {
  const void* logits;        /* bf16 or fp32 [B, V] row stride ld */
  long long ld;
  int logits_f32;
  int* out_ids;              /* [B] */
  float* out_vals;           /* [B] or NULL: winning (max) logit, used for the vocab-parallel merge */
  const float* temperature;  /* [B] or NULL (=> greedy) ; <= 0 means greedy for that row */
  const float* top_p;        /* [B] or NULL */
  const int* top_k;          /* [B] or NULL ; <= 0 means no limit (capped at 1024 internally when top_p < 1) */
  const float* rep_penalty;  /* [B] or NULL */
  const int* prev_ids;       /* [B, prev_ld] token history for the repetition penalty (-1 padded) or NULL */
  int prev_ld;
  unsigned long long seed;
  unsigned long long step;   /* Philox offset; same (seed, step, row) gives the same draw on every rank */
  int B, V;
  int vocab_offset;          /* added to the returned ids (vocab-parallel shards) */
  int* err;
  /* Vocabulary-parallel sampling in two stages.  Stage 1 (cand_vals != NULL, on every shard): instead of drawing, the
     row's best min(k, cand_k) entries after penalty and temperature go to cand_vals / cand_ids [B, cand_k] (value
     descending, global id = index + vocab_offset, unused slots -inf / -1); rows need top_k > 0 or top_p < 1.
     Stage 2 (id_map != NULL, identical on every rank): `logits` holds the gathered fp32 candidates [B, V = world * cand_k]
     (already scaled), id_map [B, ld] their global ids: top-k / top-p / draw as usual, out_ids = id_map[picked]. */
  float* cand_vals;
  int* cand_ids;
  int cand_k;
  const int* id_map;
  /* Vocabulary-parallel draw from the WHOLE vocabulary (temperature only), again in two stages.  stats_out != NULL: no
     draw; stats_out[2 * row] = the shard's largest scaled logit, [2 * row + 1] = sum of exp(logit - that maximum).
     target_in != NULL: the inverse-CDF target for this shard in the same units (a negative value = another shard owns
     the draw: out_ids = -1, out_vals = -inf; otherwise out_vals = 1). */
  float* stats_out;
  const float* target_in;
} UbSampleArgs;
int ub_sample(const UbSampleArgs* args, void* stream);
/* One-shot all-gather of (value, id) pairs through peer memory: every rank contributes `rows` x `k` pairs; row s of
   out_vals / out_ids ([rows, world * k], local) receives the ranks' pairs in rank order.  Same protocol as the one-shot
   all-reduce (parity slots, one arrival counter per CTA, bounded waits, exchange number in a device word). */
typedef struct UbPairGatherArgs {
  const float* vals;          /* [rows, k] */
  const int* ids;
  float* out_vals;            /* [rows, world * k] */
  int* out_ids;
  void* peer_vals[UB_MAX_RANKS];   /* per rank: fp32 [2][cap pairs * world] receive slots */
  void* peer_ids[UB_MAX_RANKS];
  uint32_t* peer_flags[UB_MAX_RANKS];
  const float* my_vals;
  const int* my_ids;
  const uint32_t* my_flags;
  uint32_t* round;
  uint32_t* done_count;
  int world, rank, rows, k;
  long long cap;              /* pairs per rank the slots can hold (rows * k <= cap) */
  int* err;
  uint32_t* cta_rounds;       /* local, UB_AR_MAX_CTAS words: exchanges each CTA index has taken part in */
} UbPairGatherArgs;
int ub_pair_gather_oneshot(const UbPairGatherArgs* args, void* stream);
/* vals/ids [world, B] per-shard greedy winners -> out_ids [B]; lowest id wins ties. */
int ub_argmax_merge(const float* vals, const int* ids, int world, int B, int* out_ids, void* stream);

/* ---------------- K9 / K10 / misc element-wise ---------------- */
int ub_embed_gather(const int* ids, const void* table, void* out, int T, int H, int V, float scale, int* err,
                    void* stream);
int ub_act_mul(const void* gate_up, void* out, long long T, int I, int act, void* stream); /* out = act(g)*u ; gate_up [T, 2I] */
int ub_eltwise(const void* x, void* out, long long n, int act, float alpha, void* stream);  /* out = act(alpha * x) */
int ub_add(const void* a, const void* b, void* out, long long n, float sa, float sb, void* stream);
int ub_l2_normalize(const void* x, void* out, int T, int H, float eps, void* stream);
int ub_softmax_rows(const void* x, void* out, long long rows, int n, void* stream);   /* bf16, softmax over the last dim */

/* ---------------- K7 / K13 : MoE ---------------- */
typedef struct UbMoeRouteArgs {
  const void* logits;       /* bf16 or fp32 [T, E] router logits; ignored when router_w is set */
  const void* x;            /* bf16 [T, H] activations (router_w mode) */
  const void* router_w;     /* bf16 [E, H] or NULL: the kernel computes logits = x router_w^T itself */
  int* topk_ids;            /* [T, K] */
  float* topk_w;            /* [T, K] */
  int* expert_counts;       /* [E] */
  int* expert_offsets;      /* [E+1] exclusive prefix sums */
  int* sorted_rows;         /* [T*K] source row (t*K + k) for each expert-sorted slot */
  int* row_slot;            /* [T*K] inverse permutation */
  void* tiles;              /* int4[max_tiles] token-tile table for the grouped GEMM, or NULL */
  int* err;
  int logits_f32;
  int T, E, K, H;
  int norm_topk;            /* 1: softmax over the K selected (Mixtral); 0: softmax over all E, no renormalisation */
  int round_logits_bf16;    /* router_w mode: round logits to bf16 first (what a bf16 linear layer produces) */
  float weight_scale;       /* multiplies the routing weights (0 = 1) */
  int tile_tokens;          /* token tile of the grouped GEMM that will consume `tiles` */
  int max_tiles;            /* capacity of `tiles`; ceil(T*K / tile_tokens) + E always suffices */
  /* Expert parallelism: this rank owns experts [expert_lo, expert_lo + num_local_experts).  Pairs routed elsewhere
     get row_slot = -1 and no tile; expert_counts/offsets/tiles use local expert indices.  0 = all experts local. */
  int expert_lo;
  int num_local_experts;
} UbMoeRouteArgs;
int ub_moe_route(const UbMoeRouteArgs* args, void* stream);
int ub_moe_gather(const void* x, const int* sorted_rows, void* out, int rows, int K, int H, void* stream);
int ub_moe_combine(const void* y, const int* row_slot, const float* topk_w, const void* residual, void* out, int T,
                   int K, int H, void* stream);
/* F6: combine fused with the reduce-scatter: token t's partial row is stored into the receive slot
   peer_out[owner(t)][rank][t - owner*rows_per_rank]; the CTAs arrive on the zeroed LOCAL counter local_count and the
   last one bumps every peer's counter once.  With null peer_out entries the rows go to local_out[t] instead (this
   rank's partial buffer inside a multicast-bound heap; the owners read them summed by the switch). */
int ub_moe_combine_num_ctas(int T, int H);
int ub_moe_combine_rs(const void* y, const int* row_slot, const float* topk_w, int T, int K, int H, int world, int rank,
                      int rows_per_rank, void* const* peer_out, uint32_t* const* peer_flag, uint32_t* local_count,
                      void* local_out, void* stream);

/* F5 / F6: sparse expert-parallel dispatch / combine over peer memory (csrc/moe/moe.cu).  Rank r owns token rows
   [r * R, (r + 1) * R) and experts [r * experts_local, (r + 1) * experts_local); cap = R * K rows per source region. */
typedef struct UbMoeDispatchArgs {
  const void* x;                     /* bf16 [R, H]: this rank's rows */
  const int* topk_ids;               /* [R, K] global expert ids (ub_moe_route on the R rows) */
  const float* topk_w;               /* [R, K] */
  int* send_slot;                    /* scratch [R * K] */
  int* send_counts;                  /* scratch [E] */
  void* peer_rows[UB_MAX_RANKS];     /* per rank: bf16 [world][cap][H] receive rows */
  void* peer_meta[UB_MAX_RANKS];     /* per rank: int4 [world][cap] (global pair id, local expert, weight bits, 0) */
  int* peer_counts[UB_MAX_RANKS];    /* per rank: int [world][experts_local] rows sent per (source, local expert) */
  uint32_t* peer_flag[UB_MAX_RANKS]; /* per rank: arrival counter of the dispatch (monotonic, one per source and use) */
  uint32_t* local_count;             /* zeroed local word: arrival counter of this launch's CTAs */
  int* err;
  int R, K, H, E, world, rank, experts_local, cap;
} UbMoeDispatchArgs;
int ub_moe_dispatch(const UbMoeDispatchArgs* args, void* stream);

typedef struct UbMoeRecvArgs {
  const int* counts;                 /* local [world][experts_local] */
  const void* meta;                  /* local int4 [world][cap] */
  const uint32_t* flag;              /* local arrival counter; expects `world` more arrivals per use */
  uint32_t* round;                   /* local word: uses so far (advanced by the kernel, so the launch can sit in a graph) */
  int* sorted_rows;                  /* out [world * cap]: receive row of each expert-ordered slot, -1 past the end */
  void* slot_meta;                   /* out int4 [world * cap]: (global pair id, owner rank, weight bits, 0) per slot */
  int* expert_counts;                /* out [experts_local] */
  int* expert_offsets;               /* out [experts_local + 1] */
  void* tiles;                       /* out int4 [max_tiles]: tile table of the grouped GEMM */
  int* err;
  int world, experts_local, cap, tile_tokens, max_tiles;
} UbMoeRecvArgs;
int ub_moe_recv_build(const UbMoeRecvArgs* args, void* stream);

typedef struct UbMoeReturnArgs {
  const void* y;                     /* bf16 [slots, H] expert outputs in slot order */
  const void* slot_meta;
  const int* expert_offsets;         /* [experts_local + 1]; the last entry is the number of rows */
  void* peer_comb[UB_MAX_RANKS];     /* per rank: bf16 [K][R][H] combine area, summed by the owner's norm kernel */
  uint32_t* peer_flag[UB_MAX_RANKS];
  uint32_t* local_count;
  int* err;
  int R, K, H, world, experts_local;
} UbMoeReturnArgs;
int ub_moe_combine_push(const UbMoeReturnArgs* args, int max_slots, void* stream);

/* ---------------- K12 : GGUF-quantised weights ---------------- */
/* qtype is the ggml type id: 2 Q4_0, 3 Q4_1, 6 Q5_0, 8 Q8_0, 12 Q4_K, 14 Q6_K. */
int ub_dequant(const void* blocks, void* out_bf16, long long n_elems, int qtype, void* stream);
/* out[M,N] (bf16) = x[M,K] (bf16) @ dequant(w[N,K])^T for M <= 8 without materialising w. */
int ub_qgemv(const void* blocks, const void* x, void* out, int M, int N, int K, int qtype, void* stream);

/* ---------------- K14-K17, K15 : recurrences of the O(1)-state models ----------------
   Activations are bf16 [B, L, C] (channel last); parameters and states are fp32 unless noted.  A NULL state means
   "start from zero and do not store".  L = prompt length for prefill, 1 for decode. */
/* state: bf16 [B, Kw-1, C], the inputs before this call; updated to the last Kw-1 inputs when update_state. */
int ub_causal_dwconv1d(const void* x, const float* w /*[C,Kw]*/, const float* b /*[C] or NULL*/, void* out, void* state, int B,
                       int L, int C, int Kw, int act_silu, int update_state, void* stream);
/* A [Dm,Ns], Bm/Cm bf16 [B,L,Ns], Dv [Dm] or NULL, z bf16 [B,L,Dm] or NULL (gate: y *= silu(z)), state [B,Dm,Ns]. */
int ub_selective_scan(const void* u, const void* delta, const float* A, const void* Bm, const void* Cm, const float* Dv,
                      const void* z, void* out, float* state, int B, int L, int Dm, int Ns, int delta_softplus,
                      float* workspace, void* stream);
/* h = a*h + (one_minus ? 1-a : 1)*x;  a is [C] or, with a_per_step, [B,L,C];  state [B,C]. */
int ub_linear_recurrence(const float* a, int a_per_step, const void* x, void* out, float* state, int B, int L, int C,
                         int one_minus, float* workspace, void* stream);
/* w = -exp(time_decay) [C], u = time_first [C], state [B,3,C] = (aa, bb, pp), fresh sequences start at (0, 0, -1e38). */
int ub_wkv4(const void* k, const void* v, const float* w, const float* u, void* out, float* state, int B, int L, int C,
            float* workspace, void* stream);
/* w fp32 [B,L,H*Dh] pre-activation decay (decay = exp(-exp(w))), u [H*Dh], state [B,H,Dh,Dh]; Dh = 64 or 32. */
int ub_wkv6(const void* r, const void* k, const void* v, const float* w, const float* u, void* out, float* state, int B,
            int L, int H, int Dh, float* workspace, void* stream);
/* Long sequences run the four scans above in chunks that proceed in parallel (a summary pass, a short carry over the
   chunks, an output pass).  That needs `workspace` (fp32, ub_scan_workspace_floats elements; kind: 0 selective scan
   (n = Dm, m = Ns), 1 linear recurrence (n = C), 2 WKV-4 (n = C), 3 WKV-6 (n = H, m = Dh)); with a NULL workspace, or a
   sequence for which ub_scan_chunks answers 1, the single sequential pass runs. */
int ub_scan_chunks(int L);
long long ub_scan_workspace_floats(int kind, int B, int L, int n, int m);

/* ---------------- comm helpers ---------------- */
int ub_bump_epoch(uint32_t* epoch, void* stream);
/* One-shot all-reduce for small messages: every rank pushes its vector into each peer's slot, then sums.  May run in
   place (out == in). */
#define UB_AR_MAX_CTAS 64
typedef struct UbAllReduceArgs {
  const void* in;           /* bf16 [n] local */
  void* out;                /* bf16 [n] */
  void* peer_slots[UB_MAX_RANKS];     /* each: [2][world][max_n] bf16 on that peer (two slot sets, by exchange parity) */
  uint32_t* peer_flags[UB_MAX_RANKS]; /* each: UB_AR_MAX_CTAS counters on that peer (one per CTA index) */
  const void* my_slots;     /* local [2][world][max_n] */
  const uint32_t* my_flags; /* local counters */
  uint32_t* round;          /* local device word: number of exchanges completed (advanced by the kernel) */
  uint32_t* done_count;     /* local device word, zero between launches */
  int world, rank;
  long long n;
  int* err;
  uint32_t* cta_rounds;     /* local, UB_AR_MAX_CTAS words: exchanges each CTA index has taken part in (grids vary with n) */
  long long max_n;          /* elements per rank slot (capacity); n <= max_n */
} UbAllReduceArgs;
int ub_allreduce_oneshot_ctas(long long n);
int ub_allreduce_oneshot(const UbAllReduceArgs* args, void* stream);
/* F4: merge per-shard greedy winners across tensor-parallel ranks over peer memory (see csrc/comm/comm.cu). */
typedef struct UbArgmaxMergeArgs {
  const float* vals;         /* [rows] best logit of this rank's vocabulary shard */
  const int* ids;            /* [rows] its global token id */
  int* out_ids;              /* [rows] global winners */
  void* peer_vals[UB_MAX_RANKS];   /* each: float [2][world][max_rows] on that peer */
  void* peer_ids[UB_MAX_RANKS];    /* each: int   [2][world][max_rows] */
  uint32_t* peer_flags[UB_MAX_RANKS];
  const float* my_vals;
  const int* my_ids;
  const uint32_t* my_flag;
  uint32_t* round;           /* local device word, incremented by the kernel */
  int world, rank, rows, max_rows;
  int* err;
} UbArgmaxMergeArgs;
int ub_tp_argmax_merge(const UbArgmaxMergeArgs* args, void* stream);
/* Wait until *flag (u32, wrap-safe) >= value; bounded (about 1 s), writes status 2 to err on timeout. */
int ub_wait_flag(const uint32_t* flag, uint32_t value, int* err, void* stream);
/* Same for n (<= 32) consecutive counters, one thread each. */
int ub_wait_flags(const uint32_t* flags, int n, uint32_t value, int* err, void* stream);

/* ---------------- symmetric heap + multicast (csrc/comm/symm_heap.cu) ---------------- */
const char* ub_symm_error(void);
int ub_symm_supported(int dev, int* vmm, int* multicast);
int ub_symm_round_size(unsigned long long bytes, int dev, int world, unsigned long long* out);
int ub_symm_alloc(unsigned long long bytes, int dev, unsigned long long* handle, int* fd, void** va);
int ub_symm_map_peer(int fd, unsigned long long bytes, int dev, unsigned long long* handle, void** va);
int ub_symm_unmap(void* va, unsigned long long bytes, unsigned long long handle);
int ub_symm_mc_create(unsigned long long bytes, int world, unsigned long long* mc, int* fd);
int ub_symm_mc_import(int fd, unsigned long long* mc);
int ub_symm_mc_add_device(unsigned long long mc, int dev);
int ub_symm_mc_bind(unsigned long long mc, unsigned long long local_handle, unsigned long long bytes);
int ub_symm_mc_map(unsigned long long mc, unsigned long long bytes, int dev, void** va);
int ub_symm_mc_release(unsigned long long mc, void* mc_va, unsigned long long bytes, int dev);
/* One copy kernel for bandwidth probes: kind 0 plain copy (peer mappings allowed), 1 multimem.st, 2 multimem.ld_reduce. */
int ub_symm_probe(int kind, const void* src, void* dst, long long bytes, int ctas, void* stream);

/* ---------------- device memory backend (kv/gpu_memory FFI surface) ---------------- */
int ub_cuda_device_count(void);
int ub_cuda_set_device(int dev);
int ub_cuda_malloc_aligned(void** ptr, unsigned long long bytes, unsigned long long align);
int ub_cuda_free(void* ptr);
int ub_cuda_malloc_host(void** ptr, unsigned long long bytes);
int ub_cuda_free_host(void* ptr);
int ub_cuda_memcpy_h2d_async(void* dst, const void* src, unsigned long long bytes, void* stream);
int ub_cuda_memcpy_d2h_async(void* dst, const void* src, unsigned long long bytes, void* stream);
int ub_cuda_memcpy_d2d_async(void* dst, const void* src, unsigned long long bytes, void* stream);
int ub_cuda_stream_create(void** stream);
int ub_cuda_stream_destroy(void* stream);
int ub_cuda_stream_synchronize(void* stream);
int ub_cuda_device_synchronize(void);
int ub_cuda_mem_info(unsigned long long* free_b, unsigned long long* total_b);
typedef struct UbDeviceProps {
  char name[128];
  unsigned long long total_mem;
  int sm_count, cc_major, cc_minor, max_smem_per_block, l2_bytes, clock_khz, mem_clock_khz, mem_bus_bits;
} UbDeviceProps;
int ub_cuda_device_props(int dev, UbDeviceProps* out);
const char* ub_cuda_error_string(int code);

#ifdef __cplusplus
}
#endif
#endif
