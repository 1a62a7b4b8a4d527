"""Torch-tensor front end of the sm_100a kernel library.

Every function launches on the current CUDA stream of the tensors' device and returns torch
tensors; none of them synchronises.  Arguments are checked on the host (dtype, contiguity,
alignment) so that a bad call raises in Python instead of faulting on the device.  The kernels
record device-side problems (timeouts of bounded waits, out-of-range block-table entries) in a
per-device error word that :func:`check_device_errors` reads.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Sequence

import torch

from . import _native as N
from . import _native as N_

_err_words: dict[int, torch.Tensor] = {}


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def err_word(device) -> torch.Tensor:
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    w = _err_words.get(idx)
    if w is None:
        w = torch.zeros(2, dtype=torch.int32, device=f"cuda:{idx}")
        _err_words[idx] = w
    return w


def check_device_errors(device=None, reset: bool = True) -> None:
    """Synchronises and raises if any kernel recorded an error since the last check."""
    devs = [torch.device(device)] if device is not None else [torch.device(f"cuda:{i}") for i in _err_words]
    for d in devs:
        w = err_word(d)
        code, detail = w.tolist()
        if code != 0:
            if reset:
                w.zero_()
                gemm_streamk_reset(d)
            names = {1: "mbarrier wait timed out", 2: "flag wait timed out (peer or producer missing)",
                     3: "index out of range", 4: "bad argument"}
            raise RuntimeError(f"device error {code} ({names.get(code, '?')}), detail {detail} on {d}")


def gemm_streamk_reset(device=None) -> None:
    """Lowers the flags of the GEMM's stream-K workspace (after a step that reported a timed-out wait)."""
    with torch.cuda.device(torch.device(device) if device is not None else torch.cuda.current_device()):
        N_.cuda_lib().ub_gemm_streamk_reset(C.c_void_p(torch.cuda.current_stream().cuda_stream))


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _bf16c(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16, got {t.dtype}")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")


# ---------------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------------
def gemm_tn(x: torch.Tensor, w: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
            residual: Optional[torch.Tensor] = None, act: Optional[str] = None, out: Optional[torch.Tensor] = None,
            out_dtype: torch.dtype = torch.bfloat16, out_scale: float = 1.0, tile_tokens: int = 0, splits: int = 0,
            dual_rows: int = 0, rs: Optional[dict] = None, ag: Optional[dict] = None,
            grouped: Optional[dict] = None, cta_pair: int = 0, pair_splits: int = 0) -> torch.Tensor:
    """``out[M, N] = act(x[M, K] @ w[N, K]^T * out_scale + bias) + residual`` on tcgen05 tensor cores.

    ``dual_rows = I`` switches to the gated form: ``w`` is ``[2*I, K]`` with gate rows first and the
    result is ``act(x @ w[:I]^T) * (x @ w[I:]^T)`` of shape ``[M, I]``.
    ``rs`` / ``ag`` carry the peer pointers for the fused reduce-scatter / all-gather variants (see
    :mod:`unillm_b200.dist.fused`).
    """
    _bf16c(x, "x"), _bf16c(w, "w")
    if x.dim() != 2 or w.dim() != 2:
        raise ValueError("gemm_tn takes 2-D operands")
    if x.stride(1) != 1 or w.stride(1) != 1:
        raise ValueError("operands must be K-contiguous")
    M, K = x.shape
    if w.shape[1] != K:
        raise ValueError(f"K mismatch: x {tuple(x.shape)} vs w {tuple(w.shape)}")
    dual = dual_rows > 0
    Nn = dual_rows if dual else w.shape[0]
    if dual and w.shape[0] < 2 * dual_rows:
        raise ValueError("dual GEMM needs w with 2*I rows")
    if out is None:
        out = torch.empty((M, Nn), dtype=out_dtype, device=x.device)
    if out.stride(-1) != 1:
        raise ValueError("out must be row-major")
    a = N.UbGemmArgs()
    a.x, a.w, a.out = x.data_ptr(), w.data_ptr(), out.data_ptr()
    a.bias = _p(bias)
    a.residual = _p(residual)
    a.err = err_word(x.device).data_ptr()
    a.M, a.N, a.K = M, Nn, K
    a.ldx, a.ldw, a.ldo = x.stride(0), w.stride(0), out.stride(0)
    a.ldr = residual.stride(0) if residual is not None else 0
    a.act = N.ACT[act]
    a.dual = 1 if dual else 0
    a.up_row_off = dual_rows
    a.w_rows_total = w.shape[0]
    a.out_f32 = 1 if out.dtype == torch.float32 else 0
    a.out_scale = out_scale
    a.tile_tokens = tile_tokens
    a.splits = splits
    a.cta_pair = cta_pair
    a.pair_splits = pair_splits
    if bias is not None:
        _bf16c(bias, "bias")
    if residual is not None:
        _bf16c(residual, "residual")
    if rs is not None:
        a.rs_world, a.rs_rank, a.rs_rows_per_rank = rs["world"], rs["rank"], rs["rows_per_rank"]
        for i in range(rs["world"]):
            a.rs_peer_out[i] = rs["peer_out"][i]
            a.rs_peer_flag[i] = rs["peer_flag"][i]
        a.rs_local_count = rs["local_count"]
    if ag is not None:
        a.ag_world, a.ag_rows_per_rank = ag["world"], ag["rows_per_rank"]
        a.ag_flags, a.ag_signals_per_use = ag["flags"], ag["signals_per_use"]
    if grouped is not None:
        a.grp_tiles, a.grp_max_tiles, a.grp_w_rows = grouped["tiles"], grouped["max_tiles"], grouped["w_rows"]
        a.tile_tokens = grouped["tile_tokens"]
    N.check(N.cuda_lib().ub_gemm_tn(C.byref(a), _stream(x)), "ub_gemm_tn")
    return out


def gemm_num_ctas(M: int, N: int, K: int, dual: bool = False, tile_tokens: int = 0, splits: int = 0, cta_pair: int = 0) -> int:
    """CTAs that ``gemm_tn`` launches for this problem (each signals every peer once in reduce-scatter mode)."""
    a = N_.UbGemmArgs()
    a.M, a.N, a.K, a.dual, a.tile_tokens, a.splits, a.cta_pair = M, N, K, int(dual), tile_tokens, splits, cta_pair
    return N_.cuda_lib().ub_gemm_num_ctas(C.byref(a))


def wait_flags(flags_ptr: int, n: int, value: int, device) -> None:
    """Enqueue a one-block kernel that waits (bounded) until n consecutive u32 counters reach ``value``."""
    lib = N_.cuda_lib()
    lib.ub_wait_flags.restype = C.c_int
    lib.ub_wait_flags.argtypes = [N_.vp, N_.i32, N_.u32, N_.vp, N_.vp]
    N_.check(lib.ub_wait_flags(flags_ptr, n, value, err_word(device).data_ptr(),
                               torch.cuda.current_stream(device).cuda_stream), "ub_wait_flags")


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, **kw) -> torch.Tensor:
    """``x[..., K] @ w[N, K]^T`` for any leading shape."""
    lead = x.shape[:-1]
    y = gemm_tn(x.reshape(-1, x.shape[-1]), w, bias=bias, **kw)
    return y.reshape(*lead, y.shape[-1])


# ---------------------------------------------------------------------------------------------
# Norm
# ---------------------------------------------------------------------------------------------
def norm(x: torch.Tensor, weight: Optional[torch.Tensor], *, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, eps: float = 1e-5, kind: str = "rms",
         weight_offset_one: bool = False, want_residual_out: bool = False,
         out: Optional[torch.Tensor] = None, residual_out: Optional[torch.Tensor] = None,
         rs: Optional[dict] = None, ag: Optional[dict] = None, T: Optional[int] = None,
         reset: Optional[tuple] = None, no_out: bool = False, x_ptr: Optional[int] = None):
    """RMSNorm / LayerNorm over the last dim, with optional fused ``x + residual``.

    Returns ``y`` or ``(y, h)`` when the residual stream ``h = x + residual`` is requested.
    """
    _bf16c(x, "x")
    H = x.shape[-1]
    if T is None:
        T = x.numel() // H
    if not x.is_contiguous():
        x = x.contiguous()
    if out is None and not no_out:
        out = torch.empty((T, H), dtype=torch.bfloat16, device=x.device)
    if want_residual_out and residual_out is None:
        residual_out = torch.empty((T, H), dtype=torch.bfloat16, device=x.device)
    a = N.UbNormArgs()
    a.x, a.residual, a.weight, a.bias = (x.data_ptr() if x_ptr is None else x_ptr), _p(residual), _p(weight), _p(bias)
    a.out, a.residual_out = _p(out), _p(residual_out)
    a.err = err_word(x.device).data_ptr()
    a.T, a.H, a.eps = T, H, eps
    a.kind = 0 if kind == "rms" else 1
    a.weight_offset_one = 1 if weight_offset_one else 0
    if rs is not None:
        a.rs_world, a.rs_flag, a.rs_signals_per_use = rs["world"], rs["flag"], rs["signals_per_use"]
        if rs.get("multimem_x"):
            a.x, a.rs_multimem = rs["multimem_x"], 1       # multicast address of this rank's rows of the partial buffer
    if reset is not None:
        a.reset_flags, a.reset_count = reset
    if ag is not None:
        a.ag_world, a.ag_rank = ag["world"], ag["rank"]
        for i in range(ag["world"]):
            a.ag_peer_out[i] = ag["peer_out"][i]
            a.ag_peer_flag[i] = ag["peer_flag"][i]
        a.ag_local_count = ag["local_count"]
        a.ag_mc_out = ag.get("mc_out") or None
    N.check(N.cuda_lib().ub_norm(C.byref(a), _stream(x)), "ub_norm")
    if residual_out is not None:
        return out, residual_out
    return out


# ---------------------------------------------------------------------------------------------
# RoPE + KV append
# ---------------------------------------------------------------------------------------------
def rope_kv_append(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                   k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], *, num_q_heads: int,
                   num_kv_heads: int, head_dim: int, rotary_dim: Optional[int] = None, theta: float = 10000.0,
                   pos_scale: float = 1.0, interleaved: bool = False, q_norm_w: Optional[torch.Tensor] = None,
                   k_norm_w: Optional[torch.Tensor] = None, norm_eps: float = 1e-6,
                   llama3_scaling: Optional[Sequence[float]] = None) -> torch.Tensor:
    """Rotates q and k inside ``qkv`` [T, (Hq+2Hkv)*D] in place and appends k, v to the paged cache."""
    _bf16c(qkv, "qkv")
    if not qkv.is_contiguous():
        raise ValueError("qkv must be contiguous")
    T = qkv.shape[0]
    if positions.dtype != torch.int32 or (slot_mapping is not None and slot_mapping.dtype != torch.int32):
        raise TypeError("positions / slot_mapping must be int32")
    a = N.UbRopeArgs()
    a.qkv, a.positions, a.slot_mapping = qkv.data_ptr(), positions.data_ptr(), _p(slot_mapping)
    a.k_cache, a.v_cache = _p(k_cache), _p(v_cache)
    a.q_norm_w, a.k_norm_w = _p(q_norm_w), _p(k_norm_w)
    a.err = err_word(qkv.device).data_ptr()
    a.T, a.Hq, a.Hkv, a.D = T, num_q_heads, num_kv_heads, head_dim
    a.rotary_dim = head_dim if rotary_dim is None else rotary_dim
    if k_cache is not None:
        a.block_size = k_cache.shape[2]
        a.num_slots = k_cache.shape[0] * k_cache.shape[2]
    else:
        a.block_size, a.num_slots = 16, 0
        a.slot_mapping = None
    a.theta, a.pos_scale, a.norm_eps = theta, pos_scale, norm_eps
    a.interleaved = 1 if interleaved else 0
    if llama3_scaling is not None:
        a.l3_factor, a.l3_low_freq_factor, a.l3_high_freq_factor, a.l3_orig_ctx = llama3_scaling
    N.check(N.cuda_lib().ub_rope_kv_append(C.byref(a), _stream(qkv)), "ub_rope_kv_append")
    return qkv


# ---------------------------------------------------------------------------------------------
# Attention
# ---------------------------------------------------------------------------------------------
def _attn_args(q, k_cache, v_cache, out, lse, block_tables, seq_lens, Hq, Hkv, D, scale):
    a = N.UbAttnArgs()
    a.q, a.k_cache, a.v_cache, a.out, a.lse = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _p(lse)
    a.block_tables, a.seq_lens = block_tables.data_ptr(), seq_lens.data_ptr()
    a.err = err_word(q.device).data_ptr()
    a.num_seqs, a.Hq, a.Hkv, a.D = seq_lens.shape[0], Hq, Hkv, D
    a.block_size, a.max_blocks_per_seq, a.num_blocks = k_cache.shape[2], block_tables.shape[1], k_cache.shape[0]
    a.q_stride, a.o_stride = q.stride(0), out.stride(0)
    a.scale = scale if scale is not None else 1.0 / math.sqrt(D)
    return a


def attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                seq_lens: torch.Tensor, *, scale: Optional[float] = None, window: int = 0, kv_start: int = 0,
                alibi_slopes: Optional[torch.Tensor] = None, splits: int = 0, scratch: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, return_lse: bool = False, lse: Optional[torch.Tensor] = None,
                max_seq_len: Optional[int] = None, merge: Optional[tuple] = None, kernel: Optional[str] = None):
    """One query token per sequence.  q: [B, Hq, D] (last two dims contiguous); caches [nb, Hkv, bs, D].

    ``kernel="warp"`` calls the warp-per-item kernel directly (page size 16, head size 64 / 128, ``splits == 1``, no
    window, no ALiBi) instead of going through the dispatcher's choice."""
    _bf16c(q, "q")
    B, Hq, D = q.shape
    Hkv = k_cache.shape[1]
    if out is None:
        out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=q.device)
    if return_lse and lse is None:
        lse = torch.empty((B, Hq), dtype=torch.float32, device=q.device)
    if splits <= 0:
        ctx = max_seq_len if max_seq_len is not None else block_tables.shape[1] * k_cache.shape[2]
        ctas = B * Hkv
        splits = 1
        while ctas * splits < 2 * 148 and ctx // (splits * 2) >= 256 and splits < 16:
            splits *= 2
    a = _attn_args(q, k_cache, v_cache, out, lse, block_tables, seq_lens, Hq, Hkv, D, scale)
    if splits > 1:
        need = B * Hq * splits * (D + 2)
        if scratch is None or scratch.numel() < need:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        a.scratch = scratch.data_ptr()
    a.window, a.splits, a.kv_start = window, splits, kv_start
    a.alibi_slopes = _p(alibi_slopes)
    if merge is not None:        # (o [B, Hq, D] bf16 contiguous, lse [B, Hq] fp32): partial over a disjoint key set
        a.merge_o, a.merge_lse = merge[0].data_ptr(), merge[1].data_ptr()
    if kernel == "warp":
        lib = N.cuda_lib()
        if not lib.ub_attn_decode_warp_supported(C.byref(a)):
            raise ValueError("attn_decode(kernel='warp'): page size 16, head size 64 / 128, one split, no window / ALiBi")
        N.check(lib.ub_attn_decode_warp(C.byref(a), _stream(q)), "ub_attn_decode_warp")
    else:
        N.check(N.cuda_lib().ub_attn_decode(C.byref(a), _stream(q)), "ub_attn_decode")
    return (out, lse) if return_lse else out


def attn_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                 seq_lens: torch.Tensor, q_start: torch.Tensor, max_q_len: int, *, scale: Optional[float] = None,
                 causal: bool = True, window: int = 0, kv_start: int = 0,
                 alibi_slopes: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 return_lse: bool = False, lse: Optional[torch.Tensor] = None, merge: Optional[tuple] = None,
                 kv_splits: int = 1, scratch: Optional[torch.Tensor] = None):
    """Ragged prefill: q [T, Hq, D]; sequence i owns query rows q_start[i]:q_start[i+1] and sees
    seq_lens[i] keys, its last query at kv position seq_lens[i]-1.

    ``kv_splits > 1`` (tensor-core kernel only, no ``merge``) divides every CTA's key tiles over that many CTAs and
    folds the partial results with a second small kernel: for launches with few query tiles and many keys, such as
    the shared-prefix pass of a tensor-parallel rank that holds one KV head.  ``scratch`` (fp32, at least
    :func:`attn_prefill_split_scratch_floats` elements) holds the partials."""
    _bf16c(q, "q")
    T, Hq, D = q.shape
    Hkv = k_cache.shape[1]
    if out is None:
        out = torch.empty((T, Hq, D), dtype=torch.bfloat16, device=q.device)
    if return_lse and lse is None:
        lse = torch.empty((T, Hq), dtype=torch.float32, device=q.device)
    a = _attn_args(q, k_cache, v_cache, out, lse, block_tables, seq_lens, Hq, Hkv, D, scale)
    a.q_start = q_start.data_ptr()
    a.causal, a.window, a.kv_start = (1 if causal else 0), window, kv_start
    a.total_q, a.max_q_len = T, max_q_len
    a.alibi_slopes = _p(alibi_slopes)
    if merge is not None:
        a.merge_o, a.merge_lse = merge[0].data_ptr(), merge[1].data_ptr()
    if kv_splits > 1:
        need = attn_prefill_split_scratch_floats(T, Hq, D, kv_splits)
        if scratch is None or scratch.numel() < need:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        if scratch.dtype != torch.float32:
            raise TypeError("scratch must be float32")
        a.splits, a.scratch = kv_splits, scratch.data_ptr()
    N.check(N.cuda_lib().ub_attn_prefill(C.byref(a), _stream(q)), "ub_attn_prefill")
    return (out, lse) if return_lse else out


def attn_prefill_split_scratch_floats(T: int, Hq: int, D: int, kv_splits: int) -> int:
    """fp32 elements of workspace that ``attn_prefill(kv_splits=...)`` needs: the log-sum-exps, then the bf16 rows."""
    lse = (kv_splits * T * Hq + 3) // 4 * 4
    return lse + (kv_splits * T * Hq * D + 1) // 2


def dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = False,
                    scale: Optional[float] = None) -> torch.Tensor:
    """Attention over dense tensors on the paged prefill kernels: ``q`` [B, Hq, Sq, D], ``k`` / ``v`` [B, Hkv, Sk, D]
    (bf16 CUDA, D = 64 or 128, Hq a multiple of Hkv) -> [B, Hq, Sq, D].  Keys and values are laid out as pages of 16
    positions with an identity block table, so bidirectional encoders (BERT, ViT, Whisper, CLIP), cross-attention and
    cached decoders share the kernels of the serving engine; with ``causal`` query i sees keys ``<= Sk - Sq + i``."""
    _bf16c(q, "q"), _bf16c(k, "k"), _bf16c(v, "v")
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    if D not in (64, 128) or Hq % Hkv:
        raise ValueError("dense_attention: head size 64 or 128, query heads a multiple of KV heads")
    nb = (Sk + 15) // 16
    pad = nb * 16 - Sk

    def pages(t):
        if pad:
            t = torch.nn.functional.pad(t, (0, 0, 0, pad))
        return t.reshape(B, Hkv, nb, 16, D).permute(0, 2, 1, 3, 4).reshape(B * nb, Hkv, 16, D).contiguous()

    kp, vp = pages(k), pages(v)
    bt = torch.arange(B * nb, dtype=torch.int32, device=q.device).view(B, nb)
    lens = torch.full((B,), Sk, dtype=torch.int32, device=q.device)
    qs = torch.arange(B + 1, dtype=torch.int32, device=q.device) * Sq
    qt = q.permute(0, 2, 1, 3).reshape(B * Sq, Hq, D).contiguous()
    out = attn_prefill(qt, kp, vp, bt, lens, qs, Sq, scale=scale, causal=causal)
    return out.view(B, Sq, Hq, D).permute(0, 2, 1, 3)


def softmax_rows(x: torch.Tensor) -> torch.Tensor:
    """Softmax over the last dimension of a bf16 CUDA tensor."""
    _bf16c(x, "x")
    x = x.contiguous()
    out = torch.empty_like(x)
    n = x.shape[-1]
    lib = N.cuda_lib()
    lib.ub_softmax_rows.restype = C.c_int
    lib.ub_softmax_rows.argtypes = [N.vp, N.vp, N.i64, N.i32, N.vp]
    N.check(lib.ub_softmax_rows(x.data_ptr(), out.data_ptr(), x.numel() // n, n, _stream(x)), "ub_softmax_rows")
    return out


def attn_prefill_last_path() -> str:
    """Which kernel the last ``attn_prefill`` call ran: ``"tcgen05"`` or ``"mma.sync"``."""
    lib = N.cuda_lib()
    lib.ub_attn_prefill_last_path.restype = C.c_int
    return {1: "tcgen05", 2: "mma.sync"}.get(lib.ub_attn_prefill_last_path(), "none")


def attn_merge(o_a: torch.Tensor, lse_a: torch.Tensor, o_b: torch.Tensor, lse_b: torch.Tensor,
               out: Optional[torch.Tensor] = None, lse_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Combine two attention partials over disjoint key sets.  o_*: [T, Hq, D] contiguous, lse_*: [T, Hq]."""
    if out is None:
        out = torch.empty_like(o_a)
    lib = N.cuda_lib()
    lib.ub_attn_merge.restype = C.c_int
    lib.ub_attn_merge.argtypes = [N.vp, N.vp, N.vp, N.vp, N.vp, N.vp, N.i64, N.i32, N.vp]
    rows = o_a.shape[0] * o_a.shape[1]
    N.check(lib.ub_attn_merge(o_a.data_ptr(), lse_a.data_ptr(), o_b.data_ptr(), lse_b.data_ptr(), out.data_ptr(),
                              _p(lse_out), rows, o_a.shape[-1], _stream(o_a)), "ub_attn_merge")
    return out


# ---------------------------------------------------------------------------------------------
# Sampling
# ---------------------------------------------------------------------------------------------
def sample(logits: torch.Tensor, *, temperature: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           top_k: Optional[torch.Tensor] = None, rep_penalty: Optional[torch.Tensor] = None,
           prev_ids: Optional[torch.Tensor] = None, seed: int = 0, step: int = 0, vocab_offset: int = 0,
           out_ids: Optional[torch.Tensor] = None, out_vals: Optional[torch.Tensor] = None,
           return_vals: bool = False, candidates: int = 0, id_map: Optional[torch.Tensor] = None,
           stats: bool = False, target: Optional[torch.Tensor] = None):
    """Greedy when ``temperature`` is None (or <= 0 for a row); otherwise temperature / top-k / top-p.

    Vocabulary-parallel draws run in two stages.  ``candidates = k`` (on every shard, with ``vocab_offset``): returns
    ``(vals [B, k] fp32, ids [B, k] int32)``, the row's best entries after penalty and temperature, instead of drawing.
    ``id_map`` (identical on every rank): ``logits`` are the gathered fp32 candidates ``[B, world * k]`` and ``id_map``
    their global ids; the usual top-k / top-p / draw runs over them and returns global ids.

    Whole-vocabulary (temperature only) draws over shards: ``stats=True`` returns ``[B, 2]`` fp32 (the shard's largest
    scaled logit, the sum of ``exp(logit - max)``) instead of drawing; ``target`` ([B] fp32, in those units, negative =
    another shard draws) makes the shard that owns the draw pick the token, the others return -1."""
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("logits must be [B, V] with contiguous rows")
    if logits.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("logits must be bf16 or fp32")
    B, V = logits.shape
    if out_ids is None:
        out_ids = torch.empty(B, dtype=torch.int32, device=logits.device)
    if return_vals and out_vals is None:
        out_vals = torch.empty(B, dtype=torch.float32, device=logits.device)
    a = N.UbSampleArgs()
    a.logits, a.ld, a.logits_f32 = logits.data_ptr(), logits.stride(0), int(logits.dtype == torch.float32)
    a.out_ids, a.out_vals = out_ids.data_ptr(), _p(out_vals)
    a.temperature, a.top_p, a.top_k, a.rep_penalty = _p(temperature), _p(top_p), _p(top_k), _p(rep_penalty)
    if prev_ids is not None:
        a.prev_ids, a.prev_ld = prev_ids.data_ptr(), prev_ids.shape[1]
    a.seed, a.step, a.B, a.V, a.vocab_offset = seed & (2**64 - 1), step, B, V, vocab_offset
    a.err = err_word(logits.device).data_ptr()
    cv = ci = None
    if candidates:
        cv = torch.empty(B, candidates, dtype=torch.float32, device=logits.device)
        ci = torch.empty(B, candidates, dtype=torch.int32, device=logits.device)
        a.cand_vals, a.cand_ids, a.cand_k = cv.data_ptr(), ci.data_ptr(), candidates
    if id_map is not None:
        if id_map.dtype != torch.int32 or id_map.shape != logits.shape or not id_map.is_contiguous() or \
                logits.dtype != torch.float32 or not logits.is_contiguous():
            raise ValueError("id_map: int32, contiguous, same shape as the contiguous fp32 candidate values")
        a.id_map = id_map.data_ptr()
    st = None
    if stats:
        st = torch.empty(B, 2, dtype=torch.float32, device=logits.device)
        a.stats_out = st.data_ptr()
    if target is not None:
        a.target_in = target.data_ptr()
    N.check(N.cuda_lib().ub_sample(C.byref(a), _stream(logits)), "ub_sample")
    if stats:
        return st
    if candidates:
        return cv, ci
    return (out_ids, out_vals) if return_vals else out_ids


def vocab_shard_targets(maxes: torch.Tensor, masses: torch.Tensor, uniform: torch.Tensor):
    """Where a draw from the whole vocabulary falls when the vocabulary is cut into shards.  ``maxes`` / ``masses``
    ([B, W] fp32: every shard's largest scaled logit and its sum of ``exp(logit - max)``, as ``sample(stats=True)`` reports
    them) and the row's uniform number give ``(owner [B], target [B])``: the shard whose running mass passes
    ``uniform * total`` (shards in vocabulary order, like the single-kernel inverse CDF) and the target inside that shard
    in the shard's own units."""
    gmax = maxes.max(dim=1, keepdim=True).values
    mass = masses * torch.exp(maxes - gmax)
    cum = mass.cumsum(dim=1)
    tgt = uniform * cum[:, -1]
    owner = (cum > tgt[:, None]).float().argmax(dim=1)
    owner = torch.where(cum[:, -1] > tgt, owner, torch.full_like(owner, maxes.shape[1] - 1))
    before = (cum - mass).gather(1, owner[:, None])[:, 0]
    local = (tgt - before) * torch.exp(gmax[:, 0] - maxes.gather(1, owner[:, None])[:, 0])
    return owner, local.clamp_min(0.0)


def argmax_merge(vals: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """vals/ids [world, B] per-shard greedy winners -> global winners [B]."""
    world, B = vals.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=vals.device)
    lib = N.cuda_lib()
    lib.ub_argmax_merge.restype = C.c_int
    lib.ub_argmax_merge.argtypes = [N.vp, N.vp, N.i32, N.i32, N.vp, N.vp]
    N.check(lib.ub_argmax_merge(vals.data_ptr(), ids.data_ptr(), world, B, out.data_ptr(), _stream(vals)),
            "ub_argmax_merge")
    return out


# ---------------------------------------------------------------------------------------------
# Element-wise
# ---------------------------------------------------------------------------------------------
def embed_gather(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _bf16c(table, "table")
    if ids.dtype != torch.int32:
        ids = ids.to(torch.int32)
    ids = ids.contiguous()
    T = ids.numel()
    V, H = table.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.bfloat16, device=table.device)
    lib = N.cuda_lib()
    lib.ub_embed_gather.restype = C.c_int
    lib.ub_embed_gather.argtypes = [N.vp, N.vp, N.vp, N.i32, N.i32, N.i32, N.f32, N.vp, N.vp]
    N.check(lib.ub_embed_gather(ids.data_ptr(), table.data_ptr(), out.data_ptr(), T, H, V, scale,
                                err_word(table.device).data_ptr(), _stream(table)), "ub_embed_gather")
    return out


def act_mul(gate_up: torch.Tensor, act: str = "silu", out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(gate) * up`` for gate_up [..., 2*I] (gate first)."""
    _bf16c(gate_up, "gate_up")
    gate_up = gate_up.contiguous()
    I = gate_up.shape[-1] // 2
    T = gate_up.numel() // (2 * I)
    if out is None:
        out = torch.empty((*gate_up.shape[:-1], I), dtype=torch.bfloat16, device=gate_up.device)
    lib = N.cuda_lib()
    lib.ub_act_mul.restype = C.c_int
    lib.ub_act_mul.argtypes = [N.vp, N.vp, N.i64, N.i32, N.i32, N.vp]
    N.check(lib.ub_act_mul(gate_up.data_ptr(), out.data_ptr(), T, I, N.ACT[act], _stream(gate_up)), "ub_act_mul")
    return out


def eltwise(x: torch.Tensor, act: Optional[str], alpha: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _bf16c(x, "x")
    x = x.contiguous()
    if out is None:
        out = torch.empty_like(x)
    lib = N.cuda_lib()
    lib.ub_eltwise.restype = C.c_int
    lib.ub_eltwise.argtypes = [N.vp, N.vp, N.i64, N.i32, N.f32, N.vp]
    N.check(lib.ub_eltwise(x.data_ptr(), out.data_ptr(), x.numel(), N.ACT[act], alpha, _stream(x)), "ub_eltwise")
    return out


def add(a: torch.Tensor, b: torch.Tensor, sa: float = 1.0, sb: float = 1.0,
        out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _bf16c(a, "a"), _bf16c(b, "b")
    a, b = a.contiguous(), b.contiguous()
    if a.shape != b.shape:
        raise ValueError("add: shapes differ")
    if out is None:
        out = torch.empty_like(a)
    lib = N.cuda_lib()
    lib.ub_add.restype = C.c_int
    lib.ub_add.argtypes = [N.vp, N.vp, N.vp, N.i64, N.f32, N.f32, N.vp]
    N.check(lib.ub_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), sa, sb, _stream(a)), "ub_add")
    return out


def l2_normalize(x: torch.Tensor, eps: float = 1e-12) -> torch.Tensor:
    _bf16c(x, "x")
    x = x.contiguous()
    out = torch.empty_like(x)
    H = x.shape[-1]
    lib = N.cuda_lib()
    lib.ub_l2_normalize.restype = C.c_int
    lib.ub_l2_normalize.argtypes = [N.vp, N.vp, N.i32, N.i32, N.f32, N.vp]
    N.check(lib.ub_l2_normalize(x.data_ptr(), out.data_ptr(), x.numel() // H, H, eps, _stream(x)), "ub_l2_normalize")
    return out


# ------------------------------------------------------------------------------------------------
# Mixture of experts
# ------------------------------------------------------------------------------------------------
class MoeRouting:
    """Device-side routing state of one MoE layer call (all int32 / fp32 tensors, sized from T, K, E)."""

    __slots__ = ("T", "K", "E", "tile_tokens", "max_tiles", "topk_ids", "topk_w", "counts", "offsets", "sorted_rows",
                 "row_slot", "tiles")

    def __init__(self, T: int, K: int, E: int, tile_tokens: int, device):
        self.T, self.K, self.E, self.tile_tokens = T, K, E, tile_tokens
        self.max_tiles = (T * K + tile_tokens - 1) // tile_tokens + E
        i32 = dict(dtype=torch.int32, device=device)
        self.topk_ids = torch.empty(T, K, **i32)
        self.topk_w = torch.empty(T, K, dtype=torch.float32, device=device)
        self.counts = torch.empty(E, **i32)
        self.offsets = torch.empty(E + 1, **i32)
        self.sorted_rows = torch.empty(T * K, **i32)
        self.row_slot = torch.empty(T * K, **i32)
        self.tiles = torch.empty(self.max_tiles, 4, **i32)


def moe_tile_tokens(T: int, K: int, E: int) -> int:
    """Token tile for the grouped GEMM: the power of two covering the mean rows per expert, 16..128."""
    avg = max(1, (T * K + E - 1) // E)
    tn = 16
    while tn < avg and tn < 128:
        tn <<= 1
    return tn


def moe_route(x: Optional[torch.Tensor], router_w: Optional[torch.Tensor], top_k: int, *, norm_topk: bool = True,
              logits: Optional[torch.Tensor] = None, weight_scale: float = 1.0, tile_tokens: int = 0,
              round_logits_bf16: bool = True, routing: Optional[MoeRouting] = None, expert_lo: int = 0,
              num_local_experts: int = 0) -> MoeRouting:
    """Router GEMV + top-k + softmax weights + expert sort + grouped-GEMM tile table, two launches.

    ``expert_lo`` / ``num_local_experts`` restrict the sort to the experts of this rank (expert parallelism): pairs
    routed to other ranks get ``row_slot = -1`` and take no part in the grouped GEMMs."""
    if router_w is not None:
        _bf16c(x, "x"), _bf16c(router_w, "router_w")
        T, H = x.shape
        E = router_w.shape[0]
        dev = x.device
    else:
        T, E = logits.shape
        H = 0
        dev = logits.device
        if not logits.is_contiguous():
            raise ValueError("logits must be contiguous")
    tn = tile_tokens or moe_tile_tokens(T, top_k, E)
    r = routing if routing is not None else MoeRouting(T, top_k, E, tn, dev)
    a = N.UbMoeRouteArgs()
    a.logits, a.x, a.router_w = _p(logits), _p(x) if router_w is not None else None, _p(router_w)
    a.topk_ids, a.topk_w = r.topk_ids.data_ptr(), r.topk_w.data_ptr()
    a.expert_counts, a.expert_offsets = r.counts.data_ptr(), r.offsets.data_ptr()
    a.sorted_rows, a.row_slot, a.tiles = r.sorted_rows.data_ptr(), r.row_slot.data_ptr(), r.tiles.data_ptr()
    a.err = err_word(dev).data_ptr()
    a.logits_f32 = 1 if (logits is not None and logits.dtype == torch.float32) else 0
    a.T, a.E, a.K, a.H = T, E, top_k, H
    a.norm_topk = 1 if norm_topk else 0
    a.round_logits_bf16 = 1 if round_logits_bf16 else 0
    a.weight_scale = weight_scale
    a.tile_tokens, a.max_tiles = r.tile_tokens, r.max_tiles
    a.expert_lo, a.num_local_experts = expert_lo, num_local_experts
    N.check(N.cuda_lib().ub_moe_route(C.byref(a), torch.cuda.current_stream(dev).cuda_stream), "ub_moe_route")
    return r


def moe_gather(x: torch.Tensor, r: MoeRouting, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[slot] = x[sorted_rows[slot] // K]``: activations in expert order."""
    _bf16c(x, "x")
    T, H = x.shape
    if out is None:
        out = torch.empty(T * r.K, H, dtype=torch.bfloat16, device=x.device)
    lib = N.cuda_lib()
    lib.ub_moe_gather.restype = C.c_int
    lib.ub_moe_gather.argtypes = [N.vp, N.vp, N.vp, N.i32, N.i32, N.i32, N.vp]
    N.check(lib.ub_moe_gather(x.data_ptr(), r.sorted_rows.data_ptr(), out.data_ptr(), T * r.K, r.K, H, _stream(x)),
            "ub_moe_gather")
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[i] = x[rows[i]]`` for int32 ``rows`` (negative entries leave ``out[i]`` untouched)."""
    _bf16c(x, "x")
    H = x.shape[1]
    n = rows.numel()
    if out is None:
        out = torch.empty(n, H, dtype=torch.bfloat16, device=x.device)
    lib = N.cuda_lib()
    lib.ub_moe_gather.restype = C.c_int
    lib.ub_moe_gather.argtypes = [N.vp, N.vp, N.vp, N.i32, N.i32, N.i32, N.vp]
    N.check(lib.ub_moe_gather(x.data_ptr(), rows.data_ptr(), out.data_ptr(), n, 1, H, _stream(x)), "ub_moe_gather")
    return out


def moe_combine(y: torch.Tensor, r: MoeRouting, residual: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = residual[t] + sum_k w[t,k] * y[row_slot[t,k]]``."""
    _bf16c(y, "y")
    H = y.shape[1]
    if out is None:
        out = torch.empty(r.T, H, dtype=torch.bfloat16, device=y.device)
    lib = N.cuda_lib()
    lib.ub_moe_combine.restype = C.c_int
    lib.ub_moe_combine.argtypes = [N.vp, N.vp, N.vp, N.vp, N.vp, N.i32, N.i32, N.i32, N.vp]
    N.check(lib.ub_moe_combine(y.data_ptr(), r.row_slot.data_ptr(), r.topk_w.data_ptr(), _p(residual), out.data_ptr(),
                               r.T, r.K, H, _stream(y)), "ub_moe_combine")
    return out


def moe_combine_num_ctas(T: int, H: int) -> int:
    lib = N.cuda_lib()
    lib.ub_moe_combine_num_ctas.restype = C.c_int
    lib.ub_moe_combine_num_ctas.argtypes = [N.i32, N.i32]
    return lib.ub_moe_combine_num_ctas(T, H)


def moe_combine_rs(y: torch.Tensor, r: MoeRouting, rs: dict) -> None:
    """Combine fused with the reduce-scatter: partial rows go into the owners' receive slots (``rs`` as for
    ``gemm_tn``: world, rank, rows_per_rank, peer_out, peer_flag, local_count); the last CTA signals each peer once."""
    _bf16c(y, "y")
    H = y.shape[1]
    W = rs["world"]
    outs = (C.c_void_p * W)(*[(int(p) or None) for p in rs["peer_out"][:W]])
    flags = (C.c_void_p * W)(*[int(p) for p in rs["peer_flag"][:W]])
    lib = N.cuda_lib()
    lib.ub_moe_combine_rs.restype = C.c_int
    lib.ub_moe_combine_rs.argtypes = [N.vp, N.vp, N.vp, N.i32, N.i32, N.i32, N.i32, N.i32, N.i32, N.vp, N.vp, N.vp, N.vp, N.vp]
    N.check(lib.ub_moe_combine_rs(y.data_ptr(), r.row_slot.data_ptr(), r.topk_w.data_ptr(), r.T, r.K, H, W, rs["rank"],
                                  rs["rows_per_rank"], C.cast(outs, C.c_void_p), C.cast(flags, C.c_void_p),
                                  rs["local_count"], rs.get("local_out") or None, _stream(y)),
            "ub_moe_combine_rs")


class MoeDispatch:
    """Device-side state of one sparse expert-parallel MoE call on one rank: the routing of this rank's own ``R`` rows
    (``route``), the send scratch, and what the receive side builds (row order, return addresses, tile table).  The
    attributes ``tiles`` / ``max_tiles`` / ``tile_tokens`` make it usable where ``grouped_gemm`` expects a routing."""

    def __init__(self, R: int, K: int, E: int, world: int, device):
        self.R, self.K, self.E, self.world = R, K, E, world
        self.experts_local = E // world
        self.cap = R * K
        self.slots = world * self.cap                         # = T * K: every pair of the step could land here
        self.tile_tokens = moe_tile_tokens(R * world, K, E)
        self.max_tiles = (self.slots + self.tile_tokens - 1) // self.tile_tokens + self.experts_local
        i32 = dict(dtype=torch.int32, device=device)
        self.route = MoeRouting(R, K, E, self.tile_tokens, device)
        self.send_slot = torch.empty(R * K, **i32)
        self.send_counts = torch.empty(E, **i32)
        self.sorted_rows = torch.empty(self.slots, **i32)
        self.slot_meta = torch.empty(self.slots, 4, **i32)
        self.counts = torch.empty(self.experts_local, **i32)
        self.offsets = torch.empty(self.experts_local + 1, **i32)
        self.tiles = torch.empty(self.max_tiles, 4, **i32)


def moe_dispatch(x: torch.Tensor, d: MoeDispatch, comm: dict) -> None:
    """F5 send side: rows of ``x`` ([R, H], this rank's tokens, routed in ``d.route``) go to the ranks of their
    experts.  ``comm``: world, rank, peer_rows / peer_meta / peer_counts / peer_flag (one address per rank) and
    local_count, as ``FusedComm.moe_dispatch_args`` builds them."""
    _bf16c(x, "x")
    a = N.UbMoeDispatchArgs()
    a.x, a.topk_ids, a.topk_w = x.data_ptr(), d.route.topk_ids.data_ptr(), d.route.topk_w.data_ptr()
    a.send_slot, a.send_counts = d.send_slot.data_ptr(), d.send_counts.data_ptr()
    for r in range(comm["world"]):
        a.peer_rows[r], a.peer_meta[r] = comm["peer_rows"][r], comm["peer_meta"][r]
        a.peer_counts[r], a.peer_flag[r] = comm["peer_counts"][r], comm["peer_flag"][r]
    a.local_count = comm["local_count"]
    a.err = err_word(x.device).data_ptr()
    a.R, a.K, a.H, a.E = d.R, d.K, x.shape[1], d.E
    a.world, a.rank, a.experts_local, a.cap = comm["world"], comm["rank"], d.experts_local, d.cap
    lib = N.cuda_lib()
    lib.ub_moe_dispatch.restype = C.c_int
    N.check(lib.ub_moe_dispatch(C.byref(a), _stream(x)), "ub_moe_dispatch")


def moe_recv_build(d: MoeDispatch, comm: dict, device) -> None:
    """F5 receive side: waits (bounded, on the device) for every source's arrival, then orders the received rows by
    expert: ``d.sorted_rows`` (receive row per slot), ``d.slot_meta`` (return address), ``d.tiles``."""
    a = N.UbMoeRecvArgs()
    a.counts, a.meta, a.flag, a.round = comm["counts"], comm["meta"], comm["flag"], comm["round"]
    a.sorted_rows, a.slot_meta = d.sorted_rows.data_ptr(), d.slot_meta.data_ptr()
    a.expert_counts, a.expert_offsets, a.tiles = d.counts.data_ptr(), d.offsets.data_ptr(), d.tiles.data_ptr()
    a.err = err_word(device).data_ptr()
    a.world, a.experts_local, a.cap = d.world, d.experts_local, d.cap
    a.tile_tokens, a.max_tiles = d.tile_tokens, d.max_tiles
    lib = N.cuda_lib()
    lib.ub_moe_recv_build.restype = C.c_int
    N.check(lib.ub_moe_recv_build(C.byref(a), torch.cuda.current_stream(device).cuda_stream), "ub_moe_recv_build")


def moe_combine_push(y: torch.Tensor, d: MoeDispatch, comm: dict) -> None:
    """F6: ``y[slot] * weight`` goes into slot ``[k][row]`` of the token owner's combine area; one arrival per rank."""
    _bf16c(y, "y")
    a = N.UbMoeReturnArgs()
    a.y, a.slot_meta, a.expert_offsets = y.data_ptr(), d.slot_meta.data_ptr(), d.offsets.data_ptr()
    for r in range(comm["world"]):
        a.peer_comb[r], a.peer_flag[r] = comm["peer_comb"][r], comm["peer_flag"][r]
    a.local_count = comm["local_count"]
    a.err = err_word(y.device).data_ptr()
    a.R, a.K, a.H, a.world, a.experts_local = d.R, d.K, y.shape[1], comm["world"], d.experts_local
    lib = N.cuda_lib()
    lib.ub_moe_combine_push.restype = C.c_int
    N.check(lib.ub_moe_combine_push(C.byref(a), d.slots, _stream(y)), "ub_moe_combine_push")


def grouped_gemm(x_sorted: torch.Tensor, w: torch.Tensor, r: MoeRouting, *, dual_rows: int = 0, act: Optional[str] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Expert-grouped GEMM: rows of ``x_sorted`` that belong to expert e multiply ``w[e]`` (``[E, rows, K]``).

    ``dual_rows = I``: ``w[e]`` is ``[2I, K]`` (gate rows then up rows) and the result is ``act(gate) * up``.
    """
    if w.dim() != 3 or not w.is_contiguous():
        raise ValueError("grouped_gemm takes contiguous weights [E, rows, K]")
    E, rows, Kd = w.shape
    g = {"tiles": r.tiles.data_ptr(), "max_tiles": r.max_tiles, "w_rows": rows, "tile_tokens": r.tile_tokens}
    n_out = dual_rows if dual_rows else rows
    if out is None:
        out = torch.empty(x_sorted.shape[0], n_out, dtype=torch.bfloat16, device=x_sorted.device)
    w2 = w.view(E * rows, Kd)
    if dual_rows:
        return gemm_tn(x_sorted, w2, dual_rows=dual_rows, act=act, out=out, grouped=g)
    # non-dual: N is the per-expert row count while w2 has E*rows rows
    return _gemm_grouped_plain(x_sorted, w2, rows, act, out, g)


def _gemm_grouped_plain(x, w2, rows, act, out, g):
    a = N.UbGemmArgs()
    a.x, a.w, a.out = x.data_ptr(), w2.data_ptr(), out.data_ptr()
    a.err = err_word(x.device).data_ptr()
    a.M, a.N, a.K = x.shape[0], rows, x.shape[1]
    a.ldx, a.ldw, a.ldo = x.stride(0), w2.stride(0), out.stride(0)
    a.act = N.ACT[act]
    a.w_rows_total = w2.shape[0]
    a.out_scale = 1.0
    a.grp_tiles, a.grp_max_tiles, a.grp_w_rows, a.tile_tokens = g["tiles"], g["max_tiles"], g["w_rows"], g["tile_tokens"]
    N.check(N.cuda_lib().ub_gemm_tn(C.byref(a), _stream(x)), "ub_gemm_tn(grouped)")
    return out
