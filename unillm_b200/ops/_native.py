"""ctypes bindings of the in-tree native libraries.

``cuda_lib()`` loads ``_native/libunillm_b200_cuda.so`` (all sm_100a kernels, C ABI declared in
``csrc/include/unillm_b200.h``) and ``host_lib()`` loads ``_native/libunillm_b200_host.so`` (C++ host
runtime).  Both are built on demand by ``unillm_b200._build``.  On a machine with a GPU a missing or
unloadable CUDA library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_NATIVE_DIR = Path(__file__).resolve().parent.parent / "_native"
_lock = threading.Lock()
_cuda = None
_host = None

UB_MAX_RANKS = 8

ACT = {
    None: 0, "none": 0, "silu": 1, "swish": 1, "gelu": 2, "gelu_tanh": 3, "gelu_new": 3, "gelu_pytorch_tanh": 3,
    "relu": 4, "relu2": 5, "quick_gelu": 6, "sigmoid": 7, "tanh": 8, "softplus": 9, "exp": 10,
}

vp = C.c_void_p
i32 = C.c_int
i64 = C.c_longlong
u32 = C.c_uint32
u64 = C.c_ulonglong
f32 = C.c_float


class UbGemmArgs(C.Structure):
    _fields_ = [
        ("x", vp), ("w", vp), ("out", vp), ("bias", vp), ("residual", vp), ("err", vp),
        ("M", i32), ("N", i32), ("K", i32),
        ("ldx", i64), ("ldw", i64), ("ldo", i64), ("ldr", i64),
        ("act", i32), ("dual", i32), ("up_row_off", i32), ("w_rows_total", i32), ("out_f32", i32),
        ("out_scale", f32), ("tile_tokens", i32), ("splits", i32),
        ("rs_world", i32), ("rs_rank", i32), ("rs_rows_per_rank", i32),
        ("rs_peer_out", vp * UB_MAX_RANKS), ("rs_peer_flag", vp * UB_MAX_RANKS),
        ("ag_world", i32), ("ag_rows_per_rank", i32),
        ("ag_flags", vp), ("ag_epoch", vp), ("ag_signals_per_use", u32),
        ("grp_tiles", vp), ("grp_max_tiles", i32), ("grp_w_rows", i32), ("tail_split", i32), ("cta_pair", i32), ("pair_splits", i32),
        ("rs_local_count", vp),
    ]


class UbNormArgs(C.Structure):
    _fields_ = [
        ("x", vp), ("residual", vp), ("weight", vp), ("bias", vp), ("out", vp), ("residual_out", vp), ("err", vp),
        ("T", i32), ("H", i32), ("eps", f32), ("kind", i32), ("weight_offset_one", i32),
        ("rs_world", i32), ("rs_flag", vp), ("epoch", vp), ("rs_signals_per_use", u32),
        ("ag_world", i32), ("ag_rank", i32),
        ("ag_peer_out", vp * UB_MAX_RANKS), ("ag_peer_flag", vp * UB_MAX_RANKS),
        ("reset_flags", vp), ("reset_count", i32), ("ag_local_count", vp), ("rs_multimem", i32), ("ag_mc_out", vp),
    ]


class UbRopeArgs(C.Structure):
    _fields_ = [
        ("qkv", vp), ("positions", vp), ("slot_mapping", vp), ("k_cache", vp), ("v_cache", vp),
        ("q_norm_w", vp), ("k_norm_w", vp), ("err", vp),
        ("T", i32), ("Hq", i32), ("Hkv", i32), ("D", i32), ("rotary_dim", i32), ("block_size", i32),
        ("num_slots", i64), ("theta", f32), ("pos_scale", f32), ("norm_eps", f32), ("interleaved", i32),
        ("l3_factor", f32), ("l3_low_freq_factor", f32), ("l3_high_freq_factor", f32), ("l3_orig_ctx", f32),
    ]


class UbAttnArgs(C.Structure):
    _fields_ = [
        ("q", vp), ("k_cache", vp), ("v_cache", vp), ("out", vp), ("lse", vp),
        ("block_tables", vp), ("seq_lens", vp), ("q_start", vp), ("alibi_slopes", vp), ("scratch", vp), ("err", vp),
        ("num_seqs", i32), ("Hq", i32), ("Hkv", i32), ("D", i32),
        ("block_size", i32), ("max_blocks_per_seq", i32), ("num_blocks", i32),
        ("q_stride", i64), ("o_stride", i64), ("scale", f32),
        ("causal", i32), ("window", i32), ("splits", i32), ("kv_start", i32), ("total_q", i32), ("max_q_len", i32),
        ("merge_o", vp), ("merge_lse", vp),
    ]


class UbSampleArgs(C.Structure):
    _fields_ = [
        ("logits", vp), ("ld", i64), ("logits_f32", i32), ("out_ids", vp), ("out_vals", vp),
        ("temperature", vp), ("top_p", vp), ("top_k", vp), ("rep_penalty", vp), ("prev_ids", vp), ("prev_ld", i32),
        ("seed", u64), ("step", u64), ("B", i32), ("V", i32), ("vocab_offset", i32), ("err", vp),
        ("cand_vals", vp), ("cand_ids", vp), ("cand_k", i32), ("id_map", vp), ("stats_out", vp), ("target_in", vp),
    ]


class UbPairGatherArgs(C.Structure):
    _fields_ = [
        ("vals", vp), ("ids", vp), ("out_vals", vp), ("out_ids", vp), ("peer_vals", vp * UB_MAX_RANKS),
        ("peer_ids", vp * UB_MAX_RANKS), ("peer_flags", vp * UB_MAX_RANKS), ("my_vals", vp), ("my_ids", vp),
        ("my_flags", vp), ("round", vp), ("done_count", vp), ("world", i32), ("rank", i32), ("rows", i32), ("k", i32),
        ("cap", i64), ("err", vp), ("cta_rounds", vp),
    ]


class UbMoeRouteArgs(C.Structure):
    _fields_ = [
        ("logits", vp), ("x", vp), ("router_w", vp), ("topk_ids", vp), ("topk_w", vp), ("expert_counts", vp),
        ("expert_offsets", vp), ("sorted_rows", vp), ("row_slot", vp), ("tiles", vp), ("err", vp),
        ("logits_f32", i32), ("T", i32), ("E", i32), ("K", i32), ("H", i32), ("norm_topk", i32),
        ("round_logits_bf16", i32), ("weight_scale", f32), ("tile_tokens", i32), ("max_tiles", i32),
        ("expert_lo", i32), ("num_local_experts", i32),
    ]


class UbMoeDispatchArgs(C.Structure):
    _fields_ = [
        ("x", vp), ("topk_ids", vp), ("topk_w", vp), ("send_slot", vp), ("send_counts", vp),
        ("peer_rows", vp * UB_MAX_RANKS), ("peer_meta", vp * UB_MAX_RANKS), ("peer_counts", vp * UB_MAX_RANKS),
        ("peer_flag", vp * UB_MAX_RANKS), ("local_count", vp), ("err", vp),
        ("R", i32), ("K", i32), ("H", i32), ("E", i32), ("world", i32), ("rank", i32), ("experts_local", i32), ("cap", i32),
    ]


class UbMoeRecvArgs(C.Structure):
    _fields_ = [
        ("counts", vp), ("meta", vp), ("flag", vp), ("round", vp), ("sorted_rows", vp), ("slot_meta", vp),
        ("expert_counts", vp), ("expert_offsets", vp), ("tiles", vp), ("err", vp),
        ("world", i32), ("experts_local", i32), ("cap", i32), ("tile_tokens", i32), ("max_tiles", i32),
    ]


class UbMoeReturnArgs(C.Structure):
    _fields_ = [
        ("y", vp), ("slot_meta", vp), ("expert_offsets", vp), ("peer_comb", vp * UB_MAX_RANKS),
        ("peer_flag", vp * UB_MAX_RANKS), ("local_count", vp), ("err", vp),
        ("R", i32), ("K", i32), ("H", i32), ("world", i32), ("experts_local", i32),
    ]


class UbAllReduceArgs(C.Structure):
    _fields_ = [
        ("in_", vp), ("out", vp), ("peer_slots", vp * UB_MAX_RANKS), ("peer_flags", vp * UB_MAX_RANKS),
        ("my_slots", vp), ("my_flags", vp), ("round", vp), ("done_count", vp), ("world", i32), ("rank", i32), ("n", i64),
        ("err", vp), ("cta_rounds", vp), ("max_n", i64),
    ]


class UbArgmaxMergeArgs(C.Structure):
    _fields_ = [
        ("vals", vp), ("ids", vp), ("out_ids", vp), ("peer_vals", vp * UB_MAX_RANKS), ("peer_ids", vp * UB_MAX_RANKS),
        ("peer_flags", vp * UB_MAX_RANKS), ("my_vals", vp), ("my_ids", vp), ("my_flag", vp), ("round", vp),
        ("world", i32), ("rank", i32), ("rows", i32), ("max_rows", i32), ("err", vp),
    ]


class UbDeviceProps(C.Structure):
    _fields_ = [
        ("name", C.c_char * 128), ("total_mem", u64), ("sm_count", i32), ("cc_major", i32), ("cc_minor", i32),
        ("max_smem_per_block", i32), ("l2_bytes", i32), ("clock_khz", i32), ("mem_clock_khz", i32),
        ("mem_bus_bits", i32),
    ]


def _ensure_built() -> None:
    from .. import _build

    _build.build_all()


def cuda_lib_path() -> Path:
    return _NATIVE_DIR / "libunillm_b200_cuda.so"


def host_lib_path() -> Path:
    return _NATIVE_DIR / "libunillm_b200_host.so"


def cuda_lib() -> C.CDLL:
    """The CUDA kernel library.  Raises if it cannot be built or loaded."""
    global _cuda
    if _cuda is not None:
        return _cuda
    with _lock:
        if _cuda is not None:
            return _cuda
        if not cuda_lib_path().exists() or os.environ.get("UNILLM_REBUILD"):
            _ensure_built()
        lib = C.CDLL(str(cuda_lib_path()))
        for name in (
            "ub_gemm_tn", "ub_norm", "ub_rope_kv_append", "ub_attn_decode", "ub_attn_prefill", "ub_sample",
            "ub_moe_route", "ub_allreduce_oneshot", "ub_tp_argmax_merge",
        ):
            if hasattr(lib, name):
                getattr(lib, name).restype = i32
                getattr(lib, name).argtypes = [vp, vp]
        lib.ub_gemm_num_ctas.restype = i32
        lib.ub_gemm_num_ctas.argtypes = [vp]
        lib.ub_gemm_streamk_reset.restype = i32
        lib.ub_gemm_streamk_reset.argtypes = [vp]
        lib.ub_cuda_error_string.restype = C.c_char_p
        _cuda = lib
        return lib


def host_lib() -> C.CDLL:
    """The host C++ runtime library (KV block pool, radix tree, quantisation oracle, ...)."""
    global _host
    if _host is not None:
        return _host
    with _lock:
        if _host is not None:
            return _host
        if not host_lib_path().exists() or os.environ.get("UNILLM_REBUILD"):
            _ensure_built()
        _host = C.CDLL(str(host_lib_path()))
        return _host


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = ""
        if rc < 0 and rc > -1000:
            try:
                msg = cuda_lib().ub_cuda_error_string(rc).decode()
            except Exception:  # pragma: no cover
                pass
        raise RuntimeError(f"{what} failed with code {rc} {msg}")
