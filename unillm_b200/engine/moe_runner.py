"""Mixture-of-experts block of the GPU runner.

Five launches for the routed experts: route (router GEMV + top-k + sort + tile table, 2 kernels), gather, grouped
gate/up GEMM with the activation in its epilogue, grouped down GEMM, weighted combine with the residual.  The
reference walks tokens and experts on the host (``crates/runtime/src/model_core.rs:796-905``); here nothing about
the routing ever reaches the host, so the block sits inside a CUDA graph like any dense layer.

Two multi-GPU layouts.  Tensor parallelism shards every expert's FFN width across the ranks (each rank holds all
experts).  Expert parallelism (``RunnerWeights(expert_parallel=True)``) keeps whole experts on their rank: the
hidden rows are already replicated by the attention block's reduction (the dispatch), every rank routes all tokens
identically, runs the grouped GEMMs for the pairs that picked one of its experts, and combines them into a partial
row per token.  Either way the partial rows are summed across ranks once, together with the shared experts /
parallel dense MLP: by an all-reduce, or (``combine_rs``) by the combine kernel storing straight into the owners'
receive slots over NVLink, which the next norm kernel sums.

``moe_sparse`` is the expert-parallel layout without the replication: every rank routes only the token rows it
owns, each (token, expert) pair's row goes to the one rank that holds the expert, and the weighted expert output
comes back into the token owner's combine area (see the F5 / F6 kernels in ``csrc/moe/moe.cu``).
"""
from __future__ import annotations

import torch

from ..ops import cuda_ops as K


def moe_partial(runner, i: int, h: torch.Tensor, residual=None, combine_rs=None) -> torch.Tensor:
    """MoE output for hidden rows ``h`` ([T, H]).  With ``residual`` (single rank only) it is added in the combine.
    ``combine_rs`` (peer pointers as for ``gemm_tn(rs=...)``) makes the combine kernel push its partial rows to the
    ranks that own them instead of returning them."""
    s, t = runner.spec, runner.w.t
    m = s.moe
    L = f"layers.{i}."
    T = h.shape[0]
    with runner._prof("moe_route"):
        r = K.moe_route(h, t[L + "router"], m.top_k, norm_topk=m.normalize_topk, round_logits_bf16=False,
                        expert_lo=runner.w.expert_lo if runner.w.ep else 0,
                        num_local_experts=runner.w.experts_local if runner.w.ep else 0)
        xs = K.moe_gather(h, r)
    runner.launches += 3
    gu, dn = t[L + "experts_gate_up"], t[L + "experts_down"]
    with runner._prof(f"moe_gate_up[{T * m.top_k}x{gu.shape[1]}x{gu.shape[2]}]"):
        if m.gated:
            a = K.grouped_gemm(xs, gu, r, dual_rows=gu.shape[1] // 2, act=m.act)
        else:
            a = K.grouped_gemm(xs, gu, r, act=m.act)
    with runner._prof(f"moe_down[{T * m.top_k}x{dn.shape[1]}x{dn.shape[2]}]"):
        y = K.grouped_gemm(a, dn, r)
    base = residual
    if m.num_shared_experts:
        Is = t[L + "shared_gate_up"].shape[0] // 2
        sh = runner._gemm(h, t[L + "shared_gate_up"], dual_rows=Is, act=m.act)
        base = runner._gemm(sh, t[L + "shared_down"], residual=residual)
    if m.dense_parallel and (L + "w_down") in t:
        d = runner._mlp_noresid(i, h, dense_only=True)
        base = d if base is None else K.add(base, d)
        runner.launches += 1
    with runner._prof("moe_combine"):
        if combine_rs is not None:
            if base is not None:
                raise ValueError("combine_rs pushes partial sums; shared experts / residual are added by the caller")
            K.moe_combine_rs(y, r, combine_rs)
            out = None
        else:
            out = K.moe_combine(y, r, residual=base)
    runner.launches += 3
    return out


def moe_sparse(runner, i: int, h_own: torch.Tensor, comm, R: int) -> None:
    """Sparse expert-parallel MoE for this rank's ``R`` normalised rows ``h_own``.  Nothing is returned: the weighted
    outputs of all ranks' experts for these rows arrive in ``comm.moe_comb_tensor(R)``, complete once the second
    reduce-scatter counter shows one arrival per rank (the next norm kernel waits for exactly that)."""
    s, t = runner.spec, runner.w.t
    m = s.moe
    L = f"layers.{i}."
    W = comm.world
    key = (R, m.top_k, m.num_experts)
    d = runner._moe_dispatch_state.get(key) if hasattr(runner, "_moe_dispatch_state") else None
    if d is None:
        if not hasattr(runner, "_moe_dispatch_state"):
            runner._moe_dispatch_state = {}
        d = runner._moe_dispatch_state[key] = K.MoeDispatch(R, m.top_k, m.num_experts, W, h_own.device)
    with runner._prof("moe_route_dispatch"):
        K.moe_route(h_own, t[L + "router"], m.top_k, norm_topk=m.normalize_topk, round_logits_bf16=False, routing=d.route)
        K.moe_dispatch(h_own, d, comm.moe_dispatch_args())
    with runner._prof("moe_recv"):
        K.moe_recv_build(d, comm.moe_recv_args(), h_own.device)
        xs = K.gather_rows(comm.moe_recv_rows(d.slots), d.sorted_rows)
    runner.launches += 6
    gu, dn = t[L + "experts_gate_up"], t[L + "experts_down"]
    with runner._prof(f"moe_gate_up[{d.slots}x{gu.shape[1]}x{gu.shape[2]}]"):
        if m.gated:
            a = K.grouped_gemm(xs, gu, d, dual_rows=gu.shape[1] // 2, act=m.act)
        else:
            a = K.grouped_gemm(xs, gu, d, act=m.act)
    with runner._prof(f"moe_down[{d.slots}x{dn.shape[1]}x{dn.shape[2]}]"):
        y = K.grouped_gemm(a, dn, d)
    with runner._prof("moe_combine_push"):
        K.moe_combine_push(y, d, comm.moe_return_args())
    runner.launches += 3


def moe_forward(runner, i: int, h: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    """``residual + MoE(h)`` including the tensor-parallel reduction."""
    tp = runner.tp
    if tp.world == 1:
        return moe_partial(runner, i, h, residual)
    y = moe_partial(runner, i, h, None)
    tp.all_reduce(y)
    runner.launches += 1
    return K.add(y, residual)
