"""Recurrences of the O(1)-state architectures: depthwise causal conv, selective scan, diagonal linear recurrence,
WKV-4, WKV-6.

Every function has two implementations with one signature: a plain PyTorch fp32 loop over time (the oracle, used on
CPU and by the tests) and the CUDA kernel of ``csrc/scan/scan.cu`` (used for bf16 CUDA tensors).  From 1024 steps on
the kernels run the sequence in 256-step chunks in parallel (chunk summaries, a short carry over the chunks, outputs).  States are updated
in place when given, so prefill (``L`` = prompt length) and decode (``L`` = 1) chain naturally.

Reference math: ``models_v2/mamba.rs:632-742`` (conv), ``:745-888`` (scan), ``rwkv4.rs:468-529``, ``rwkv6.rs:483-553``,
``recurrent_gemma.rs:624-690``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.nn.functional as F


def _use_kernel(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def _lib():
    from . import _native as N

    lib = N.cuda_lib()
    if not getattr(lib, "_scan_bound", False):
        vp, i32 = N.vp, N.i32
        lib.ub_causal_dwconv1d.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]
        lib.ub_selective_scan.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]
        lib.ub_linear_recurrence.argtypes = [vp, i32, vp, vp, vp, i32, i32, i32, i32, vp, vp]
        lib.ub_wkv4.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp]
        lib.ub_wkv6.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp]
        lib.ub_scan_chunks.argtypes = [i32]
        lib.ub_scan_workspace_floats.argtypes = [i32, i32, i32, i32, i32]
        lib.ub_scan_workspace_floats.restype = C.c_longlong
        for n in ("ub_causal_dwconv1d", "ub_selective_scan", "ub_linear_recurrence", "ub_wkv4", "ub_wkv6", "ub_scan_chunks"):
            getattr(lib, n).restype = i32
        lib._scan_bound = True
    return lib, N


def _st(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _f32c(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.float().contiguous()


CHUNKED = True      # long sequences run the scans in parallel chunks (tests switch it off to compare with the single pass)


def _workspace(lib, kind: int, B: int, L: int, n: int, m: int, device) -> Optional[torch.Tensor]:
    """fp32 workspace of the chunked form of a scan, or None when the single sequential pass is used."""
    need = lib.ub_scan_workspace_floats(kind, B, L, n, m) if CHUNKED else 0
    return torch.empty(need, dtype=torch.float32, device=device) if need > 0 else None


# ------------------------------------------------------------------------------------------------
def causal_dwconv1d(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None,
                    act_silu: bool = False, update_state: bool = True) -> torch.Tensor:
    """``x`` [B, L, C]; ``w`` [C, Kw]; ``state`` [B, Kw-1, C] = the inputs preceding this call (same dtype as x)."""
    Bn, L, Cn = x.shape
    Kw = w.shape[1]
    if _use_kernel(x):
        lib, N = _lib()
        x = x.contiguous()
        out = torch.empty_like(x)
        wf, bf = _f32c(w), _f32c(b)
        N.check(lib.ub_causal_dwconv1d(x.data_ptr(), wf.data_ptr(), _p(bf), out.data_ptr(), _p(state), Bn, L, Cn, Kw,
                                       int(act_silu), int(update_state), _st(x)), "ub_causal_dwconv1d")
        return out
    xf = x.float()
    left = state.float() if state is not None else torch.zeros(Bn, Kw - 1, Cn)
    full = torch.cat([left.to(xf.device), xf], 1)                     # [B, Kw-1+L, C]
    y = F.conv1d(full.transpose(1, 2), w.float()[:, None, :], None if b is None else b.float(), groups=Cn).transpose(1, 2)
    if act_silu:
        y = F.silu(y)
    if state is not None and update_state and Kw > 1:
        state.copy_(full[:, -(Kw - 1):].to(state.dtype))
    return y.to(x.dtype)


def selective_scan(u: torch.Tensor, delta: torch.Tensor, A: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor,
                   D: Optional[torch.Tensor] = None, z: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None,
                   delta_softplus: bool = True) -> torch.Tensor:
    """``u, delta, z`` [B, L, Dm]; ``A`` [Dm, Ns]; ``Bm, Cm`` [B, L, Ns]; ``D`` [Dm]; ``state`` fp32 [B, Dm, Ns]."""
    Bn, L, Dm = u.shape
    Ns = A.shape[1]
    if _use_kernel(u) and Ns in (4, 8, 16, 32):
        lib, N = _lib()
        u, delta, Bm, Cm = u.contiguous(), delta.contiguous(), Bm.contiguous(), Cm.contiguous()
        z = None if z is None else z.contiguous()
        out = torch.empty_like(u)
        Af, Df = _f32c(A), _f32c(D)
        ws = _workspace(lib, 0, Bn, L, Dm, Ns, u.device)
        N.check(lib.ub_selective_scan(u.data_ptr(), delta.data_ptr(), Af.data_ptr(), Bm.data_ptr(), Cm.data_ptr(), _p(Df),
                                      _p(z), out.data_ptr(), _p(state), Bn, L, Dm, Ns, int(delta_softplus), _p(ws), _st(u)),
                "ub_selective_scan")
        return out
    uf, dt, Af = u.float(), delta.float(), A.float()
    if delta_softplus:
        dt = F.softplus(dt)
    h = state.float().clone() if state is not None else torch.zeros(Bn, Dm, Ns, device=u.device)
    ys = []
    Bf, Cf = Bm.float(), Cm.float()
    for l in range(L):
        dA = torch.exp(dt[:, l, :, None] * Af[None])
        h = dA * h + dt[:, l, :, None] * Bf[:, l, None, :] * uf[:, l, :, None]
        ys.append((h * Cf[:, l, None, :]).sum(-1))
    y = torch.stack(ys, 1)
    if D is not None:
        y = y + D.float() * uf
    if z is not None:
        y = y * F.silu(z.float())
    if state is not None:
        state.copy_(h)
    return y.to(u.dtype)


def linear_recurrence(a: torch.Tensor, x: torch.Tensor, state: Optional[torch.Tensor] = None, one_minus: bool = False) -> torch.Tensor:
    """``h = a*h + (1-a if one_minus else 1)*x`` along L.  ``a`` [C] or [B, L, C]; ``x`` [B, L, C]; ``state`` fp32 [B, C]."""
    Bn, L, Cn = x.shape
    per_step = a.dim() == 3
    if _use_kernel(x):
        lib, N = _lib()
        x = x.contiguous()
        af = _f32c(a)
        out = torch.empty_like(x)
        ws = _workspace(lib, 1, Bn, L, Cn, 0, x.device)
        N.check(lib.ub_linear_recurrence(af.data_ptr(), int(per_step), x.data_ptr(), out.data_ptr(), _p(state), Bn, L, Cn,
                                         int(one_minus), _p(ws), _st(x)), "ub_linear_recurrence")
        return out
    af, xf = a.float(), x.float()
    h = state.float().clone() if state is not None else torch.zeros(Bn, Cn, device=x.device)
    ys = []
    for l in range(L):
        al = af[:, l] if per_step else af
        h = al * h + ((1 - al) if one_minus else 1.0) * xf[:, l]
        ys.append(h)
    if state is not None:
        state.copy_(h)
    return torch.stack(ys, 1).to(x.dtype)


def wkv4_new_state(B: int, C_: int, device) -> torch.Tensor:
    s = torch.zeros(B, 3, C_, dtype=torch.float32, device=device)
    s[:, 2] = -1e38
    return s


def wkv4(k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor, state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RWKV-4 time mixing core.  ``k, v`` [B, L, C]; ``w`` = -exp(time_decay) [C]; ``u`` = time_first [C];
    ``state`` fp32 [B, 3, C] = (aa, bb, pp) (see ``wkv4_new_state``)."""
    Bn, L, Cn = k.shape
    if _use_kernel(k):
        lib, N = _lib()
        k, v = k.contiguous(), v.contiguous()
        out = torch.empty_like(k)
        wf, uf = _f32c(w), _f32c(u)
        ws = _workspace(lib, 2, Bn, L, Cn, 0, k.device)
        N.check(lib.ub_wkv4(k.data_ptr(), v.data_ptr(), wf.data_ptr(), uf.data_ptr(), out.data_ptr(), _p(state), Bn, L, Cn,
                            _p(ws), _st(k)), "ub_wkv4")
        return out
    kf, vf, wf, uf = k.float(), v.float(), w.float(), u.float()
    if state is not None:
        aa, bb, pp = state[:, 0].float().clone(), state[:, 1].float().clone(), state[:, 2].float().clone()
    else:
        aa = torch.zeros(Bn, Cn, device=k.device)
        bb = torch.zeros(Bn, Cn, device=k.device)
        pp = torch.full((Bn, Cn), -1e38, device=k.device)
    ys = []
    for l in range(L):
        kk, vv = kf[:, l], vf[:, l]
        ww = uf + kk
        p = torch.maximum(pp, ww)
        e1, e2 = torch.exp(pp - p), torch.exp(ww - p)
        ys.append((e1 * aa + e2 * vv) / (e1 * bb + e2))
        ww = pp + wf
        p = torch.maximum(ww, kk)
        e1, e2 = torch.exp(ww - p), torch.exp(kk - p)
        aa, bb, pp = e1 * aa + e2 * vv, e1 * bb + e2, p
    if state is not None:
        state[:, 0], state[:, 1], state[:, 2] = aa, bb, pp
    return torch.stack(ys, 1).to(k.dtype)


def wkv6(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor, num_heads: int,
         state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RWKV-6 core.  ``r, k, v`` [B, L, H*Dh]; ``w`` fp32 [B, L, H*Dh] pre-activation decay (decay = exp(-exp(w)));
    ``u`` [H*Dh]; ``state`` fp32 [B, H, Dh, Dh] (key index first)."""
    Bn, L, Cn = r.shape
    H = num_heads
    Dh = Cn // H
    if _use_kernel(r) and Dh in (32, 64):
        lib, N = _lib()
        r, k, v = r.contiguous(), k.contiguous(), v.contiguous()
        wf, uf = _f32c(w), _f32c(u)
        out = torch.empty_like(r)
        ws = _workspace(lib, 3, Bn, L, H, Dh, r.device)
        N.check(lib.ub_wkv6(r.data_ptr(), k.data_ptr(), v.data_ptr(), wf.data_ptr(), uf.data_ptr(), out.data_ptr(), _p(state),
                            Bn, L, H, Dh, _p(ws), _st(r)), "ub_wkv6")
        return out
    rf, kf, vf = (t.float().view(Bn, L, H, Dh) for t in (r, k, v))
    dec = torch.exp(-torch.exp(w.float())).view(Bn, L, H, Dh)
    uf = u.float().view(H, Dh)
    S = state.float().clone() if state is not None else torch.zeros(Bn, H, Dh, Dh, device=r.device)
    ys = []
    for l in range(L):
        kv = kf[:, l, :, :, None] * vf[:, l, :, None, :]                  # [B, H, Dh(i), Dh(j)]
        ys.append(torch.einsum("bhi,bhij->bhj", rf[:, l], S + uf[None, :, :, None] * kv))
        S = S * dec[:, l, :, :, None] + kv
    if state is not None:
        state.copy_(S)
    return torch.stack(ys, 1).reshape(Bn, L, Cn).to(r.dtype)
