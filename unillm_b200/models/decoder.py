"""``DecoderModel``: the parametric decoder-only transformer behind most of the model zoo.

Parameters live in a flat dict under canonical names (``embed``, ``layers.{i}.wqkv``, ``layers.{i}.wo``,
``layers.{i}.w_gate_up`` ...).  Q, K and V are always fused into one ``[(Hq + 2 Hkv) * D, H]`` matrix and
gate / up into one ``[2 I, H]`` matrix at load time -- one GEMM each on the device -- whatever packing
the family uses on disk; ``KeyScheme`` describes the on-disk names and ``export_hf`` writes them back.

``forward`` / ``forward_with_cache`` here are the straightforward PyTorch statement of the math and
serve as the numerical oracle (fp32 on CPU) and as the generic path for long-tail families; the
serving engine runs the same parameters through the fused sm_100a kernels with a paged KV cache
(``unillm_b200.engine.runner``).

Reference: ``crates/runtime/src/models_v2/llama.rs`` -- ``forward`` ``:203-236``, ``forward_with_cache``
``:421-464``, layer ``:631-680``, attention ``:921-1156``, MLP ``:1274-1297``, weight loading ``:175-201,
682-747``; the other families as cited in ``unillm_b200/models/families.py``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..kv_cache import KVCache
from ..model_core import Model, ModelInputs, ModelOutputs, ModelWeights, WeightMetadata
from ..precompute import RoPECache, alibi_slopes, apply_rope
from ..tensor_core import ops_fn
from ..types import InvalidInput, LoadingError
from .spec import DecoderSpec, KeyScheme, MoESpec


def _f(x):
    return x.float() if x.dtype in (torch.bfloat16, torch.float16) else x


class DecoderModel(Model):
    """Subclasses set ``config_class``, ``scheme`` and implement ``spec_from_config``."""

    scheme: KeyScheme = KeyScheme()

    def __init__(self, config, reference_quirks: bool = False):
        super().__init__(config)
        self.spec: DecoderSpec = self.spec_from_config(config)
        self.reference_quirks = reference_quirks
        self.p: Dict[str, torch.Tensor] = {}
        self._rope: Optional[RoPECache] = None
        self._alibi: Optional[torch.Tensor] = None

    @classmethod
    def spec_from_config(cls, config) -> DecoderSpec:  # pragma: no cover - abstract
        raise NotImplementedError

    # ------------------------------------------------------------------------------------------
    # parameter inventory
    # ------------------------------------------------------------------------------------------
    def param_shapes(self) -> Dict[str, tuple]:
        s = self.spec
        H, D = s.hidden_size, s.head_dim
        E = s.embed_proj_dim or H
        shp: Dict[str, tuple] = {"embed": (s.vocab_size, E)}
        if s.embed_proj_dim:
            shp["project_in"] = (H, E)
            shp["project_out"] = (E, H)
        if s.pos == "learned":
            shp["pos_embed"] = (s.max_position_embeddings + s.learned_pos_offset, H)
        if s.embed_norm:
            shp["embed_norm.w"] = (H,)
            shp["embed_norm.b"] = (H,)
        for i in range(s.num_layers):
            L = f"layers.{i}."
            shp[L + "ln1.w"] = (H,)
            if s.norm_bias:
                shp[L + "ln1.b"] = (H,)
            if not (s.parallel_residual and s.parallel_shared_norm):
                shp[L + "ln2.w"] = (H,)
                if s.norm_bias:
                    shp[L + "ln2.b"] = (H,)
            shp[L + "wqkv"] = (s.q_size + 2 * s.kv_size, H)
            if s.qkv_bias:
                shp[L + "bqkv"] = (s.q_size + 2 * s.kv_size,)
            if s.qk_norm:
                shp[L + "q_norm"] = (D,)
                shp[L + "k_norm"] = (D,)
            shp[L + "wo"] = (H, s.q_size)
            if s.o_bias:
                shp[L + "bo"] = (H,)
            moe = s.layer_is_moe(i)
            if (not moe) or s.moe.dense_parallel:
                I = s.intermediate_size
                if s.mlp == "gated":
                    shp[L + "w_gate_up"] = (2 * I, H)
                else:
                    shp[L + "w_up"] = (I, H)
                    if s.mlp_bias:
                        shp[L + "b_up"] = (I,)
                shp[L + "w_down"] = (H, I)
                if s.mlp_bias:
                    shp[L + "b_down"] = (H,)
            if moe:
                m = s.moe
                shp[L + "router"] = (m.num_experts, H)
                shp[L + "experts_gate_up"] = (m.num_experts, (2 if m.gated else 1) * m.intermediate_size, H)
                shp[L + "experts_down"] = (m.num_experts, H, m.intermediate_size)
                if m.num_shared_experts:
                    Is = m.num_shared_experts * m.intermediate_size
                    shp[L + "shared_gate_up"] = (2 * Is, H)
                    shp[L + "shared_down"] = (H, Is)
        if s.final_norm:
            shp["final_norm.w"] = (H,)
            if s.norm_bias:
                shp["final_norm.b"] = (H,)
        if not s.tie_embeddings:
            shp["lm_head"] = (s.vocab_size, E)
        if s.lm_head_bias:
            shp["lm_head_bias"] = (s.vocab_size,)
        return shp

    def _init_params(self, init="zeros", seed=0, dtype=torch.float32, device=torch.device("cpu")):
        g = torch.Generator(device="cpu").manual_seed(seed)
        std = self.spec.initializer_range
        self.p = {}
        for name, shape in self.param_shapes().items():
            is_norm_w = name.endswith((".w", "q_norm", "k_norm")) and len(shape) == 1
            if init == "zeros":
                t = torch.zeros(shape, dtype=dtype)
            elif is_norm_w:
                t = torch.zeros(shape, dtype=dtype) if self.spec.norm_weight_offset_one else torch.ones(shape, dtype=dtype)
            elif name.endswith((".b", "bqkv", "bo", "b_up", "b_down", "lm_head_bias")):
                t = torch.zeros(shape, dtype=dtype)
            else:
                t = (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(dtype)
            self.p[name] = t.to(device)
        self.device, self.dtype = device, dtype
        self._rope = self._alibi = None

    # ------------------------------------------------------------------------------------------
    # loading from / exporting to the family's on-disk names
    # ------------------------------------------------------------------------------------------
    @staticmethod
    def _find(w: ModelWeights, prefixes, names, suffix=".weight"):
        """First present alias; block-quantised (GGUF) tensors are dequantised on the way in."""
        for pre in prefixes:
            for n in names:
                t = w.get(pre + n + suffix)
                if t is not None:
                    return t
                q = w.get_quantized(pre + n + suffix)
                if q is not None:
                    return q.dequantize()
        return None

    def _load(self, weights: ModelWeights, dtype=None, device=None):
        s, k = self.spec, self.scheme
        dtype = dtype or torch.float32
        dev = torch.device(device) if device is not None else torch.device("cpu")
        shapes = self.param_shapes()
        out: Dict[str, torch.Tensor] = {}

        def T(t):
            return t.t() if (k.transposed and t is not None and t.dim() == 2) else t

        def need(t, what):
            if t is None:
                raise LoadingError(f"{type(self).__name__}: missing weight {what}")
            return t

        def deq(name_candidates):
            # quantised GGUF tensors are dequantised here; the engine re-quantises on demand
            for n in name_candidates:
                q = weights.get_quantized(n)
                if q is not None:
                    return q.dequantize()
            return None

        root = ("",)
        out["embed"] = need(self._find(weights, root, k.embed), "embedding " + str(k.embed))
        if s.embed_proj_dim:
            out["project_in"] = need(self._find(weights, root, k.project_in), "project_in")
            out["project_out"] = need(self._find(weights, root, k.project_out), "project_out")
        if s.pos == "learned":
            out["pos_embed"] = need(self._find(weights, root, k.pos_embed), "position embedding")
        if s.embed_norm:
            out["embed_norm.w"] = need(self._find(weights, root, k.embed_norm), "embed norm")
            b = self._find(weights, root, k.embed_norm, ".bias")
            out["embed_norm.b"] = b if b is not None else torch.zeros(s.hidden_size)
        for i in range(s.num_layers):
            L = f"layers.{i}."
            pre = tuple(p.format(i=i) for p in k.layer)
            out[L + "ln1.w"] = need(self._find(weights, pre, k.ln1), f"layer {i} ln1")
            if s.norm_bias:
                b = self._find(weights, pre, k.ln1, ".bias")
                out[L + "ln1.b"] = b if b is not None else torch.zeros(s.hidden_size)
            if L + "ln2.w" in shapes:
                t = self._find(weights, pre, k.ln2)
                out[L + "ln2.w"] = t if t is not None else out[L + "ln1.w"].clone()
                if s.norm_bias:
                    b = self._find(weights, pre, k.ln2, ".bias")
                    out[L + "ln2.b"] = b if b is not None else torch.zeros(s.hidden_size)
            # ---- attention projections ----
            packed = T(self._find(weights, pre, k.qkv)) if k.qkv else None
            pb = self._find(weights, pre, k.qkv, ".bias") if k.qkv else None
            if packed is not None:
                out[L + "wqkv"], bq = self._unpack_qkv(packed, pb)
            else:
                q = T(self._find(weights, pre, k.q))
                kk = T(self._find(weights, pre, k.k))
                v = T(self._find(weights, pre, k.v))
                if q is None:
                    names = [p + n + ".weight" for p in pre for n in k.q]
                    q, kk, v = deq(names), deq([n.replace(k.q[0], k.k[0]) for n in names]), \
                        deq([n.replace(k.q[0], k.v[0]) for n in names])
                need(q, f"layer {i} q_proj"), need(kk, f"layer {i} k_proj"), need(v, f"layer {i} v_proj")
                out[L + "wqkv"] = torch.cat([q, kk, v], dim=0)
                bq = None
                qb = self._find(weights, pre, k.q, ".bias")
                if qb is not None:
                    kb = self._find(weights, pre, k.k, ".bias")
                    vb = self._find(weights, pre, k.v, ".bias")
                    bq = torch.cat([qb, kb if kb is not None else torch.zeros(s.kv_size),
                                    vb if vb is not None else torch.zeros(s.kv_size)])
            if s.qkv_bias:
                out[L + "bqkv"] = bq if bq is not None else torch.zeros(s.q_size + 2 * s.kv_size)
            if s.qk_norm:
                out[L + "q_norm"] = need(self._find(weights, pre, k.q_norm), "q_norm")
                out[L + "k_norm"] = need(self._find(weights, pre, k.k_norm), "k_norm")
            wo = T(self._find(weights, pre, k.o))
            if wo is None:
                wo = deq([p + n + ".weight" for p in pre for n in k.o])
            out[L + "wo"] = need(wo, f"layer {i} o_proj")
            if s.o_bias:
                b = self._find(weights, pre, k.o, ".bias")
                out[L + "bo"] = b if b is not None else torch.zeros(s.hidden_size)
            # ---- MLP ----
            moe = s.layer_is_moe(i)
            if (not moe) or s.moe.dense_parallel:
                if s.mlp == "gated":
                    gu = T(self._find(weights, pre, k.gate_up)) if k.gate_up else None
                    if gu is None:
                        g = T(self._find(weights, pre, k.gate))
                        u = T(self._find(weights, pre, k.up))
                        if g is None:
                            g = deq([p + n + ".weight" for p in pre for n in k.gate])
                            u = deq([p + n + ".weight" for p in pre for n in k.up])
                        gu = torch.cat([need(g, f"layer {i} gate_proj"), need(u, f"layer {i} up_proj")], dim=0)
                    out[L + "w_gate_up"] = gu
                else:
                    out[L + "w_up"] = need(T(self._find(weights, pre, k.up)), f"layer {i} fc1")
                    if s.mlp_bias:
                        b = self._find(weights, pre, k.up, ".bias")
                        out[L + "b_up"] = b if b is not None else torch.zeros(s.intermediate_size)
                dn = T(self._find(weights, pre, k.down))
                if dn is None:
                    dn = deq([p + n + ".weight" for p in pre for n in k.down])
                out[L + "w_down"] = need(dn, f"layer {i} down_proj")
                if s.mlp_bias:
                    b = self._find(weights, pre, k.down, ".bias")
                    out[L + "b_down"] = b if b is not None else torch.zeros(s.hidden_size)
            if moe:
                m = s.moe
                out[L + "router"] = need(self._find(weights, pre, k.router), f"layer {i} router")
                gus, dns = [], []
                for e in range(m.num_experts):
                    epre = tuple(p + x.format(e=e) for p in pre for x in k.expert)
                    g = self._find(weights, epre, k.e_gate)
                    u = self._find(weights, epre, k.e_up) if m.gated else None
                    d = self._find(weights, epre, k.e_down)
                    need(g, f"layer {i} expert {e} gate"), need(d, f"layer {i} expert {e} down")
                    gus.append(torch.cat([g, need(u, f"layer {i} expert {e} up")], 0) if m.gated else g)
                    dns.append(d)
                out[L + "experts_gate_up"] = torch.stack(gus)
                out[L + "experts_down"] = torch.stack(dns)
                if m.num_shared_experts:
                    g = need(self._find(weights, pre, k.shared_gate), "shared gate")
                    u = need(self._find(weights, pre, k.shared_up), "shared up")
                    out[L + "shared_gate_up"] = torch.cat([g, u], 0)
                    out[L + "shared_down"] = need(self._find(weights, pre, k.shared_down), "shared down")
        if s.final_norm:
            out["final_norm.w"] = need(self._find(weights, root, k.final_norm), "final norm")
            if s.norm_bias:
                b = self._find(weights, root, k.final_norm, ".bias")
                out["final_norm.b"] = b if b is not None else torch.zeros(s.hidden_size)
        if not s.tie_embeddings:
            lm = self._find(weights, root, k.lm_head)
            if lm is None:
                lm = deq([n + ".weight" for n in k.lm_head])
            out["lm_head"] = lm if lm is not None else out["embed"]
        if s.lm_head_bias:
            b = self._find(weights, root, k.lm_head, ".bias")
            out["lm_head_bias"] = b if b is not None else torch.zeros(s.vocab_size)
        for name, shape in shapes.items():
            if name not in out:
                raise LoadingError(f"internal: parameter {name} was not produced by the loader")
            if tuple(out[name].shape) != tuple(shape):
                raise LoadingError(f"{name}: expected shape {tuple(shape)}, file has {tuple(out[name].shape)}")
        self.p = {n: t.to(device=dev, dtype=dtype).contiguous() for n, t in out.items() if n in shapes}
        self.device, self.dtype = dev, dtype
        self._rope = self._alibi = None

    def _unpack_qkv(self, w: torch.Tensor, b: Optional[torch.Tensor]):
        """On-disk packed QKV -> canonical [Q; K; V] row order."""
        s, lay = self.spec, self.scheme.qkv_layout
        D, Hq, Hkv = s.head_dim, s.num_heads, s.num_kv_heads
        if lay == "concat":
            return w, b
        if lay == "per_head":        # [h][q, k, v] (GPT-NeoX, BLOOM); MHA only
            wr = w.reshape(Hq, 3, D, -1)
            w2 = torch.cat([wr[:, 0].reshape(Hq * D, -1), wr[:, 1].reshape(Hq * D, -1), wr[:, 2].reshape(Hq * D, -1)])
            b2 = None
            if b is not None:
                br = b.reshape(Hq, 3, D)
                b2 = torch.cat([br[:, 0].reshape(-1), br[:, 1].reshape(-1), br[:, 2].reshape(-1)])
            return w2, b2
        if lay == "grouped":         # [kv group][G q heads, k, v] (Falcon new decoder architecture)
            G = Hq // Hkv
            wr = w.reshape(Hkv, G + 2, D, -1)
            w2 = torch.cat([wr[:, :G].reshape(Hq * D, -1), wr[:, G].reshape(Hkv * D, -1), wr[:, G + 1].reshape(Hkv * D, -1)])
            b2 = None
            if b is not None:
                br = b.reshape(Hkv, G + 2, D)
                b2 = torch.cat([br[:, :G].reshape(-1), br[:, G].reshape(-1), br[:, G + 1].reshape(-1)])
            return w2, b2
        raise LoadingError(f"unknown qkv layout {lay}")

    def _pack_qkv(self, w: torch.Tensor) -> torch.Tensor:
        """Inverse of ``_unpack_qkv`` for weights (used by ``export_hf``)."""
        s, lay = self.spec, self.scheme.qkv_layout
        D, Hq, Hkv = s.head_dim, s.num_heads, s.num_kv_heads
        if lay == "concat":
            return w
        q, k, v = w[:Hq * D], w[Hq * D:Hq * D + Hkv * D], w[Hq * D + Hkv * D:]
        if lay == "per_head":
            return torch.stack([q.reshape(Hq, D, -1), k.reshape(Hq, D, -1), v.reshape(Hq, D, -1)], 1).reshape(3 * Hq * D, -1)
        G = Hq // Hkv
        return torch.cat([q.reshape(Hkv, G, D, -1), k.reshape(Hkv, 1, D, -1), v.reshape(Hkv, 1, D, -1)], 1).reshape((Hq + 2 * Hkv) * D, -1)

    def export_hf(self) -> ModelWeights:
        """Parameters under the family's on-disk names (first alias of each scheme entry)."""
        s, k = self.spec, self.scheme
        out: Dict[str, torch.Tensor] = {}

        def T(t):
            return t.t().contiguous() if k.transposed and t.dim() == 2 else t

        out[k.embed[0] + ".weight"] = self.p["embed"]
        if s.embed_proj_dim:
            out[k.project_in[0] + ".weight"] = self.p["project_in"]
            out[k.project_out[0] + ".weight"] = self.p["project_out"]
        if s.pos == "learned":
            out[k.pos_embed[0] + ".weight"] = self.p["pos_embed"]
        if s.embed_norm:
            out[k.embed_norm[0] + ".weight"] = self.p["embed_norm.w"]
            out[k.embed_norm[0] + ".bias"] = self.p["embed_norm.b"]
        for i in range(s.num_layers):
            L, pre = f"layers.{i}.", k.layer[0].format(i=i)
            out[pre + k.ln1[0] + ".weight"] = self.p[L + "ln1.w"]
            if s.norm_bias:
                out[pre + k.ln1[0] + ".bias"] = self.p[L + "ln1.b"]
            if L + "ln2.w" in self.p:
                out[pre + k.ln2[0] + ".weight"] = self.p[L + "ln2.w"]
                if s.norm_bias:
                    out[pre + k.ln2[0] + ".bias"] = self.p[L + "ln2.b"]
            wqkv = self.p[L + "wqkv"]
            if k.qkv:
                out[pre + k.qkv[0] + ".weight"] = T(self._pack_qkv(wqkv))
                if s.qkv_bias:
                    out[pre + k.qkv[0] + ".bias"] = self._pack_qkv(self.p[L + "bqkv"][:, None])[:, 0]
            else:
                q, kk, v = wqkv.split([s.q_size, s.kv_size, s.kv_size])
                out[pre + k.q[0] + ".weight"], out[pre + k.k[0] + ".weight"], out[pre + k.v[0] + ".weight"] = T(q), T(kk), T(v)
                if s.qkv_bias:
                    qb, kb, vb = self.p[L + "bqkv"].split([s.q_size, s.kv_size, s.kv_size])
                    out[pre + k.q[0] + ".bias"], out[pre + k.k[0] + ".bias"], out[pre + k.v[0] + ".bias"] = qb, kb, vb
            if s.qk_norm:
                out[pre + k.q_norm[0] + ".weight"] = self.p[L + "q_norm"]
                out[pre + k.k_norm[0] + ".weight"] = self.p[L + "k_norm"]
            out[pre + k.o[0] + ".weight"] = T(self.p[L + "wo"])
            if s.o_bias:
                out[pre + k.o[0] + ".bias"] = self.p[L + "bo"]
            if L + "w_gate_up" in self.p:
                if k.gate_up:
                    out[pre + k.gate_up[0] + ".weight"] = T(self.p[L + "w_gate_up"])
                else:
                    g, u = self.p[L + "w_gate_up"].chunk(2, 0)
                    out[pre + k.gate[0] + ".weight"], out[pre + k.up[0] + ".weight"] = T(g), T(u)
            if L + "w_up" in self.p:
                out[pre + k.up[0] + ".weight"] = T(self.p[L + "w_up"])
                if s.mlp_bias:
                    out[pre + k.up[0] + ".bias"] = self.p[L + "b_up"]
            if L + "w_down" in self.p:
                out[pre + k.down[0] + ".weight"] = T(self.p[L + "w_down"])
                if s.mlp_bias:
                    out[pre + k.down[0] + ".bias"] = self.p[L + "b_down"]
            if L + "router" in self.p:
                m = s.moe
                out[pre + k.router[0] + ".weight"] = self.p[L + "router"]
                for e in range(m.num_experts):
                    ep = pre + k.expert[0].format(e=e)
                    gu = self.p[L + "experts_gate_up"][e]
                    if m.gated:
                        g, u = gu.chunk(2, 0)
                        out[ep + k.e_gate[0] + ".weight"], out[ep + k.e_up[0] + ".weight"] = g, u
                    else:
                        out[ep + k.e_gate[0] + ".weight"] = gu
                    out[ep + k.e_down[0] + ".weight"] = self.p[L + "experts_down"][e]
                if m.num_shared_experts:
                    g, u = self.p[L + "shared_gate_up"].chunk(2, 0)
                    out[pre + k.shared_gate[0] + ".weight"], out[pre + k.shared_up[0] + ".weight"] = g, u
                    out[pre + k.shared_down[0] + ".weight"] = self.p[L + "shared_down"]
        if s.final_norm:
            out[k.final_norm[0] + ".weight"] = self.p["final_norm.w"]
            if s.norm_bias:
                out[k.final_norm[0] + ".bias"] = self.p["final_norm.b"]
        if not s.tie_embeddings:
            out[k.lm_head[0] + ".weight"] = self.p["lm_head"]
        if s.lm_head_bias:
            out[k.lm_head[0] + ".bias"] = self.p["lm_head_bias"]
        md = WeightMetadata(architecture=type(self._config).__name__, total_params=sum(t.numel() for t in out.values()),
                            format="memory", dtype=str(self.dtype))
        return ModelWeights({n: t.contiguous() for n, t in out.items()}, md)

    def parameters(self) -> Dict[str, torch.Tensor]:
        return self.p

    def _move(self, dev, dtype):
        self.p = {n: (t.to(device=dev, dtype=dtype) if dtype is not None else t.to(dev)) for n, t in self.p.items()}
        self._rope = self._alibi = None

    # ------------------------------------------------------------------------------------------
    # math
    # ------------------------------------------------------------------------------------------
    def _norm(self, x, name, layer_level=True):
        s = self.spec
        w, b = self.p[name + ".w"], self.p.get(name + ".b")
        eps = s.norm_eps
        if self.reference_quirks:
            if layer_level and s.ref_layer_eps is not None:
                eps = s.ref_layer_eps
            if s.ref_ln_star:
                return ops_fn.layer_norm(x, w, None, eps)
        if s.norm == "layer":
            return ops_fn.layer_norm(x, w, b, eps)
        if s.norm_weight_offset_one:
            return ops_fn.rms_norm(x, (w.float() + 1.0).to(w.dtype), eps)
        return ops_fn.rms_norm(x, w, eps)

    def _rope_cache(self, need_len: int) -> RoPECache:
        s = self.spec
        if self._rope is None or self._rope.max_seq_len < need_len or self._rope.cos.device != self.device:
            n = max(need_len, min(s.max_position_embeddings, 8192))
            self._rope = RoPECache(s.head_dim, n, s.rope_theta, rotary_dim=s.rd, position_scale=s.rope_pos_scale,
                                   llama3=s.rope_llama3, device=self.device)
        return self._rope

    def _attention(self, i: int, h: torch.Tensor, past: int, cache: Optional[KVCache]) -> torch.Tensor:
        s = self.spec
        L = f"layers.{i}."
        B, T, _ = h.shape
        qkv = ops_fn.linear(h, self.p[L + "wqkv"], self.p.get(L + "bqkv"))
        q, k, v = qkv.split([s.q_size, s.kv_size, s.kv_size], dim=-1)
        q = q.reshape(B, T, s.num_heads, s.head_dim)
        k = k.reshape(B, T, s.num_kv_heads, s.head_dim)
        v = v.reshape(B, T, s.num_kv_heads, s.head_dim)
        if s.qk_norm:
            q = ops_fn.rms_norm(q, self.p[L + "q_norm"], s.norm_eps)
            k = ops_fn.rms_norm(k, self.p[L + "k_norm"], s.norm_eps)
        if s.pos == "rope" and s.rd > 0:
            cos, sin = self._rope_cache(past + T).get_range(past, past + T)
            q = apply_rope(q, cos, sin, s.rd, s.rope_interleaved)
            k = apply_rope(k, cos, sin, s.rd, s.rope_interleaved)
        k, v = k.transpose(1, 2), v.transpose(1, 2)      # [B, Hkv, T, D]
        if cache is not None:
            lc = cache.layer(i)
            lc.append(k, v)
            k, v = lc.get_kv()
        q = q.transpose(1, 2)                             # [B, Hq, T, D]
        S = k.shape[2]
        g = s.num_heads // s.num_kv_heads
        kf, vf = _f(k), _f(v)
        if g > 1:
            kf, vf = kf.repeat_interleave(g, dim=1), vf.repeat_interleave(g, dim=1)
        scale = s.attn_scale if s.attn_scale is not None else 1.0 / math.sqrt(s.head_dim)
        qpos = torch.arange(past, past + T, device=h.device)[:, None]
        kpos = torch.arange(S, device=h.device)[None, :]
        vis = kpos <= qpos
        if s.window > 0:
            vis = vis & (kpos > qpos - s.window)
        bias = torch.zeros(T, S, device=h.device, dtype=torch.float32).masked_fill(~vis, float("-inf"))
        if s.pos == "alibi":
            if self._alibi is None or self._alibi.device != h.device:
                self._alibi = alibi_slopes(s.num_heads).to(h.device)
            bias = bias[None] + self._alibi[:, None, None] * (kpos - qpos)[None].float()
        y = F.scaled_dot_product_attention(_f(q), kf, vf, attn_mask=bias, scale=scale)
        y = y.transpose(1, 2).reshape(B, T, s.q_size).to(h.dtype)
        return ops_fn.linear(y, self.p[L + "wo"], self.p.get(L + "bo"))

    def _dense_mlp(self, x, w_gate_up=None, w_up=None, b_up=None, w_down=None, b_down=None, act="silu"):
        if w_gate_up is not None:
            gu = ops_fn.linear(x, w_gate_up)
            g, u = gu.chunk(2, dim=-1)
            hdn = (ops_fn.activation(act)(_f(g)) * _f(u)).to(x.dtype)
        else:
            hdn = ops_fn.activation(act)(_f(ops_fn.linear(x, w_up, b_up))).to(x.dtype)
        return ops_fn.linear(hdn, w_down, b_down)

    def _moe(self, i: int, x: torch.Tensor) -> torch.Tensor:
        s, m = self.spec, self.spec.moe
        L = f"layers.{i}."
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        logits = F.linear(_f(x2), _f(self.p[L + "router"]))
        if m.normalize_topk:
            v, idx = torch.topk(logits, m.top_k, dim=-1)
            w = torch.softmax(v, dim=-1)
        else:
            w, idx = torch.topk(torch.softmax(logits, dim=-1), m.top_k, dim=-1)
        out = torch.zeros(x2.shape, dtype=torch.float32, device=x.device)
        gu, dn = self.p[L + "experts_gate_up"], self.p[L + "experts_down"]
        for e in range(m.num_experts):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            if m.gated:
                y = self._dense_mlp(x2[tok], w_gate_up=gu[e], w_down=dn[e], act=m.act)
            else:
                y = self._dense_mlp(x2[tok], w_up=gu[e], w_down=dn[e], act=m.act)
            out.index_add_(0, tok, _f(y) * w[tok, slot].unsqueeze(-1))
        if m.num_shared_experts:
            out = out + _f(self._dense_mlp(x2, w_gate_up=self.p[L + "shared_gate_up"], w_down=self.p[L + "shared_down"],
                                           act=m.act))
        return out.to(x.dtype).reshape(shape)

    def _mlp(self, i: int, x: torch.Tensor) -> torch.Tensor:
        s = self.spec
        L = f"layers.{i}."
        y = None
        if L + "w_down" in self.p:
            y = self._dense_mlp(x, self.p.get(L + "w_gate_up"), self.p.get(L + "w_up"), self.p.get(L + "b_up"),
                                self.p[L + "w_down"], self.p.get(L + "b_down"), s.act)
        if s.layer_is_moe(i):
            mo = self._moe(i, x)
            y = mo if y is None else y + mo
        return y

    def _layer(self, i: int, x: torch.Tensor, past: int, cache: Optional[KVCache]) -> torch.Tensor:
        s = self.spec
        L = f"layers.{i}."
        rs = s.residual_scale
        if s.post_ln:
            x = self._norm(x + self._attention(i, x, past, cache) * rs, L + "ln1")
            return self._norm(x + self._mlp(i, x) * rs, L + "ln2")
        h = self._norm(x, L + "ln1")
        a = self._attention(i, h, past, cache)
        if s.parallel_residual:
            m_in = h if s.parallel_shared_norm else self._norm(x, L + "ln2")
            return x + (a + self._mlp(i, m_in)) * rs
        x = x + a * rs
        return x + self._mlp(i, self._norm(x, L + "ln2")) * rs

    def hidden_states(self, input_ids: torch.Tensor, cache: Optional[KVCache] = None,
                      inputs_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        s = self.spec
        if input_ids is not None and input_ids.dim() != 2:
            raise InvalidInput("input_ids must be [batch, seq]")
        past = cache.seq_len() if cache is not None else 0
        if inputs_embeds is None:
            if int(input_ids.max()) >= s.vocab_size or int(input_ids.min()) < 0:
                raise InvalidInput("token id out of range")
            x = ops_fn.embedding(input_ids.to(self.device), self.p["embed"])
            if s.embed_proj_dim:
                x = ops_fn.linear(x, self.p["project_in"])
            if s.embed_scale != 1.0:
                x = (_f(x) * s.embed_scale).to(x.dtype)
        else:
            x = inputs_embeds
        T = x.shape[1]
        if s.pos == "learned":
            pos = torch.arange(past, past + T, device=self.device) + s.learned_pos_offset
            x = x + self.p["pos_embed"][pos][None]
        if s.embed_norm:
            x = ops_fn.layer_norm(x, self.p["embed_norm.w"], self.p["embed_norm.b"], s.norm_eps)
        for i in range(s.num_layers):
            x = self._layer(i, x, past, cache)
        if cache is not None:
            cache.set_seq_len(past + T)
        if s.final_norm:
            x = self._norm(x, "final_norm", layer_level=False)
        return x

    def lm_logits(self, x: torch.Tensor) -> torch.Tensor:
        s = self.spec
        if s.embed_proj_dim:
            x = ops_fn.linear(x, self.p["project_out"])
        w = self.p["embed"] if s.tie_embeddings else self.p["lm_head"]
        y = ops_fn.linear(x, w, self.p.get("lm_head_bias"))
        if s.logit_scale != 1.0:
            y = (_f(y) * s.logit_scale).to(y.dtype)
        return y

    def forward(self, inputs: ModelInputs) -> ModelOutputs:
        if inputs.input_ids is None:
            raise InvalidInput(f"{type(self).__name__} takes text inputs")
        x = self.hidden_states(inputs.input_ids)
        return ModelOutputs.from_logits(self.lm_logits(x), hidden_states=x)

    def new_cache(self, max_seq_len: Optional[int] = None) -> KVCache:
        return KVCache(self.spec.num_layers, max_seq_len or max(2048, min(self.spec.max_position_embeddings, 8192)))

    def forward_with_cache(self, input_ids: torch.Tensor, cache: Optional[KVCache] = None) -> torch.Tensor:
        """Logits ``[B, T_new, V]`` for the new tokens only; keys / values are appended to ``cache``."""
        if input_ids.dim() == 1:
            input_ids = input_ids[None]
        return self.lm_logits(self.hidden_states(input_ids, cache))

    def generate_with_cache(self, prompt: str, config=None) -> str:
        return self.generate(prompt, config)
