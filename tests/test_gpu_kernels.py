"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

from tests.gpu_util import make_paged_cache, ref_attention

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _check_err_word():
    yield
    from unillm_b200.ops import cuda_ops

    torch.cuda.synchronize()
    cuda_ops.check_device_errors()


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).cuda()


def _close(got, ref, rtol=2e-2, atol=2e-2):
    got, ref = got.float().cpu(), ref.float().cpu()
    err = (got - ref).abs()
    tol = atol + rtol * ref.abs()
    bad = (err > tol).sum().item()
    assert bad == 0, f"{bad}/{err.numel()} elements off; max err {err.max().item():.4g}, ref max {ref.abs().max().item():.4g}"


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (16, 256, 512), (7, 384, 4096), (33, 1024, 1024),
                                   (100, 4096, 4096), (128, 6144, 4096), (256, 4096, 14336), (300, 520, 264),
                                   (1024, 2048, 2048), (2000, 768, 3072)])
def test_gemm_tn(M, N, K):
    from unillm_b200.ops import cuda_ops

    x, w = _rand(M, K, seed=1), _rand(N, K, scale=1 / math.sqrt(K), seed=2)
    y = cuda_ops.gemm_tn(x, w)
    ref = x.float() @ w.float().t()
    _close(y, ref)


@pytest.mark.parametrize("tile", [16, 32, 64, 128, 256])
def test_gemm_tile_variants(tile):
    from unillm_b200.ops import cuda_ops

    M, N, K = 260, 640, 1088
    x, w = _rand(M, K, seed=3), _rand(N, K, scale=1 / math.sqrt(K), seed=4)
    y = cuda_ops.gemm_tn(x, w, tile_tokens=tile)
    _close(y, x.float() @ w.float().t())


@pytest.mark.parametrize("splits", [2, 4, 8])
@pytest.mark.parametrize("M,N,K,dual", [(256, 768, 4096, 0), (40, 512, 1792, 0), (256, 1792, 4096, 1), (16, 256, 8192, 1)])
def test_gemm_splitk_cluster(splits, M, N, K, dual):
    from unillm_b200.ops import cuda_ops

    x = _rand(M, K, seed=21)
    w = _rand(N * (2 if dual else 1), K, scale=1 / math.sqrt(K), seed=22)
    b, r = _rand(N, seed=23), _rand(M, N, seed=24)
    if dual:
        y = cuda_ops.gemm_tn(x, w, dual_rows=N, act="silu", splits=splits, residual=r)
        ref = torch.nn.functional.silu(x.float() @ w[:N].float().t()) * (x.float() @ w[N:].float().t()) + r.float()
    else:
        y = cuda_ops.gemm_tn(x, w, bias=b, residual=r, splits=splits)
        ref = x.float() @ w.float().t() + b.float() + r.float()
    _close(y, ref)
    y2 = cuda_ops.gemm_tn(x, w, dual_rows=N, act="silu", splits=splits, residual=r) if dual else \
        cuda_ops.gemm_tn(x, w, bias=b, residual=r, splits=splits)
    assert torch.equal(y, y2)


def test_gemm_bias_residual_act_f32():
    from unillm_b200.ops import cuda_ops

    M, N, K = 77, 512, 768
    x, w = _rand(M, K, seed=5), _rand(N, K, scale=1 / math.sqrt(K), seed=6)
    b, r = _rand(N, seed=7), _rand(M, N, seed=8)
    y = cuda_ops.gemm_tn(x, w, bias=b, residual=r, act="gelu")
    ref = torch.nn.functional.gelu(x.float() @ w.float().t() + b.float()) + r.float()
    _close(y, ref)
    y32 = cuda_ops.gemm_tn(x, w, out_dtype=torch.float32)
    assert y32.dtype == torch.float32
    _close(y32, x.float() @ w.float().t(), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("M", [5, 64, 130, 512])
@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_gemm_dual_swiglu(M, act):
    from unillm_b200.ops import cuda_ops

    K, I = 1024, 1408
    x, w = _rand(M, K, seed=9), _rand(2 * I, K, scale=1 / math.sqrt(K), seed=10)
    y = cuda_ops.gemm_tn(x, w, dual_rows=I, act=act)
    g = x.float() @ w[:I].float().t()
    u = x.float() @ w[I:].float().t()
    f = torch.nn.functional.silu if act == "silu" else (lambda t: torch.nn.functional.gelu(t, approximate="tanh"))
    _close(y, f(g) * u)


def test_gemm_deterministic():
    from unillm_b200.ops import cuda_ops

    x, w = _rand(200, 2048, seed=11), _rand(1536, 2048, scale=0.02, seed=12)
    a = cuda_ops.gemm_tn(x, w)
    b = cuda_ops.gemm_tn(x, w)
    assert torch.equal(a, b)


@pytest.mark.parametrize("kind", ["rms", "layer"])
@pytest.mark.parametrize("H", [64, 1000, 4096, 8192])
def test_norm(kind, H):
    from unillm_b200.ops import cuda_ops

    T = 37
    x, r, w, b = _rand(T, H, seed=1), _rand(T, H, seed=2), _rand(H, seed=3), _rand(H, seed=4)
    y, h = cuda_ops.norm(x, w, bias=b if kind == "layer" else None, residual=r, eps=1e-5, kind=kind,
                         want_residual_out=True)
    hr = (x.float() + r.float()).to(torch.bfloat16).float()
    if kind == "rms":
        ref = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    else:
        ref = torch.nn.functional.layer_norm(hr, (H,), w.float(), b.float(), 1e-5)
    _close(h, hr, rtol=0, atol=0)
    _close(y, ref)


def _ref_rope(x, pos, theta, rd, interleaved=False):
    # x [T, H, D] fp32
    T, H, D = x.shape
    half = rd // 2
    inv = theta ** (-torch.arange(half).float() * 2 / rd)
    ang = pos.float()[:, None] * inv[None]
    c, s = ang.cos()[:, None], ang.sin()[:, None]
    out = x.clone()
    if interleaved:
        x0, x1 = x[..., 0:rd:2], x[..., 1:rd:2]
        out[..., 0:rd:2] = x0 * c - x1 * s
        out[..., 1:rd:2] = x1 * c + x0 * s
    else:
        x0, x1 = x[..., :half], x[..., half:rd]
        out[..., :half] = x0 * c - x1 * s
        out[..., half:rd] = x1 * c + x0 * s
    return out


@pytest.mark.parametrize("D,rd,inter", [(128, 128, False), (64, 32, False), (128, 64, True)])
def test_rope_kv_append(D, rd, inter):
    from unillm_b200.ops import cuda_ops

    T, Hq, Hkv, bs, nb = 21, 8, 2, 16, 9
    qkv = _rand(T, (Hq + 2 * Hkv) * D, seed=1)
    pos = torch.randint(0, 5000, (T,), dtype=torch.int32)
    slots = torch.randperm(nb * bs)[:T].to(torch.int32)
    kc = torch.zeros(nb, Hkv, bs, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    src = qkv.clone().float().cpu().view(T, Hq + 2 * Hkv, D)
    cuda_ops.rope_kv_append(qkv, pos.cuda(), slots.cuda(), kc, vc, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                            rotary_dim=rd, theta=10000.0, interleaved=inter)
    ref_qk = _ref_rope(src[:, :Hq + Hkv], pos, 10000.0, rd, inter)
    got = qkv.float().cpu().view(T, Hq + 2 * Hkv, D)
    _close(got[:, :Hq + Hkv], ref_qk, rtol=1e-2, atol=1e-2)
    _close(got[:, Hq + Hkv:], src[:, Hq + Hkv:], rtol=0, atol=0)
    for t in range(T):
        blk, off = int(slots[t]) // bs, int(slots[t]) % bs
        _close(kc[blk, :, off].cpu(), got[t, Hq:Hq + Hkv], rtol=0, atol=0)
        _close(vc[blk, :, off].cpu(), src[t, Hq + Hkv:].to(torch.bfloat16), rtol=0, atol=0)


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 128), (4, 4, 64), (16, 2, 128), (10, 1, 256)])
@pytest.mark.parametrize("splits", [1, 4])
def test_attn_decode(Hq, Hkv, D, splits):
    from unillm_b200.ops import cuda_ops

    lens = [1, 17, 300, 1000, 64]
    kc, vc, bt, sl, dk, dv = make_paged_cache(len(lens), lens, Hkv, D)
    q = _rand(len(lens), Hq, D, seed=5)
    out, lse = cuda_ops.attn_decode(q, kc, vc, bt, sl, splits=splits, return_lse=True)
    for i, l in enumerate(lens):
        ro, rl = ref_attention(q[i:i + 1].cpu(), dk[i], dv[i], causal_offset=l - 1)
        _close(out[i:i + 1], ro)
        _close(lse[i:i + 1], rl, rtol=1e-2, atol=1e-2)


def test_attn_decode_window_alibi_kvstart():
    from unillm_b200.ops import cuda_ops

    Hq, Hkv, D = 8, 2, 128
    lens = [500, 77]
    kc, vc, bt, sl, dk, dv = make_paged_cache(len(lens), lens, Hkv, D, seed=3)
    q = _rand(len(lens), Hq, D, seed=6)
    slopes = torch.tensor([2 ** (-(i + 1)) for i in range(Hq)], dtype=torch.float32)
    out = cuda_ops.attn_decode(q, kc, vc, bt, sl, window=128, alibi_slopes=slopes.cuda(), splits=2)
    for i, l in enumerate(lens):
        ro, _ = ref_attention(q[i:i + 1].cpu(), dk[i], dv[i], causal_offset=l - 1, window=128, alibi=slopes)
        _close(out[i:i + 1], ro)
    out2 = cuda_ops.attn_decode(q, kc, vc, bt, sl, kv_start=64, splits=1)
    for i, l in enumerate(lens):
        ro, _ = ref_attention(q[i:i + 1].cpu(), dk[i], dv[i], causal_offset=l - 1, kv_start=64)
        _close(out2[i:i + 1], ro)


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 128), (4, 4, 64), (6, 1, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_attn_prefill(Hq, Hkv, D, causal):
    from unillm_b200.ops import cuda_ops

    kv_lens = [130, 64, 700, 33]
    q_lens = [130, 10, 200, 33]     # full prefill, chunk with cached prefix, ...
    kc, vc, bt, sl, dk, dv = make_paged_cache(len(kv_lens), kv_lens, Hkv, D, seed=4)
    qs = [0]
    for l in q_lens:
        qs.append(qs[-1] + l)
    q = _rand(qs[-1], Hq, D, seed=7)
    q_start = torch.tensor(qs, dtype=torch.int32, device="cuda")
    out, lse = cuda_ops.attn_prefill(q, kc, vc, bt, sl, q_start, max(q_lens), causal=causal, return_lse=True)
    for i, (kl, ql) in enumerate(zip(kv_lens, q_lens)):
        ro, rl = ref_attention(q[qs[i]:qs[i + 1]].cpu(), dk[i], dv[i], causal_offset=(kl - ql) if causal else None)
        _close(out[qs[i]:qs[i + 1]], ro)
        _close(lse[qs[i]:qs[i + 1]], rl, rtol=1e-2, atol=1e-2)


def test_attn_prefill_window_and_cascade_merge():
    from unillm_b200.ops import cuda_ops

    Hq, Hkv, D = 8, 2, 128
    kv_lens, q_lens = [400], [400]
    kc, vc, bt, sl, dk, dv = make_paged_cache(1, kv_lens, Hkv, D, seed=5)
    q = _rand(400, Hq, D, seed=8)
    q_start = torch.tensor([0, 400], dtype=torch.int32, device="cuda")
    out = cuda_ops.attn_prefill(q, kc, vc, bt, sl, q_start, 400, causal=True, window=100)
    ro, _ = ref_attention(q.cpu(), dk[0], dv[0], causal_offset=0, window=100)
    _close(out, ro)
    # cascade: keys [0,256) as a bidirectional "shared prefix" pass + suffix pass, merged
    pre_len = torch.tensor([256], dtype=torch.int32, device="cuda")
    oa, la = cuda_ops.attn_prefill(q, kc, vc, bt, pre_len, q_start, 400, causal=False, return_lse=True)
    # the suffix pass is causal over all 400 keys but only sees keys >= 256
    ob, lb = cuda_ops.attn_prefill(q, kc, vc, bt, sl, q_start, 400, causal=True, kv_start=256, return_lse=True)
    merged = cuda_ops.attn_merge(oa, la, ob, lb)
    # reference: rows >= 256 see all keys <= their position; rows < 256 see the whole prefix + nothing else
    ro_full, _ = ref_attention(q.cpu(), dk[0], dv[0], causal_offset=0)
    _close(merged[256:], ro_full[256:])


def test_sample_greedy_and_penalty():
    from unillm_b200.ops import cuda_ops

    B, V = 9, 32000
    logits = _rand(B, V, seed=1)
    ids, vals = cuda_ops.sample(logits, return_vals=True)
    assert torch.equal(ids.cpu().long(), logits.float().argmax(-1).cpu())
    _close(vals, logits.float().max(-1).values, rtol=0, atol=0)
    prev = logits.float().argmax(-1).to(torch.int32)[:, None].contiguous()
    pen = torch.full((B,), 100.0, device="cuda")
    ids2 = cuda_ops.sample(logits, rep_penalty=pen, prev_ids=prev)
    assert (ids2 != ids).all()


def test_sample_topk_topp_distribution():
    from unillm_b200.ops import cuda_ops

    B, V = 512, 1000
    base = torch.randn(V, generator=torch.Generator().manual_seed(3)) * 2
    logits = base[None].repeat(B, 1).cuda()
    temp = torch.full((B,), 0.8, device="cuda")
    topk = torch.full((B,), 5, dtype=torch.int32, device="cuda")
    ids = cuda_ops.sample(logits, temperature=temp, top_k=topk, seed=1234, step=7)
    top5 = set(base.topk(5).indices.tolist())
    assert set(ids.tolist()) <= top5
    assert len(set(ids.tolist())) >= 3          # not degenerate
    ids_again = cuda_ops.sample(logits, temperature=temp, top_k=topk, seed=1234, step=7)
    assert torch.equal(ids, ids_again)          # same (seed, step, row) -> same draw
    topp = torch.full((B,), 0.5, device="cuda")
    ids_p = cuda_ops.sample(logits, temperature=temp, top_p=topp, seed=99, step=1)
    probs = torch.softmax(base / 0.8, -1)
    sp, si = probs.sort(descending=True)
    cut = int((sp.cumsum(0) >= 0.5).nonzero()[0]) + 1
    assert set(ids_p.tolist()) <= set(si[:cut].tolist())
    # temperature only: empirical frequency of the mode is close to its probability
    ids_t = cuda_ops.sample(logits, temperature=temp, seed=5, step=3)
    mode = int(probs.argmax())
    freq = (ids_t == mode).float().mean().item()
    assert abs(freq - probs[mode].item()) < 0.08


def test_eltwise_embed_actmul():
    from unillm_b200.ops import cuda_ops

    x = _rand(33, 1000, seed=1)
    for act, f in [("gelu", torch.nn.functional.gelu), ("silu", torch.nn.functional.silu),
                   ("relu2", lambda t: torch.relu(t) ** 2), ("sigmoid", torch.sigmoid), ("tanh", torch.tanh),
                   ("quick_gelu", lambda t: t * torch.sigmoid(1.702 * t)), ("softplus", torch.nn.functional.softplus)]:
        _close(cuda_ops.eltwise(x, act), f(x.float()))
    _close(cuda_ops.add(x, x, 0.5, 2.0), 2.5 * x.float())
    table = _rand(500, 256, seed=2)
    ids = torch.randint(0, 500, (40,), dtype=torch.int32, device="cuda")
    _close(cuda_ops.embed_gather(ids, table, scale=2.0), table[ids.long()].float() * 2.0)
    gu = _rand(17, 2 * 384, seed=3)
    _close(cuda_ops.act_mul(gu, "silu"), torch.nn.functional.silu(gu[:, :384].float()) * gu[:, 384:].float())
    _close(cuda_ops.l2_normalize(x), torch.nn.functional.normalize(x.float(), dim=-1))


@pytest.mark.parametrize("Hq,Hkv", [(32, 8), (8, 8), (16, 2), (8, 1)])
@pytest.mark.parametrize("causal", [True, False])
def test_attn_prefill_tensor_core_path(Hq, Hkv, causal):
    """Head dim 128 without window / ALiBi runs on the tcgen05 kernel: long and short sequences, chunked prefill
    with a cached prefix, tiles that end inside a page, more than two KV tiles (stage reuse)."""
    from unillm_b200.ops import cuda_ops

    kv_lens = [1100, 17, 300, 129, 640]
    q_lens = [37, 17, 300, 1, 130]
    kc, vc, bt, sl, dk, dv = make_paged_cache(len(kv_lens), kv_lens, Hkv, 128, seed=11)
    qs = [0]
    for l in q_lens:
        qs.append(qs[-1] + l)
    q = _rand(qs[-1], Hq, 128, seed=12)
    q_start = torch.tensor(qs, dtype=torch.int32, device="cuda")
    out, lse = cuda_ops.attn_prefill(q, kc, vc, bt, sl, q_start, max(q_lens), causal=causal, return_lse=True)
    assert cuda_ops.attn_prefill_last_path() == "tcgen05"
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
    for i, (kl, ql) in enumerate(zip(kv_lens, q_lens)):
        ro, rl = ref_attention(q[qs[i]:qs[i + 1]].cpu(), dk[i], dv[i], causal_offset=(kl - ql) if causal else None)
        _close(out[qs[i]:qs[i + 1]], ro)
        _close(lse[qs[i]:qs[i + 1]], rl, rtol=1e-2, atol=1e-2)
    # strided query view (rows of a fused QKV matrix), as the runner passes it
    qkv = _rand(qs[-1], Hq + 2 * Hkv, 128, seed=13)
    out2 = cuda_ops.attn_prefill(qkv[:, :Hq], kc, vc, bt, sl, q_start, max(q_lens), causal=causal)
    for i, (kl, ql) in enumerate(zip(kv_lens, q_lens)):
        ro, _ = ref_attention(qkv[qs[i]:qs[i + 1], :Hq].cpu(), dk[i], dv[i], causal_offset=(kl - ql) if causal else None)
        _close(out2[qs[i]:qs[i + 1]], ro)
    cuda_ops.check_device_errors()


@pytest.mark.parametrize("Hq,Hkv,splits", [(4, 1, 4), (4, 1, 8), (32, 8, 3), (8, 2, 16)])
@pytest.mark.parametrize("causal", [True, False])
def test_attn_prefill_key_split(Hq, Hkv, splits, causal):
    """Key split of the tcgen05 prefill kernel: every CTA walks a share of the KV tiles and a second kernel folds the
    partials.  Compared with the fp32 reference; includes sequences with fewer tiles than splits (empty shares), a
    lower key bound (kv_start) and the strided output of a fused-QKV view."""
    from unillm_b200.ops import cuda_ops

    kv_lens = [1024, 17, 300, 1100]
    q_lens = [260, 17, 40, 1]
    kc, vc, bt, sl, dk, dv = make_paged_cache(len(kv_lens), kv_lens, Hkv, 128, seed=21)
    qs = [0]
    for l in q_lens:
        qs.append(qs[-1] + l)
    q = _rand(qs[-1], Hq, 128, seed=22)
    q_start = torch.tensor(qs, dtype=torch.int32, device="cuda")
    for kv_start in (0, 144):
        out = torch.full((qs[-1], Hq, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        out, lse = cuda_ops.attn_prefill(q, kc, vc, bt, sl, q_start, max(q_lens), causal=causal, return_lse=True,
                                         kv_splits=splits, kv_start=kv_start, out=out)
        assert cuda_ops.attn_prefill_last_path() == "tcgen05"
        torch.cuda.synchronize()
        cuda_ops.check_device_errors()
        for i, (kl, ql) in enumerate(zip(kv_lens, q_lens)):
            ro, rl = ref_attention(q[qs[i]:qs[i + 1]].cpu(), dk[i], dv[i], causal_offset=(kl - ql) if causal else None,
                                   kv_start=kv_start)
            seen = torch.isfinite(rl)                     # rows that see no key at all have lse = -inf and output 0
            oc, lc = out[qs[i]:qs[i + 1]].cpu(), lse[qs[i]:qs[i + 1]].cpu()
            _close(oc[seen], ro[seen])
            _close(lc[seen], rl[seen], rtol=1e-2, atol=1e-2)
            assert torch.all(oc[~seen] == 0)
    # same answer as the unsplit kernel, bit for bit in the log-sum-exp up to fp32 rounding of the fold
    a, la = cuda_ops.attn_prefill(q, kc, vc, bt, sl, q_start, max(q_lens), causal=causal, return_lse=True)
    b, lb = cuda_ops.attn_prefill(q, kc, vc, bt, sl, q_start, max(q_lens), causal=causal, return_lse=True, kv_splits=splits)
    _close(b, a.float(), rtol=2e-2, atol=2e-2)
    _close(lb, la, rtol=1e-3, atol=1e-3)
    cuda_ops.check_device_errors()


@pytest.mark.parametrize("M,N,K,tile", [(256, 512, 512, 256), (512, 1024, 1024, 256), (300, 520, 264, 128), (1000, 2048, 4096, 256),
                                        (128, 768, 1024, 64), (640, 4096, 4096, 0)])
def test_gemm_2cta_pairs(M, N, K, tile):
    """cta_group::2 kernel: tiles of 256 weight rows on CTA pairs; ragged M / N / K edges, several token tiles."""
    from unillm_b200.ops import cuda_ops

    x, w = _rand(M, K, seed=21), _rand(N, K, scale=1 / math.sqrt(K), seed=22)
    out = cuda_ops.gemm_tn(x, w, tile_tokens=tile, cta_pair=2)
    _close(out, x.float() @ w.float().t())
    bias, res = _rand(N, seed=23), _rand(M, N, seed=24)
    out2 = cuda_ops.gemm_tn(x, w, bias=bias, residual=res, act="gelu", tile_tokens=tile, cta_pair=2)
    ref2 = torch.nn.functional.gelu(x.float() @ w.float().t() + bias.float()) + res.float()
    _close(out2, ref2)
    out3 = cuda_ops.gemm_tn(x, w, tile_tokens=tile, cta_pair=2, out_dtype=torch.float32)
    _close(out3, x.float() @ w.float().t())
    assert torch.equal(cuda_ops.gemm_tn(x, w, tile_tokens=tile, cta_pair=2), out)      # deterministic


@pytest.mark.parametrize("M,I,K,tile", [(256, 512, 1024, 128), (500, 1408, 2048, 128), (512, 1024, 1024, 256), (200, 768, 512, 64)])
def test_gemm_2cta_dual(M, I, K, tile):
    from unillm_b200.ops import cuda_ops

    x, w = _rand(M, K, seed=31), _rand(2 * I, K, scale=1 / math.sqrt(K), seed=32)
    out = cuda_ops.gemm_tn(x, w, dual_rows=I, act="silu", tile_tokens=tile, cta_pair=2)
    g, u = x.float() @ w[:I].float().t(), x.float() @ w[I:].float().t()
    _close(out, torch.nn.functional.silu(g) * u)


def test_decode_suffix_persistent_many_items():
    """The persistent suffix-decode kernel with more work items than resident CTAs (every CTA walks over several
    items with the next item's copies in flight), ragged suffix lengths, sequences that end before the suffix
    starts, with and without the fused merge; oracle = fp32 attention over the visible keys."""
    from unillm_b200.ops import cuda_ops

    Hq, Hkv, D, P, B = 16, 4, 128, 64, 160                 # 160 x 4 = 640 items > 3 x 148 CTAs
    g = torch.Generator().manual_seed(5)
    kv_lens = [int(v) for v in torch.randint(P + 1, P + 200, (B,), generator=g)]
    kv_lens[3], kv_lens[77] = P, P - 7                      # nothing behind the prefix
    kc, vc, bt, sl, dk, dv = make_paged_cache(B, kv_lens, Hkv, D, seed=43)
    q = _rand(B, Hq, D, seed=44)
    out, lse = cuda_ops.attn_decode(q, kc, vc, bt, sl, kv_start=P, splits=1, return_lse=True)
    oa = _rand(B, Hq, D, seed=45)
    la = torch.randn(B, Hq, generator=torch.Generator().manual_seed(46)).cuda()
    fused = cuda_ops.attn_decode(q, kc, vc, bt, sl, kv_start=P, splits=1, merge=(oa, la))
    sep = cuda_ops.attn_merge(oa, la, out, lse)
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
    for i in (0, 1, 2, 3, 50, 77, 78, 158, 159):
        l = kv_lens[i]
        if l <= P:
            assert out[i].abs().max().item() == 0.0 and torch.isinf(lse[i]).all()
            continue
        ro, _ = ref_attention(q[i:i + 1].cpu(), dk[i], dv[i], causal_offset=l - 1, kv_start=P)
        _close(out[i:i + 1], ro)
    _close(fused, sep, rtol=2e-2, atol=1e-2)
    # the one-item-per-CTA kernel gives the same answer
    import os, subprocess, sys
    code = ("import torch,sys;sys.path.insert(0,%r);from tests.test_gpu_kernels import make_paged_cache,_rand;"
            "from unillm_b200.ops import cuda_ops;"
            "kc,vc,bt,sl,dk,dv=make_paged_cache(%d,%r,%d,%d,seed=43);q=_rand(%d,%d,%d,seed=44);"
            "o=cuda_ops.attn_decode(q,kc,vc,bt,sl,kv_start=%d,splits=1);torch.save(o.cpu(),sys.argv[1])"
            % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))), B, kv_lens, Hkv, D, B, Hq, D, P))
    import tempfile
    with tempfile.TemporaryDirectory() as td:
        f = os.path.join(td, "o.pt")
        r = subprocess.run([sys.executable, "-c", code, f], env=dict(os.environ, UB_DECODE_PERSIST="0"),
                           capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        ref = torch.load(f)
    _close(out.cpu(), ref.float(), rtol=1e-2, atol=5e-3)


def test_attention_fused_merge_matches_separate_merge():
    """Suffix kernels that fold a prefix partial into their output == suffix partial + merge kernel == full attention."""
    from unillm_b200.ops import cuda_ops

    Hq, Hkv, D, P = 16, 4, 128, 256                       # P keys of shared prefix (here: simply the first P keys)
    kv_lens = [300, 257, 512, 290, 400, 333, 270, 260]
    kc, vc, bt, sl, dk, dv = make_paged_cache(len(kv_lens), kv_lens, Hkv, D, seed=41)
    B = len(kv_lens)
    q = _rand(B, Hq, D, seed=42)
    plen = torch.tensor([P], dtype=torch.int32, device="cuda")
    qs_all = torch.tensor([0, B], dtype=torch.int32, device="cuda")
    # decode: the prefix partial uses sequence 0's first P keys for everybody, so build the reference the same way
    oa, la = cuda_ops.attn_prefill(q, kc, vc, bt[:1], plen, qs_all, B, causal=False, return_lse=True)
    ob, lb = cuda_ops.attn_decode(q, kc, vc, bt, sl, kv_start=P, splits=1, return_lse=True)
    sep = cuda_ops.attn_merge(oa, la, ob, lb)
    fused = cuda_ops.attn_decode(q, kc, vc, bt, sl, kv_start=P, splits=1, merge=(oa, la))
    _close(fused, sep, rtol=2e-2, atol=1e-2)
    for i, l in enumerate(kv_lens):
        k = torch.cat([dk[0][:P], dk[i][P:l]])
        v = torch.cat([dv[0][:P], dv[i][P:l]])
        ro, _ = ref_attention(q[i:i + 1].cpu(), k, v, causal_offset=l - 1)
        _close(fused[i:i + 1], ro)
    # prefill chunks behind the prefix
    q_lens = [44, 1, 130, 30, 64, 70, 9, 3]
    qs = [0]
    for n in q_lens:
        qs.append(qs[-1] + n)
    T = qs[-1]
    qp = _rand(T, Hq, D, seed=43)
    q_start = torch.tensor(qs, dtype=torch.int32, device="cuda")
    oa2, la2 = cuda_ops.attn_prefill(qp, kc, vc, bt[:1], plen, torch.tensor([0, T], dtype=torch.int32, device="cuda"), T,
                                     causal=False, return_lse=True)
    ob2, lb2 = cuda_ops.attn_prefill(qp, kc, vc, bt, sl, q_start, max(q_lens), causal=True, kv_start=P, return_lse=True)
    assert cuda_ops.attn_prefill_last_path() == "tcgen05"
    sep2 = cuda_ops.attn_merge(oa2, la2, ob2, lb2)
    fused2 = cuda_ops.attn_prefill(qp, kc, vc, bt, sl, q_start, max(q_lens), causal=True, kv_start=P, merge=(oa2, la2))
    _close(fused2, sep2, rtol=2e-2, atol=1e-2)
    for i, (l, n) in enumerate(zip(kv_lens, q_lens)):
        k = torch.cat([dk[0][:P], dk[i][P:l]])
        v = torch.cat([dv[0][:P], dv[i][P:l]])
        ro, _ = ref_attention(qp[qs[i]:qs[i + 1]].cpu(), k, v, causal_offset=l - n)
        _close(fused2[qs[i]:qs[i + 1]], ro)


@pytest.mark.parametrize("M,N,K,tile,ps", [(512, 1024, 4096, 256, 2), (510, 4096, 4096, 256, 2), (300, 768, 8192, 128, 4),
                                           (512, 512, 2048, 256, 4)])
def test_gemm_2cta_splitk(M, N, K, tile, ps):
    """K split over 2 / 4 CTA pairs of one cluster, partial tiles reduced through distributed shared memory."""
    from unillm_b200.ops import cuda_ops

    x, w = _rand(M, K, seed=51), _rand(N, K, scale=1 / math.sqrt(K), seed=52)
    bias, res = _rand(N, seed=53), _rand(M, N, seed=54)
    out = cuda_ops.gemm_tn(x, w, bias=bias, residual=res, tile_tokens=tile, cta_pair=2, pair_splits=ps)
    _close(out, x.float() @ w.float().t() + bias.float() + res.float())
    assert torch.equal(cuda_ops.gemm_tn(x, w, bias=bias, residual=res, tile_tokens=tile, cta_pair=2, pair_splits=ps), out)


def _pair_schedule_case(M, N, K, dual, seed=61):
    from unillm_b200.ops import cuda_ops

    x = _rand(M, K, seed=seed)
    if dual:
        w = _rand(2 * N, K, scale=1 / math.sqrt(K), seed=seed + 1)
        out = cuda_ops.gemm_tn(x, w, dual_rows=N, act="silu")
        g, u = x.float() @ w[:N].float().t(), x.float() @ w[N:].float().t()
        _close(out, torch.nn.functional.silu(g) * u)
        assert torch.equal(cuda_ops.gemm_tn(x, w, dual_rows=N, act="silu"), out)
    else:
        w = _rand(N, K, scale=1 / math.sqrt(K), seed=seed + 1)
        bias, res = _rand(N, seed=seed + 2), _rand(M, N, seed=seed + 3)
        out = cuda_ops.gemm_tn(x, w, bias=bias, residual=res)
        _close(out, x.float() @ w.float().t() + bias.float() + res.float())
        assert torch.equal(cuda_ops.gemm_tn(x, w, bias=bias, residual=res), out)
        out32 = cuda_ops.gemm_tn(x, w, out_dtype=torch.float32)
        _close(out32, x.float() @ w.float().t(), rtol=5e-3, atol=5e-3)
    cuda_ops.check_device_errors()


@pytest.mark.parametrize("M,N,K,dual", [(1020, 6144, 4096, False), (1020, 6272, 2048, False), (1020, 4096, 14336, False),
                                        (640, 4096, 4096, False), (1020, 4864, 2048, True), (1000, 4992, 2048, True),
                                        (1020, 14336, 4096, True), (508, 14336, 4096, True)])
def test_gemm_pair_stream_k(M, N, K, dual):
    """The planner's own choice for shapes whose CTA-pair tiles do not fill whole rounds of the SM pairs.  Plain GEMMs that
    lose a round that way (the first two shapes) run the stream-K schedule: teams of pairs take equal shares of the
    (weight row, k-block) units and partial tiles are summed through the fp32 workspace; gated GEMMs run full rounds plus
    1-CTA tiles with K split for the thin last round.  Ragged token and feature edges, bias / residual / activation
    epilogues, bf16 and fp32 outputs, repeated launches (the flags are lowered by the owner); against fp32."""
    _pair_schedule_case(M, N, K, dual)


def test_gemm_pair_stream_k_back_to_back():
    """Different stream-K shapes in one stream share the workspace lane: results must not depend on what ran before."""
    from unillm_b200.ops import cuda_ops

    shapes = [(1020, 6144, 4096), (640, 4096, 4096), (1020, 6272, 2048)]
    xs = [_rand(M, K, seed=70 + i) for i, (M, N, K) in enumerate(shapes)]
    ws = [_rand(N, K, scale=1 / math.sqrt(K), seed=80 + i) for i, (M, N, K) in enumerate(shapes)]
    first = [cuda_ops.gemm_tn(x, w) for x, w in zip(xs, ws)]
    for _ in range(3):
        for i in (2, 0, 1, 1, 0, 2):
            assert torch.equal(cuda_ops.gemm_tn(xs[i], ws[i]), first[i])
    for (x, w, o) in zip(xs, ws, first):
        _close(o, x.float() @ w.float().t())
    cuda_ops.check_device_errors()


def test_gemm_pair_two_phase_without_stream_k():
    """With the stream-K schedule switched off (the variable is read once per process, hence the child process) the gated
    GEMM falls back to full rounds on pairs plus 1-CTA tiles with K split for the thin last round."""
    import os
    import subprocess
    import sys

    code = (
        "import math, torch\n"
        "from unillm_b200.ops import cuda_ops\n"
        "g = torch.Generator().manual_seed(5)\n"
        "M, N, K = 1020, 4864, 2048\n"
        "x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()\n"
        "w = (torch.randn(2 * N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).cuda()\n"
        "sms = torch.cuda.get_device_properties(0).multi_processor_count\n"
        "assert sms < 132 or cuda_ops.gemm_num_ctas(M, N, K, True) > sms\n"
        "out = cuda_ops.gemm_tn(x, w, dual_rows=N, act='silu').float()\n"
        "ref = torch.nn.functional.silu(x.float() @ w[:N].float().t()) * (x.float() @ w[N:].float().t())\n"
        "err = (out - ref).abs().max().item()\n"
        "assert err < 0.05, err\n"
        "cuda_ops.check_device_errors()\n"
        "print('ok')\n")
    env = dict(os.environ, UB_GEMM_STREAMK="0")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("D,Hq,Hkv,Sq,Sk,causal", [(128, 4, 2, 70, 70, True), (128, 4, 4, 33, 50, False), (64, 6, 2, 40, 40, False),
                                                   (64, 4, 4, 1, 37, True), (128, 2, 1, 17, 64, True)])
def test_dense_attention_on_the_paged_kernels(D, Hq, Hkv, Sq, Sk, causal):
    """Dense [B, H, S, D] attention (encoders, cross-attention, the whole-model decoders) on identity-paged K/V."""
    from unillm_b200.ops import cuda_ops as K

    g = torch.Generator().manual_seed(D + Sq)
    B = 3
    q = torch.randn(B, Hq, Sq, D, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(B, Hkv, Sk, D, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(B, Hkv, Sk, D, generator=g).to(torch.bfloat16).cuda()
    got = K.dense_attention(q, k, v, causal=causal).float().cpu()
    rep = Hq // Hkv
    kf, vf = k.float().cpu().repeat_interleave(rep, 1), v.float().cpu().repeat_interleave(rep, 1)
    s = q.float().cpu() @ kf.transpose(-1, -2) * D ** -0.5
    if causal:
        i = torch.arange(Sq)[:, None] + (Sk - Sq)
        s = s.masked_fill(torch.arange(Sk)[None] > i, float("-inf"))
    ref = torch.softmax(s, -1) @ vf
    assert (got - ref).abs().max().item() < 0.03
    torch.cuda.synchronize()
    K.check_device_errors()


def test_softmax_rows_kernel():
    from unillm_b200.ops import cuda_ops as K

    x = (torch.randn(37, 5, 1000) * 3).to(torch.bfloat16).cuda()
    got = K.softmax_rows(x).float().cpu()
    ref = torch.softmax(x.float().cpu(), -1)
    assert (got - ref).abs().max().item() < 4e-3
    assert (got.sum(-1) - 1).abs().max().item() < 2e-2


def test_encoder_attention_takes_the_kernel_path():
    """A bf16 BERT on the GPU (bidirectional attention, head size 64) against its fp32 CPU copy."""
    from unillm_b200.model_core import ModelInputs
    from unillm_b200.models import configs as C
    from unillm_b200.models.encoders import BertModel
    from unillm_b200.ops import cuda_ops as K

    cfg = C.BertConfig(vocab_size=200, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, intermediate_size=512)
    m = BertModel.new(cfg, init="random", seed=2)
    m.p = {k: v.to(torch.bfloat16).float() for k, v in m.p.items()}
    ids = torch.randint(0, 200, (2, 45))
    ref = m.forward(ModelInputs.text(ids)).main_tensor().float()
    mg = BertModel.new(cfg, init="random", seed=2)
    mg.p = {k: v.to(torch.bfloat16).cuda() for k, v in m.p.items()}
    got = mg.forward(ModelInputs.text(ids.cuda())).main_tensor().float().cpu()
    assert K.attn_prefill_last_path() in ("mma.sync", "tcgen05")
    assert (got - ref).abs().max().item() < 0.08 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("Hq,Hkv,D,P,B", [(16, 4, 128, 64, 700), (4, 1, 128, 1024, 130), (8, 8, 64, 0, 90), (24, 2, 128, 48, 40),
                                         (40, 2, 64, 16, 33)])
def test_decode_warp_pipelines(Hq, Hkv, D, P, B):
    """The decode kernel with one copy / MMA pipeline per warp: more items than warps (a warp walks over several, with the
    next one's length and block-table entries requested early), fewer items than warps (deep ring), GQA groups of 1, 4,
    12 and 20 heads (MMA rows 8..15 in use, two row chunks per KV head), ranges longer than 32 pages (block-table
    entries reloaded), ranges that end before they start, first pages that start inside a page, with and without the
    fused merge; oracle = fp32 attention over the visible keys."""
    from unillm_b200.ops import cuda_ops

    g = torch.Generator().manual_seed(B + Hq)
    kv_lens = [int(v) for v in torch.randint(P + 1, P + 230, (B,), generator=g)]
    kv_lens[1] = P + 700                                    # 44 pages: more than one round of block-table entries
    kv_lens[2] = max(P, 1)
    if P >= 7:
        kv_lens[3] = P - 7
    kc, vc, bt, sl, dk, dv = make_paged_cache(B, kv_lens, Hkv, D, seed=51)
    q = _rand(B, Hq, D, seed=52)
    start = P if P != 48 else 43                            # a range that starts in the middle of a page
    out, lse = cuda_ops.attn_decode(q, kc, vc, bt, sl, kv_start=start, splits=1, return_lse=True, kernel="warp")
    oa = _rand(B, Hq, D, seed=53)
    la = torch.randn(B, Hq, generator=torch.Generator().manual_seed(54)).cuda()
    fused = cuda_ops.attn_decode(q, kc, vc, bt, sl, kv_start=start, splits=1, merge=(oa, la), kernel="warp")
    sep = cuda_ops.attn_merge(oa, la, out, lse)
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
    for i in sorted({0, 1, 2, 3, 4, B // 2, B - 2, B - 1}):
        l = kv_lens[i]
        if l <= start:
            assert out[i].abs().max().item() == 0.0 and torch.isinf(lse[i]).all()
            continue
        ro, rl = ref_attention(q[i:i + 1].cpu(), dk[i], dv[i], causal_offset=l - 1, kv_start=start)
        _close(out[i:i + 1], ro)
        _close(lse[i:i + 1], rl, rtol=1e-2, atol=1e-2)
    _close(fused, sep, rtol=2e-2, atol=1e-2)
    # and it agrees with the dispatcher's default kernel on every row
    ref = cuda_ops.attn_decode(q, kc, vc, bt, sl, kv_start=start, splits=1)
    _close(out, ref.float(), rtol=1e-2, atol=5e-3)


def test_vocab_parallel_sampling_in_two_stages_equals_the_single_shard_draw():
    """Top-k / top-p draws over a vocabulary cut into shards: every shard hands in its best candidates after penalty
    and temperature, the merge over all shards' candidates (here: concatenated by hand, as the pair gather delivers them)
    draws the same token as the kernel that sees the whole row -- for top-k rows, top-p rows, rows with both, greedy rows
    in the same batch and a repetition penalty."""
    from unillm_b200.ops import cuda_ops as K

    B, V, W = 12, 4096, 4
    g = torch.Generator().manual_seed(9)
    logits = (torch.randn(B, V, generator=g) * 3).to(torch.bfloat16).cuda()
    temp = torch.tensor([0.7, 1.0, 1.3, 0.0, 0.9, 1.0, 0.5, 2.0, 1.0, 0.0, 1.1, 0.8]).cuda()
    top_p = torch.tensor([1.0, 0.9, 0.5, 1.0, 0.95, 1.0, 0.3, 0.99, 0.8, 1.0, 1.0, 0.6]).cuda()
    top_k = torch.tensor([40, 0, 0, 0, 64, 1, 5, 0, 17, 0, 3, 0], dtype=torch.int32).cuda()
    pen = torch.full((B,), 1.2).cuda()
    prev = torch.randint(0, V, (B, 9), generator=g).to(torch.int32).cuda()
    for step in range(4):
        ref = K.sample(logits, temperature=temp, top_p=top_p, top_k=top_k, rep_penalty=pen, prev_ids=prev, seed=123, step=step)
        kc = 1024
        cvs, cis = [], []
        for r in range(W):
            shard = logits[:, r * (V // W):(r + 1) * (V // W)].contiguous()
            pr = prev - r * (V // W)                  # history in shard coordinates (out-of-range ids are ignored)
            cv, ci = K.sample(shard, temperature=temp, top_p=top_p, top_k=top_k, rep_penalty=pen, prev_ids=pr.contiguous(),
                              seed=123, step=step, vocab_offset=r * (V // W), candidates=kc)
            cvs.append(cv)
            cis.append(ci)
        av = torch.cat(cvs, 1).contiguous()
        ai = torch.cat(cis, 1).contiguous()
        got = K.sample(av, temperature=temp, top_p=top_p, top_k=top_k, seed=123, step=step, id_map=ai)
        assert torch.equal(got.cpu(), ref.cpu()), (step, got.cpu().tolist(), ref.cpu().tolist())
    # the candidate lists are sorted, global ids, padded with -inf / -1
    assert bool((cvs[1][:, :-1] >= cvs[1][:, 1:]).all())
    ok = cis[1] >= 0
    assert bool(((cis[1] >= V // W) & (cis[1] < 2 * (V // W)))[ok].all())


def test_pair_gather_emulated_ranks():
    """The one-shot (value, id) all-gather with all ranks emulated on one GPU.  Kernels of different emulated ranks
    cannot wait for one another on one stream, so every rank's counters are credited up front with the arrivals of the
    ranks that launch after it; the last launch sees all data and its result is checked.  Two exchanges in a row
    cover the parity slots and the counted (never reset) arrival words."""
    from unillm_b200.dist.fused import SG_FLAGS, FusedComm

    W, rows, k = 4, 37, 24
    comms = FusedComm.emulated(W, 256, 64, "cuda")
    g = torch.Generator().manual_seed(1)
    vals = [torch.randn(rows, k, generator=g).cuda() for _ in range(W)]
    ids = [torch.randint(0, 1 << 20, (rows, k), generator=g).to(torch.int32).cuda() for _ in range(W)]
    for rnd in range(1, 3):
        outs = None
        for r in range(W):
            c = comms[r]
            fl = c.buf[c.flags.offset:c.flags.offset + 1024].view(torch.int32)
            fl[SG_FLAGS:SG_FLAGS + 64] += (W - 1 - r)
        for r in range(W):
            outs = comms[r].gather_pairs(vals[r], ids[r])
        torch.cuda.synchronize()
        from unillm_b200.ops import cuda_ops as K
        K.check_device_errors()
        ov, oi = outs
        assert torch.equal(ov, torch.cat(vals, 1)) and torch.equal(oi, torch.cat(ids, 1))
        for r in range(W):
            c = comms[r]
            fl = c.buf[c.flags.offset:c.flags.offset + 1024].view(torch.int32)
            # every rank's counters end at rnd * W plus its pre-credit: remove the credit so both rounds start alike
            fl[SG_FLAGS:SG_FLAGS + 64] -= (W - 1 - r)
            assert int(fl[SG_FLAGS]) == rnd * W
        vals = [v + 1 for v in vals]


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K,dual", [(6144, 4096, False), (1000, 520, False), (1792, 4096, True), (37, 264, True)])
def test_gemv_small_token_counts(M, N, K, dual):
    """Up to 16 tokens take the weight-streaming kernel (one or two token tiles of 8): plain and gated form, bias, activation, residual, scale,
    fp32 output, column counts that do not divide by the CTA's eight columns, K that leaves warps without work."""
    from unillm_b200.ops import cuda_ops as K_

    g = torch.Generator().manual_seed(M * 7 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N * (2 if dual else 1), K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    xf, wf = x.float(), w.float()
    if dual:
        got = K_.gemm_tn(x, w, dual_rows=N, act="silu")
        ref = torch.nn.functional.silu(xf @ wf[:N].t()) * (xf @ wf[N:].t())
        _close(got, ref, rtol=2e-2, atol=2e-2)
        return
    bias = torch.randn(N, generator=g).to(torch.bfloat16).cuda()
    res = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    got = K_.gemm_tn(x, w, bias=bias, residual=res, act="gelu", out_scale=0.5)
    ref = torch.nn.functional.gelu(xf @ wf.t() * 0.5 + bias.float()) + res.float()
    _close(got, ref, rtol=2e-2, atol=2e-2)
    got32 = K_.gemm_tn(x, w, out_dtype=torch.float32)
    _close(got32, xf @ wf.t(), rtol=1e-3, atol=1e-3)
    # and the tensor-core tiles agree on the same inputs (tile width forced, so the dispatcher does not divert)
    tc = K_.gemm_tn(x, w, tile_tokens=16)
    _close(tc, got32, rtol=2e-2, atol=2e-2)


def test_oneshot_all_reduce_emulated_ranks_two_exchanges():
    """The one-shot all-reduce with all ranks emulated on one GPU, four exchanges of different sizes in a row (parity
    slots, counted arrival words, grids of one and two CTAs).  Kernels of different emulated ranks cannot wait for one another on one stream, so every rank's per-CTA
    counters are credited up front with the arrivals of the ranks that launch after it; the last launch sees every
    rank's data and its sum is checked against fp32."""
    from unillm_b200.dist.fused import AR_FLAGS, FusedComm
    from unillm_b200.ops import cuda_ops as K

    W, H = 4, 512
    comms = FusedComm.emulated(W, H, 64, "cuda")
    g = torch.Generator().manual_seed(3)
    for rnd, rows in ((1, 24), (2, 8), (3, 32), (4, 24)):      # 2, 1, 2, 2 CTAs: every CTA index counts its own exchanges
        xs = [torch.randn(rows, H, generator=g).to(torch.bfloat16).cuda() for _ in range(W)]
        want = torch.stack([x.float() for x in xs]).sum(0)
        for r in range(W):
            c = comms[r]
            fl = c.buf[c.flags.offset:c.flags.offset + 1024].view(torch.int32)
            fl[AR_FLAGS:AR_FLAGS + 64] += (W - 1 - r)
        outs = [comms[r].all_reduce(xs[r].clone()) for r in range(W)]
        torch.cuda.synchronize()
        K.check_device_errors()
        assert (outs[-1].float() - want).abs().max().item() < 0.06 * max(1.0, want.abs().max().item())
        for r in range(W):
            c = comms[r]
            fl = c.buf[c.flags.offset:c.flags.offset + 1024].view(torch.int32)
            fl[AR_FLAGS:AR_FLAGS + 64] -= (W - 1 - r)
            assert int(fl[AR_FLAGS]) == rnd * W


def test_whole_vocabulary_draw_over_shards_equals_the_single_kernel_draw():
    """Temperature-only sampling with the vocabulary cut into shards: per-shard (maximum, mass), the shard and in-shard
    target worked out from all of them, the owner's pick merged like a greedy winner -- the token of the kernel that
    sees the whole row, for several Philox steps."""
    from unillm_b200.ops import cuda_ops as K
    from unillm_b200.sampling import philox_uniform

    B, V, W = 16, 4096, 4
    g = torch.Generator().manual_seed(21)
    logits = (torch.randn(B, V, generator=g) * 2.5).to(torch.bfloat16).cuda()
    temp = (torch.rand(B, generator=g) * 1.5 + 0.3).cuda()
    same = 0
    for step in range(6):
        ref = K.sample(logits, temperature=temp, seed=77, step=step).cpu()
        stats = [K.sample(logits[:, r * (V // W):(r + 1) * (V // W)].contiguous(), temperature=temp, seed=77, step=step, stats=True)
                 for r in range(W)]
        maxes = torch.stack([s_[:, 0] for s_ in stats], 1)
        masses = torch.stack([s_[:, 1] for s_ in stats], 1)
        uni = torch.tensor([philox_uniform(77, step, r) for r in range(B)], dtype=torch.float32).cuda()
        owner, local = K.vocab_shard_targets(maxes, masses, uni)
        vals, ids = [], []
        for r in range(W):
            tgt = torch.where(owner == r, local, torch.full_like(local, -1.0)).contiguous()
            i_, v_ = K.sample(logits[:, r * (V // W):(r + 1) * (V // W)].contiguous(), temperature=temp, seed=77, step=step,
                              vocab_offset=r * (V // W), target=tgt, return_vals=True)
            ids.append(i_)
            vals.append(v_)
        got = K.argmax_merge(torch.stack(vals).contiguous(), torch.stack(ids).contiguous()).cpu()
        assert ((torch.stack(ids) >= 0).sum(0) == 1).all()                     # exactly one shard draws every row
        same += int((got == ref).sum())
    # sums over shards and over the whole row round differently: a target that sits within rounding of a token's
    # boundary may land on its neighbour
    assert same >= 6 * B - 2, same
