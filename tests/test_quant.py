"""Block-quantised formats: C++ oracle and host vector kernels against the NumPy reader; CUDA kernels against both."""
import numpy as np
import pytest
import torch

from unillm_b200.ops import quant as Q
from unillm_b200.weights.gguf import BLOCK, Q4_0, Q8_0, dequantize_blocks, quantize_blocks


def random_blocks(qtype: int, n_elems: int, seed: int = 0) -> np.ndarray:
    """Valid random blocks: random payload bytes, small finite f16 scales."""
    rng = np.random.default_rng(seed)
    epb, bpb = BLOCK[qtype]
    nb = n_elems // epb
    raw = rng.integers(0, 256, size=(nb, bpb), dtype=np.uint8)

    def put_f16(col, lo=0.01, hi=0.2, signed=True):
        v = rng.uniform(lo, hi, size=nb)
        if signed:
            v *= rng.choice([-1.0, 1.0], size=nb)
        raw[:, col:col + 2] = v.astype(np.float16).view(np.uint8).reshape(nb, 2)

    if qtype in (2, 6, 8):
        put_f16(0)
    elif qtype == 3:
        put_f16(0), put_f16(2)
    elif qtype == 12:
        put_f16(0, signed=False), put_f16(2, signed=False)
    elif qtype == 14:
        put_f16(208, 0.001, 0.02)
    return raw.reshape(-1)


@pytest.mark.parametrize("qtype", Q.QTYPES)
def test_host_oracle_matches_numpy_reader(qtype):
    n = 256 * 6
    raw = random_blocks(qtype, n, seed=qtype)
    ref = dequantize_blocks(raw, qtype, (n,))
    got = Q.dequantize_host(raw, qtype, n)
    assert torch.equal(got, ref)


def test_quantise_roundtrip_through_oracle():
    x = torch.randn(4, 64)
    for qt, tol in ((Q8_0, 0.02), (Q4_0, 0.3)):
        raw = quantize_blocks(x, qt)
        back = Q.dequantize_host(raw, qt, x.numel()).reshape(4, 64)
        assert (back - x).abs().max() < tol * x.abs().max()


@pytest.mark.parametrize("qtype", Q.QTYPES)
def test_host_gemv_and_simd_gemm(qtype):
    N_, K, M = 7, 512, 3
    raw = random_blocks(qtype, N_ * K, seed=10 + qtype)
    w = dequantize_blocks(raw, qtype, (N_, K))
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(1))
    ref = x @ w.t()
    assert torch.allclose(Q.qgemv_host(raw, x, N_, qtype), ref, atol=1e-3, rtol=1e-4)
    be = Q.get_simd_backend()
    assert torch.allclose(be.q_gemm(raw, x, N_, qtype), ref, atol=1e-3, rtol=1e-4)
    assert torch.allclose(be.q_gemv(raw, x[0], N_, qtype), ref[0], atol=1e-3, rtol=1e-4)


@pytest.mark.parametrize("qtype", [2, 8, 12])
@pytest.mark.parametrize("level", [0, None])
def test_tiled_parallel_quantised_gemm(qtype, level):
    """Prefill-sized quantised GEMM: 64-row tiles of the weight handed to several threads; the vector row kernels
    (Q4_0 / Q8_0 / Q4_K at level >= 1) and the portable ones must agree with the dequantised matrix product."""
    be = Q.SimdBackend(force_level=level if level is not None else -1)
    N_, K, M = 333, 1024, 19
    raw = random_blocks(qtype, N_ * K, seed=3 + qtype)
    w = dequantize_blocks(raw, qtype, (N_, K))
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(2))
    ref = x @ w.t()
    tol = 2e-3 * float(ref.abs().max())
    for threads in (1, 4, 0):
        be.set_threads(threads)
        got = be.q_gemm(raw, x, N_, qtype)
        assert float((got - ref).abs().max()) < tol, (threads, float((got - ref).abs().max()), tol)
    be.set_threads(0)
    Q.SimdBackend(force_level=-1)


@pytest.mark.parametrize("level", [0, None])
def test_simd_backend_ops(level):
    be = Q.SimdBackend(force_level=level if level is not None else -1)
    assert be.name and be.level >= 0
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(5, 133, generator=g), torch.randn(5, 133, generator=g)
    assert abs(be.dot(a, b) - float((a * b).sum())) < 1e-3
    assert torch.allclose(be.add(a, b), a + b) and torch.allclose(be.mul(a, b), a * b)
    assert torch.allclose(be.silu(a), torch.nn.functional.silu(a), atol=1e-6)
    assert torch.allclose(be.fused_swiglu(a, b), torch.nn.functional.silu(a) * b, atol=1e-6)
    w = torch.randn(133, generator=g)
    ref = a * torch.rsqrt(a.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    assert torch.allclose(be.rms_norm(a, w), ref, atol=1e-5)
    assert torch.allclose(be.rms_norm_inplace(a.clone(), w), ref, atol=1e-5)
    assert torch.allclose(be.softmax(a), torch.softmax(a, -1), atol=1e-6)
    x = torch.randn(6, 2, 16, generator=g)
    pos = torch.arange(6)
    from unillm_b200.models.simple import apply_rope, rope_tables

    cos, sin = rope_tables(8, 16)
    ref = apply_rope(x.permute(1, 0, 2)[None].contiguous(), cos, sin)[0].permute(1, 0, 2)
    assert torch.allclose(be.apply_rope(x.clone(), pos), ref, atol=1e-5)
    Q.SimdBackend(force_level=-1)


@pytest.mark.gpu
@pytest.mark.parametrize("qtype", Q.QTYPES)
def test_cuda_dequant_and_qgemv(qtype):
    from unillm_b200.ops import cuda_ops

    N_, K = 200, 1024
    raw = random_blocks(qtype, N_ * K, seed=20 + qtype)
    w = dequantize_blocks(raw, qtype, (N_, K))
    dev = torch.from_numpy(raw).cuda()
    got = Q.dequantize_cuda(dev, qtype, (N_, K))
    assert torch.equal(got.cpu(), w.to(torch.bfloat16))
    for M in (1, 3, 8):
        x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(torch.bfloat16)
        ref = x.float() @ w.t()
        out = Q.qgemv_cuda(dev, x.cuda(), N_, qtype).float().cpu()
        assert (out - ref).abs().max() < 0.02 * max(1.0, ref.abs().max().item())
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
