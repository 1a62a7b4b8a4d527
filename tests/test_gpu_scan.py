"""Recurrence kernels (conv, selective scan, linear recurrence, WKV-4, WKV-6) against the PyTorch fp32 oracle, including
state carry-over across calls; Mamba and RWKV models in bf16 on the GPU against their fp32 CPU selves."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf(t):
    return t.to(torch.bfloat16)


def _close(got, ref, tol):
    err = (got.float().cpu() - ref.float()).abs().max().item()
    assert err < tol * max(1.0, ref.float().abs().max().item()), err


@pytest.mark.parametrize("B,L,Cn,Kw", [(2, 37, 96, 4), (3, 1, 257, 4), (1, 600, 64, 3)])
def test_dwconv1d(B, L, Cn, Kw):
    from unillm_b200.ops import recurrent as R

    g = torch.Generator().manual_seed(L)
    x, w, b = _bf(torch.randn(B, L, Cn, generator=g)), torch.randn(Cn, Kw, generator=g), torch.randn(Cn, generator=g)
    st0 = _bf(torch.randn(B, Kw - 1, Cn, generator=g))
    st_ref, st_dev = st0.clone(), st0.clone().cuda()
    ref = R.causal_dwconv1d(x, w, b, st_ref, act_silu=True)
    got = R.causal_dwconv1d(x.cuda(), w.cuda(), b.cuda(), st_dev, act_silu=True)
    _close(got, ref, 0.02)
    assert torch.equal(st_dev.cpu(), st_ref)
    x2 = _bf(torch.randn(B, 2, Cn, generator=g))
    _close(R.causal_dwconv1d(x2.cuda(), w.cuda(), b.cuda(), st_dev), R.causal_dwconv1d(x2, w, b, st_ref), 0.02)
    assert torch.equal(st_dev.cpu(), st_ref)


@pytest.mark.parametrize("B,L,Dm,Ns", [(2, 50, 96, 16), (1, 1, 130, 16), (2, 33, 64, 8)])
def test_selective_scan(B, L, Dm, Ns):
    from unillm_b200.ops import recurrent as R

    g = torch.Generator().manual_seed(Dm)
    u, dt, z = (_bf(torch.randn(B, L, Dm, generator=g)) for _ in range(3))
    Bm, Cm = (_bf(torch.randn(B, L, Ns, generator=g)) for _ in range(2))
    A, Dv = -torch.rand(Dm, Ns, generator=g) * 2, torch.randn(Dm, generator=g)
    st_ref = torch.randn(B, Dm, Ns, generator=g) * 0.1
    st_dev = st_ref.clone().cuda()
    ref = R.selective_scan(u, dt, A, Bm, Cm, Dv, z, st_ref)
    got = R.selective_scan(u.cuda(), dt.cuda(), A.cuda(), Bm.cuda(), Cm.cuda(), Dv.cuda(), z.cuda(), st_dev)
    _close(got, ref, 0.03)
    _close(st_dev, st_ref, 0.01)


def test_linear_recurrence_and_wkv():
    from unillm_b200.ops import recurrent as R

    g = torch.Generator().manual_seed(5)
    B, L, Cn = 2, 70, 200
    x, a = _bf(torch.randn(B, L, Cn, generator=g)), torch.rand(Cn, generator=g)
    s_ref = torch.zeros(B, Cn)
    s_dev = s_ref.clone().cuda()
    _close(R.linear_recurrence(a.cuda(), x.cuda(), s_dev, True), R.linear_recurrence(a, x, s_ref, True), 0.02)
    _close(s_dev, s_ref, 0.01)
    ap = torch.rand(B, L, Cn, generator=g)
    _close(R.linear_recurrence(ap.cuda(), x.cuda(), None, False), R.linear_recurrence(ap, x, None, False), 0.02)
    k, v = _bf(torch.randn(B, L, Cn, generator=g)), _bf(torch.randn(B, L, Cn, generator=g))
    wd, u = -torch.exp(torch.randn(Cn, generator=g)), torch.randn(Cn, generator=g)
    s4r = R.wkv4_new_state(B, Cn, "cpu")
    s4d = R.wkv4_new_state(B, Cn, "cuda")
    _close(R.wkv4(k.cuda(), v.cuda(), wd.cuda(), u.cuda(), s4d), R.wkv4(k, v, wd, u, s4r), 0.02)
    _close(s4d[:, :2], s4r[:, :2], 0.01)
    for H, Dh in ((3, 64), (4, 32)):
        r6, k6, v6 = (_bf(torch.randn(B, L, H * Dh, generator=g) * 0.5) for _ in range(3))
        w6, u6 = torch.randn(B, L, H * Dh, generator=g) - 1.0, torch.randn(H * Dh, generator=g) * 0.3
        s6r = torch.zeros(B, H, Dh, Dh)
        s6d = s6r.clone().cuda()
        _close(R.wkv6(r6.cuda(), k6.cuda(), v6.cuda(), w6.cuda(), u6.cuda(), H, s6d), R.wkv6(r6, k6, v6, w6, u6, H, s6r), 0.03)
        _close(s6d, s6r, 0.02)


@pytest.mark.parametrize("name", ["mamba", "rwkv4", "rwkv6", "recurrent_gemma"])
def test_state_models_bf16_gpu_vs_fp32_cpu(name):
    from unillm_b200.model_core import ModelInputs
    from unillm_b200.models import ALL_MODELS, configs as C
    from unillm_b200.ops import cuda_ops

    cfgs = {
        "mamba": C.MambaConfig(vocab_size=512, hidden_size=256, num_hidden_layers=2),
        "rwkv4": C.Rwkv4Config(vocab_size=512, hidden_size=256, num_hidden_layers=2),
        "rwkv6": C.Rwkv6Config(vocab_size=512, hidden_size=256, num_hidden_layers=2, head_size=64),
        "recurrent_gemma": C.RecurrentGemmaConfig(vocab_size=512, hidden_size=256, num_hidden_layers=4, intermediate_size=512,
                                                  num_attention_heads=4, num_key_value_heads=1, head_dim=64,
                                                  max_position_embeddings=256),
    }
    cls = ALL_MODELS[name]
    m = cls.new(cfgs[name], init="random", seed=4)
    m.p = {k: v.to(torch.bfloat16).float() for k, v in m.p.items()}
    ids = torch.randint(0, 512, (2, 40), generator=torch.Generator().manual_seed(0))
    ref = m.forward(ModelInputs.text(ids)).main_tensor()
    md = cls.from_weights(cfgs[name], m.export_hf(), dtype=torch.bfloat16, device="cuda")
    cache = md.new_cache()
    got = torch.cat([md.forward_with_cache(ids[:, :33].cuda(), cache)] +
                    [md.forward_with_cache(ids[:, i:i + 1].cuda(), cache) for i in range(33, 40)], 1)
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
    err = (got.float().cpu() - ref).abs().max().item()
    assert err < 0.08 * max(1.0, ref.abs().max().item()), err


def test_conv_transpose1d_as_gemm():
    """Transposed convolution (EnCodec decoder upsampling) on the tcgen05 GEMM + overlap-add vs the fp32 operator."""
    from unillm_b200.models.simple import conv_transpose1d

    g = torch.Generator().manual_seed(1)
    for (B, Ci, L, Co, k, st) in ((2, 32, 40, 16, 8, 4), (1, 64, 33, 32, 16, 8), (2, 16, 25, 8, 4, 2), (1, 8, 10, 8, 3, 1)):
        x, w, b = _bf(torch.randn(B, Ci, L, generator=g)), _bf(torch.randn(Ci, Co, k, generator=g) * 0.2), _bf(torch.randn(Co, generator=g))
        ref = torch.nn.functional.conv_transpose1d(x.float(), w.float(), b.float(), stride=st)
        got = conv_transpose1d(x.cuda(), w.cuda(), b.cuda(), stride=st)
        assert got.shape == ref.shape and got.dtype == torch.bfloat16
        _close(got, ref, 0.03)


def test_conv1d_as_gemm_and_whisper_bf16():
    from unillm_b200.model_core import ModelInputs
    from unillm_b200.models import ALL_MODELS, configs as C
    from unillm_b200.models.simple import conv1d
    from unillm_b200.ops import cuda_ops

    g = torch.Generator().manual_seed(0)
    from unillm_b200.models import simple

    # implicit GEMM (overlapping strided window view): strides 1 / 2 / 3, odd lengths, several batch elements whose
    # straddling windows are dropped, long inputs (tcgen05 tiles) and short ones (weight-streaming kernel)
    for (B, Cc, L, O, k, st, pad) in ((2, 16, 50, 24, 3, 1, 1), (1, 8, 64, 32, 3, 2, 1), (2, 8, 40, 16, 7, 1, 0),
                                       (3, 80, 301, 96, 3, 2, 1), (1, 384, 1500, 384, 3, 1, 1), (2, 24, 9, 8, 5, 3, 2)):
        x, w, b = _bf(torch.randn(B, Cc, L, generator=g)), _bf(torch.randn(O, Cc, k, generator=g) * 0.2), _bf(torch.randn(O, generator=g))
        ref = torch.nn.functional.conv1d(x.float(), w.float(), b.float(), stride=st, padding=pad)
        got = conv1d(x.cuda(), w.cuda(), b.cuda(), stride=st, padding=pad)
        assert got.shape == ref.shape
        _close(got, ref, 0.03 * max(1.0, float(ref.abs().max()) / 8))
    assert simple._IMPLICIT_CONV["ok"], "the overlapping window descriptor was refused; conv1d fell back to the window matrix"
    # grouped: one implicit GEMM per group (the positional convolution of wav2vec2: even kernel, padding k // 2)
    x, w, b = _bf(torch.randn(2, 64, 90, generator=g)), _bf(torch.randn(64, 16, 8, generator=g) * 0.1), _bf(torch.randn(64, generator=g))
    ref = torch.nn.functional.conv1d(x.float(), w.float(), b.float(), padding=4, groups=4)
    got = conv1d(x.cuda(), w.cuda(), b.cuda(), padding=4, groups=4)
    assert got.shape == ref.shape
    _close(got, ref, 0.03)
    # dilation keeps the window-matrix path
    x, w = _bf(torch.randn(1, 16, 70, generator=g)), _bf(torch.randn(8, 16, 3, generator=g) * 0.2)
    _close(conv1d(x.cuda(), w.cuda(), None, dilation=3), torch.nn.functional.conv1d(x.float(), w.float(), dilation=3), 0.03)
    cfg = C.WhisperConfig(vocab_size=512, d_model=128, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4,
                          decoder_attention_heads=4, encoder_ffn_dim=256, decoder_ffn_dim=256, max_source_positions=64,
                          max_target_positions=32, num_mel_bins=16, hidden_size=128, decoder_start_token_id=1, eos_token_id=2)
    cls = ALL_MODELS["whisper"]
    m = cls.new(cfg, init="random", seed=3)
    m.p = {k_: v.to(torch.bfloat16).float() for k_, v in m.p.items()}
    mel = _bf(torch.randn(1, 16, 100, generator=g)).float()
    dec = torch.tensor([[1, 7, 9, 30]])
    ref = m.forward(ModelInputs.audio(mel, decoder_input_ids=dec)).logits
    md = cls.from_weights(cfg, m.export_hf(), dtype=torch.bfloat16, device="cuda")
    got = md.forward(ModelInputs.audio(mel.cuda().to(torch.bfloat16), decoder_input_ids=dec.cuda())).logits
    torch.cuda.synchronize()
    cuda_ops.check_device_errors()
    _close(got, ref, 0.08)


def test_chunked_scans_equal_the_single_pass_on_long_sequences():
    """From 1024 steps on the scans run as parallel 256-step chunks (summary pass, carry over the chunks, output pass).
    Same inputs through the single sequential pass of the same kernels: outputs and final states must agree up to the
    rounding of a different summation order; a ragged last chunk and a non-zero starting state are included."""
    from unillm_b200.ops import recurrent as R

    g = torch.Generator().manual_seed(31)
    L = 1024 + 256 + 77

    def both(fn):
        R.CHUNKED = False
        a = fn()
        R.CHUNKED = True
        b = fn()
        return a, b

    # selective scan
    B, Dm, Ns = 2, 160, 16
    u, dt, z = (_bf(torch.randn(B, L, Dm, generator=g)).cuda() for _ in range(3))
    Bm, Cm = (_bf(torch.randn(B, L, Ns, generator=g)).cuda() for _ in range(2))
    A, Dv = (-torch.rand(Dm, Ns, generator=g) * 2).cuda(), torch.randn(Dm, generator=g).cuda()
    st0 = (torch.randn(B, Dm, Ns, generator=g) * 0.1).cuda()
    states = []

    def run_ss():
        st = st0.clone()
        states.append(st)
        return R.selective_scan(u, dt, A, Bm, Cm, Dv, z, st)

    seq, chk = both(run_ss)
    _close(chk, seq.cpu(), 0.02)
    _close(states[1], states[0].cpu(), 1e-3)

    # diagonal linear recurrence, per-step coefficients
    Cn = 300
    x = _bf(torch.randn(1, L, Cn, generator=g)).cuda()
    a = torch.rand(1, L, Cn, generator=g).cuda() * 0.2 + 0.8
    st0l = torch.randn(1, Cn, generator=g).cuda()
    states.clear()

    def run_lr():
        st = st0l.clone()
        states.append(st)
        return R.linear_recurrence(a, x, st, True)

    seq, chk = both(run_lr)
    _close(chk, seq.cpu(), 0.02)
    _close(states[1], states[0].cpu(), 1e-3)

    # WKV-4
    k, v = (_bf(torch.randn(2, L, Cn, generator=g)).cuda() for _ in range(2))
    w, uu = (-torch.exp(torch.randn(Cn, generator=g) * 0.5 - 2)).cuda(), torch.randn(Cn, generator=g).cuda()
    states.clear()

    def run_w4():
        st = R.wkv4_new_state(2, Cn, "cuda")
        states.append(st)
        return R.wkv4(k, v, w, uu, st)

    seq, chk = both(run_w4)
    _close(chk, seq.cpu(), 0.02)
    true = lambda s: (s[:, 0] * torch.exp(s[:, 2] - s[:, 2].max()), s[:, 1] * torch.exp(s[:, 2] - s[:, 2].max()))  # noqa: E731
    # the (aa, bb, pp) triple is not unique; the ratio aa / bb (the carried average) and pp + log(bb) are
    r0, r1 = states[0][:, 0] / states[0][:, 1], states[1][:, 0] / states[1][:, 1]
    _close(r1, r0.cpu(), 1e-3)
    _close(states[1][:, 2] + torch.log(states[1][:, 1]), (states[0][:, 2] + torch.log(states[0][:, 1])).cpu(), 1e-3)

    # WKV-6
    H, Dh = 3, 64
    r6, k6, v6 = (_bf(torch.randn(1, L, H * Dh, generator=g) * 0.5).cuda() for _ in range(3))
    w6 = (torch.randn(1, L, H * Dh, generator=g) * 0.5 - 1.5).cuda()
    u6 = torch.randn(H * Dh, generator=g).cuda() * 0.3
    st06 = (torch.randn(1, H, Dh, Dh, generator=g) * 0.1).cuda()
    states.clear()

    def run_w6():
        st = st06.clone()
        states.append(st)
        return R.wkv6(r6, k6, v6, w6, u6, H, st)

    seq, chk = both(run_w6)
    _close(chk, seq.cpu(), 0.02)
    _close(states[1], states[0].cpu(), 2e-3)
