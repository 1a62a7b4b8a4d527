"""The allocation-free decode-attention entry point (``ub_attn_decode_static_scratch``).

Some callers of the kernel library may not allocate device memory (a fixed memory budget owned by
another allocator, a serving loop that bans driver allocations after start-up).  For them the split-KV
partials live in an array inside the library image.  The test calls the function through its exported
C symbol, twice in a row (the array is shared and keeps the previous call's contents), and compares
with the regular entry point that takes a caller-provided scratch buffer.  Two more properties are
checked because they are what the entry point is for: the ``scratch`` field of the arguments is not
used (it points at a sentinel buffer that must come back untouched), and the driver reports the same
amount of free device memory before and after the calls.  An oversized request is refused with a clear
message instead of being launched.
This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes as C

import pytest
import torch

from tests.gpu_util import make_paged_cache

pytestmark = pytest.mark.gpu


def _args(q, kc, vc, bt, sl, out, splits):
    from unillm_b200.ops import _native as N
    from unillm_b200.ops import cuda_ops

    B, Hq, D = q.shape
    a = N.UbAttnArgs()
    a.q, a.k_cache, a.v_cache, a.out = q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr()
    a.block_tables, a.seq_lens = bt.data_ptr(), sl.data_ptr()
    a.err = cuda_ops.err_word(q.device).data_ptr()
    a.num_seqs, a.Hq, a.Hkv, a.D = B, Hq, kc.shape[1], D
    a.block_size, a.max_blocks_per_seq, a.num_blocks = kc.shape[2], bt.shape[1], kc.shape[0]
    a.q_stride, a.o_stride = q.stride(0), out.stride(0)
    a.scale = 1.0 / D ** 0.5
    a.splits = splits
    return a


def test_static_scratch_decode_matches_regular_entry_point():
    from unillm_b200.ops import _native as N
    from unillm_b200.ops import cuda_ops

    lib = N.cuda_lib()
    fn = lib.ub_attn_decode_static_scratch
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p]
    lib.ub_attn_decode_static_scratch_error.restype = C.c_char_p
    stream = torch.cuda.current_stream().cuda_stream
    for trial, (lens, Hq, Hkv, D, splits) in enumerate([([700, 33, 1000, 257], 8, 2, 128, 4),
                                                         ([64, 900, 5], 4, 4, 64, 8)]):
        kc, vc, bt, sl, _, _ = make_paged_cache(len(lens), lens, Hkv, D, seed=11 + trial)
        g = torch.Generator().manual_seed(trial)
        q = (torch.randn(len(lens), Hq, D, generator=g)).to(torch.bfloat16).cuda()
        ref = cuda_ops.attn_decode(q, kc, vc, bt, sl, splits=splits)
        outs = [torch.full_like(ref, float("nan")) for _ in range(3)]
        # what a caller might leave in args.scratch: a buffer large enough for the partials, filled with a sentinel
        sentinel = torch.full((len(lens) * Hq * splits * (D + 2),), -12345.0, dtype=torch.float32, device="cuda")

        def call(out):
            a = _args(q, kc, vc, bt, sl, out, splits)
            a.scratch = sentinel.data_ptr()
            rc = fn(C.byref(a), stream)
            assert rc == 0, lib.ub_attn_decode_static_scratch_error()

        # The first call on a device does the documented set-up (it looks up the array's address, which is also when
        # the CUDA runtime loads the part of the library that holds the array); memory is compared around the calls
        # after it.
        call(outs[0])
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        for out in outs[1:]:                               # two calls in a row share the built-in array
            call(out)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, (free_before, free_after)     # the driver handed out no device memory
        cuda_ops.check_device_errors()
        assert torch.all(sentinel == -12345.0)                          # args.scratch was never written
        for out in outs:
            err = (out.float() - ref.float()).abs().max().item()
            assert err <= 2e-2, err


def test_static_scratch_rejects_oversized_request():
    from unillm_b200.ops import _native as N

    lib = N.cuda_lib()
    fn = lib.ub_attn_decode_static_scratch
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p]
    lib.ub_attn_decode_static_scratch_error.restype = C.c_char_p
    a = N.UbAttnArgs()
    a.num_seqs, a.Hq, a.Hkv, a.D, a.splits = 4096, 64, 8, 128, 16      # 545 M floats: far beyond the array
    rc = fn(C.byref(a), torch.cuda.current_stream().cuda_stream)
    assert rc == -20
    msg = lib.ub_attn_decode_static_scratch_error().decode()
    assert "built-in scratch holds" in msg
    torch.cuda.synchronize()
