"""The allocation-free decode-attention entry point, called the way its intended
users call it: through the exported C symbol of the shared library, with raw
device pointers.  (Collected last on purpose: the file name sorts after every
other test module.)

Those users are programs without PyTorch's caching allocator behind them, or
with all device memory already committed to the KV cache, so they cannot supply
scratch memory per call; the library keeps an 8 MiB scratch array of its own.
The result must equal the regular entry point's, on two calls in a row (the
array is reused and keeps the first call's contents).
"""
import ctypes
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = Path(__file__).resolve().parent.parent / "omni_npu_b200" / "_C.so"


def _lib():
    import omni_npu_b200.ops as ops
    ops.load_extension(required=True)          # resolves the torch symbols _C.so depends on
    lib = ctypes.CDLL(str(LIB))
    fn = lib.b200_gqa_decode_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 8 + [ctypes.c_longlong] * 2 + \
        [ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.b200_gqa_decode_static_status.restype = ctypes.c_int
    lib.b200_gqa_decode_static_status.argtypes = [ctypes.c_int]
    lib.b200_gqa_decode_static_strerror.restype = ctypes.c_char_p
    lib.b200_gqa_decode_static_strerror.argtypes = [ctypes.c_int]
    lib.b200_gqa_decode_static_required_bytes.restype = ctypes.c_size_t
    lib.b200_gqa_decode_static_required_bytes.argtypes = [ctypes.c_int] * 4
    return lib


def _problem(seed, seq_lens, hq=32, hk=8, d=128, bs=16):
    g = torch.Generator().manual_seed(seed)
    b = len(seq_lens)
    max_blocks = max((s + bs - 1) // bs for s in seq_lens) + 1
    nblocks = b * max_blocks + 2
    bt = torch.randperm(nblocks, generator=g)[: b * max_blocks].view(b, max_blocks).to(torch.int32).cuda()
    kc = torch.randn(nblocks, hk, bs, d, generator=g).bfloat16().cuda()
    vc = torch.randn(nblocks, hk, bs, d, generator=g).bfloat16().cuda()
    q = torch.randn(b, hq * d, generator=g).bfloat16().cuda()
    sl = torch.tensor(seq_lens, dtype=torch.int32).cuda()
    return q, kc, vc, bt, sl


def _call_static(lib, q, kc, vc, bt, sl, hq, scale, splits):
    out = torch.empty_like(q)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.b200_gqa_decode_static(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(),
                                    bt.data_ptr(), sl.data_ptr(), q.shape[0], 1, bt.shape[1],
                                    kc.shape[2], kc.shape[0], hq, kc.shape[1], kc.shape[3], q.stride(0),
                                    out.stride(0), scale, 0, splits, stream)
    return rc, out


def test_static_scratch_decode_matches_regular_entry_point_twice():
    from omni_npu_b200 import ops
    lib = _lib()
    scale = 128 ** -0.5
    for seed, seq_lens, splits in ((0, [700, 33, 1500, 64, 257, 1], 4), (1, [90, 2048, 511], 3)):
        q, kc, vc, bt, sl = _problem(seed, seq_lens)
        want = ops.gqa_decode(q, kc, vc, bt, sl, len(seq_lens), 32, scale, splits=splits)
        rc, got = _call_static(lib, q, kc, vc, bt, sl, 32, scale, splits)
        assert rc == 0, lib.b200_gqa_decode_static_strerror(rc)
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        assert lib.b200_gqa_decode_static_status(1) == 0
    ops.check_status()


@pytest.mark.parametrize("hq,hk,d,bs,splits", [
    (32, 8, 128, 16, 1),       # one split: no scratch at all
    (16, 4, 64, 16, 3),        # head size 64
    (8, 2, 128, 4, 2),         # 4-token blocks: the variant that reads the cache with plain loads
])
def test_static_scratch_decode_other_shapes(hq, hk, d, bs, splits):
    from omni_npu_b200 import ops
    lib = _lib()
    scale = d ** -0.5
    seq_lens = [130, 5, 77, 300]
    q, kc, vc, bt, sl = _problem(7, seq_lens, hq=hq, hk=hk, d=d, bs=bs)
    want = ops.gqa_decode(q, kc, vc, bt, sl, len(seq_lens), hq, scale, splits=splits)
    for _ in range(2):
        rc, got = _call_static(lib, q, kc, vc, bt, sl, hq, scale, splits)
        assert rc == 0, lib.b200_gqa_decode_static_strerror(rc)
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    assert lib.b200_gqa_decode_static_status(1) == 0
    ops.check_status()


def test_static_scratch_rejects_oversized_problems_without_launching():
    lib = _lib()
    assert lib.b200_gqa_decode_static_required_bytes(128, 8, 128, 8) > (8 << 20)
    rc = lib.b200_gqa_decode_static(None, None, None, None, None, None, 128, 1, 1, 16, 64, 32, 8, 128, 0, 0,
                                    0.1, 0, 8, None)
    assert rc != 0
    assert b"8 MiB" in lib.b200_gqa_decode_static_strerror(rc)
    # a cache size must be given: it bounds what the kernel may read
    rc = lib.b200_gqa_decode_static(None, None, None, None, None, None, 4, 1, 1, 16, 0, 32, 8, 128, 0, 0,
                                    0.1, 0, 2, None)
    assert rc != 0 and b"num_cache_blocks" in lib.b200_gqa_decode_static_strerror(rc)
