"""Numerics of every CUDA kernel against the fp32 PyTorch references."""
import math

import pytest
import torch

from omni_npu_b200 import ops
from omni_npu_b200.ops import ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol, rtol):
    torch.testing.assert_close(a.float().cpu(), b.float().cpu(), atol=atol, rtol=rtol)


@pytest.fixture(autouse=True)
def _status():
    yield
    ops.check_status()


# ------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 256, 128), (256, 512, 4096), (77, 200, 136),
                                   (1, 4096, 4096), (128, 6144, 4096), (1000, 1024, 2048),
                                   (8192, 4096, 4096)])
def test_gemm_bf16(m, n, k):
    torch.manual_seed(0)
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * 0.05
    out = ops.gemm(a, w)
    want = ref.gemm(a.cpu(), w.cpu())
    _close(out, want, atol=2e-2 * math.sqrt(k / 64), rtol=2e-2)


@pytest.mark.parametrize("bn,splits", [(32, 1), (64, 2), (112, 4), (128, 3), (208, 1), (256, 1), (256, 8),
                                       (64, -2), (112, -4), (128, 8), (96, 5), (16, 7)])
def test_gemm_tile_widths_and_split_k(bn, splits):
    torch.manual_seed(1)
    m, n, k = 200, 1000, 4096
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * 0.05
    out = ops.gemm(a, w, bn=bn, splits=splits)
    _close(out, ref.gemm(a.cpu(), w.cpu()), atol=0.15, rtol=2e-2)
    # split-K leaves its counters at rest: a second call must agree
    out2 = ops.gemm(a, w, bn=bn, splits=splits)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("m,n,k", [(128, 4096, 4096), (64, 6144, 4096), (1, 4096, 14336), (100, 1000, 4104)])
def test_gemm_small_m_default_plan(m, n, k):
    """Decode-shaped problems take the cluster split-K path by default."""
    torch.manual_seed(5)
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(m, n, device=DEV, dtype=torch.bfloat16)
    out = ops.gemm(a, w, bias, res)
    _close(out, ref.gemm(a.cpu(), w.cpu(), bias.cpu(), res.cpu()), 0.2, 2e-2)
    assert torch.equal(out, ops.gemm(a, w, bias, res))


def test_gemm_epilogues():
    torch.manual_seed(2)
    m, n, k = 300, 768, 1024
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(m, n, device=DEV, dtype=torch.bfloat16)
    _close(ops.gemm(a, w, bias, res), ref.gemm(a.cpu(), w.cpu(), bias.cpu(), res.cpu()), 0.08, 2e-2)
    _close(ops.gemm(a, w, bias, res, splits=2, bn=128), ref.gemm(a.cpu(), w.cpu(), bias.cpu(), res.cpu()), 0.08, 2e-2)
    _close(ops.gemm(a, w, bias, res, splits=-2), ref.gemm(a.cpu(), w.cpu(), bias.cpu(), res.cpu()), 0.08, 2e-2)
    o32 = ops.gemm(a, w, out_dtype=torch.float32)
    assert o32.dtype == torch.float32
    _close(o32, ref.gemm(a.cpu(), w.cpu(), out_dtype=torch.float32), 2e-2, 1e-2)
    # fused SwiGLU with interleaved gate/up rows
    i = n // 2
    wi = ref.interleave_gate_up(w[:i], w[i:])
    fused = ops.gemm(a, wi, swiglu=True)
    want = ref.silu_and_mul(ref.gemm(a.cpu(), w.cpu(), out_dtype=torch.float32))
    _close(fused, want, 0.06, 3e-2)


@pytest.mark.parametrize("m,n,k,bn", [(256, 256, 128, 0), (512, 1024, 4096, 0), (300, 200, 136, 0),
                                      (1000, 1024, 2048, 128), (8192, 4096, 4096, 0), (257, 96, 64, 96),
                                      (2048, 6144, 4096, 192), (130, 4096, 512, 32)])
def test_gemm_cta_pair(m, n, k, bn):
    """256-row tiles computed by two SMs (tcgen05 cta_group::2)."""
    torch.manual_seed(6)
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * 0.05
    out = ops.gemm(a, w, bn=bn, pair=True)
    torch.cuda.synchronize()
    ops.check_status()
    _close(out, ref.gemm(a.cpu(), w.cpu()), atol=2e-2 * math.sqrt(k / 64), rtol=2e-2)
    assert torch.equal(out, ops.gemm(a, w, bn=bn, pair=True))


def test_gemm_cta_pair_epilogues_and_fp8():
    torch.manual_seed(7)
    m, n, k = 700, 768, 1024
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(m, n, device=DEV, dtype=torch.bfloat16)
    _close(ops.gemm(a, w, bias, res, pair=True), ref.gemm(a.cpu(), w.cpu(), bias.cpu(), res.cpu()), 0.08, 2e-2)
    o32 = ops.gemm(a, w, out_dtype=torch.float32, pair=True)
    assert o32.dtype == torch.float32
    _close(o32, ref.gemm(a.cpu(), w.cpu(), out_dtype=torch.float32), 2e-2, 1e-2)
    i = n // 2
    wi = ref.interleave_gate_up(w[:i], w[i:])
    fused = ops.gemm(a, wi, swiglu=True, pair=True)
    _close(fused, ref.silu_and_mul(ref.gemm(a.cpu(), w.cpu(), out_dtype=torch.float32)), 0.06, 3e-2)
    a8 = (torch.randn(512, 1024, device=DEV) * 0.5).to(torch.float8_e4m3fn)
    w8 = (torch.randn(512, 1024, device=DEV) * 0.5).to(torch.float8_e4m3fn)
    _close(ops.gemm(a8, w8, pair=True), ref.gemm(a8.cpu(), w8.cpu()), 0.25, 2e-2)
    torch.cuda.synchronize()
    ops.check_status()


@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (200, 1000, 4096), (1, 4096, 4096), (777, 6144, 1024)])
def test_gemm_int8_scaled(m, n, k):
    """int8 x int8 with s32 accumulation on the tensor cores; per-token x per-channel scales."""
    torch.manual_seed(8)
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV) * 0.05
    xq, xs = ops.quant_int8_per_token(x)
    rq, rs = ref.quant_int8_per_token(x.cpu())
    assert (xq.cpu().int() - rq.int()).abs().max() <= 1 and torch.allclose(xs.cpu(), rs, rtol=1e-3)
    ws = w.abs().amax(dim=1) / 127.0
    wq = torch.round(w / ws[:, None]).clamp(-127, 127).to(torch.int8)
    bias = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    out = ops.gemm_scaled(xq, wq, xs, ws, bias, out_dtype=torch.float32)
    torch.cuda.synchronize()
    ops.check_status()
    want = ref.gemm_scaled(xq.cpu(), wq.cpu(), xs.cpu(), ws.cpu(), bias.cpu(), out_dtype=torch.float32)
    _close(out, want, atol=2e-3 * math.sqrt(k / 64), rtol=1e-3)     # integer accumulation is exact
    # against the unquantised product: quantisation error only
    full = x.float().cpu() @ w.cpu().t() + bias.float().cpu()
    assert (out.cpu() - full).abs().max() < 0.05 * full.abs().max() + 0.05


def test_gemm_fp8_scaled():
    torch.manual_seed(9)
    m, n, k = 300, 512, 1024
    a = (torch.randn(m, k, device=DEV) * 0.5).to(torch.float8_e4m3fn)
    w = (torch.randn(n, k, device=DEV) * 0.5).to(torch.float8_e4m3fn)
    sa = torch.rand(m, device=DEV) + 0.5
    sw = torch.rand(n, device=DEV) + 0.5
    out = ops.gemm_scaled(a, w, sa, sw, out_dtype=torch.float32)
    want = (a.float().cpu() @ w.float().cpu().t()) * sa.cpu()[:, None] * sw.cpu()[None, :]
    _close(out, want, atol=0.05, rtol=1e-2)


def test_grouped_gemm():
    torch.manual_seed(3)
    e, n, k = 8, 512, 1024
    counts = [0, 5, 128, 129, 300, 1, 0, 77]
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32)
    rows = int(offs[-1])
    a = torch.randn(rows, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(e, n, k, device=DEV, dtype=torch.bfloat16) * 0.05
    out = ops.grouped_gemm(a, w, offs.to(DEV))
    _close(out, ref.grouped_gemm(a.cpu(), w.cpu(), offs), 0.08, 2e-2)
    wi = ref.interleave_gate_up(w[:, : n // 2], w[:, n // 2:])
    out = ops.grouped_gemm(a, wi, offs.to(DEV), swiglu=True)
    want = ref.silu_and_mul(ref.grouped_gemm(a.cpu().float(), w.cpu().float(), offs))
    _close(out, want, 0.06, 3e-2)


def test_gemm_fp8_plain():
    torch.manual_seed(4)
    m, n, k = 256, 512, 1024
    a = (torch.randn(m, k, device=DEV) * 0.5).to(torch.float8_e4m3fn)
    w = (torch.randn(n, k, device=DEV) * 0.5).to(torch.float8_e4m3fn)
    out = ops.gemm(a, w)
    _close(out, ref.gemm(a.cpu(), w.cpu()), 0.25, 2e-2)


# --------------------------------------------------------------- row kernels
@pytest.mark.parametrize("t,h", [(1, 4096), (37, 4096), (128, 2048), (5, 7168), (16, 128), (33, 16384)])
def test_rms_norm(t, h):
    torch.manual_seed(0)
    x = torch.randn(t, h, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(h, device=DEV, dtype=torch.bfloat16)
    _close(ops.rms_norm(x, w, 1e-6), ref.rms_norm(x.cpu(), w.cpu(), 1e-6), 2e-2, 2e-2)
    r = torch.randn(t, h, device=DEV, dtype=torch.bfloat16)
    r_ref = r.cpu().clone()
    y = ops.fused_add_rms_norm(x, r, w, 1e-6)
    y_ref = ref.fused_add_rms_norm(x.cpu(), r_ref, w.cpu(), 1e-6)
    _close(r, r_ref, 1e-2, 1e-2)
    _close(y, y_ref, 3e-2, 2e-2)


def test_rms_norm_strided_heads():
    x = torch.randn(9, 3 * 128 * 4, device=DEV, dtype=torch.bfloat16)
    q = x[:, : 128 * 4]
    w = torch.randn(128, device=DEV, dtype=torch.bfloat16)
    got = ops.rms_norm(q.reshape(-1, 128), w, 1e-6)
    _close(got, ref.rms_norm(q.cpu().reshape(-1, 128), w.cpu(), 1e-6), 2e-2, 2e-2)


def test_silu_and_mul_and_quant():
    x = torch.randn(50, 2 * 1408, device=DEV, dtype=torch.bfloat16)
    _close(ops.silu_and_mul(x), ref.silu_and_mul(x.cpu()), 2e-2, 2e-2)
    y = torch.randn(19, 1024, device=DEV, dtype=torch.bfloat16) * 3
    q, s = ops.quant_fp8_1x128(y)
    qr, sr = ref.quant_fp8_1x128(y.cpu())
    _close(s, sr, 1e-6, 1e-5)
    deq = q.float().view(19, 8, 128) * s.unsqueeze(-1)
    _close(deq.view(19, 1024), y, 0.25, 0.07)


@pytest.mark.parametrize("neox", [True, False])
@pytest.mark.parametrize("rot", [128, 64])
def test_rope_qk(neox, rot):
    t, hq, hk, d = 23, 8, 2, 128
    q = torch.randn(t, hq * d, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(t, hk * d, device=DEV, dtype=torch.bfloat16)
    pos = torch.randint(0, 4000, (t,), device=DEV, dtype=torch.int32)
    cs = ref.build_cos_sin_cache(rot, 4096, 10000.0).to(DEV)
    qr, kr = ref.rope_qk(q.cpu(), k.cpu(), pos.cpu(), cs.cpu(), d, rot, neox)
    ops.rope_qk_(q, k, pos, cs, d, rot, neox)
    _close(q, qr, 2e-2, 2e-2)
    _close(k, kr, 2e-2, 2e-2)


@pytest.mark.parametrize("interleaved", [False, True])
def test_mrope(interleaved):
    t, hq, hk, d = 11, 4, 2, 128
    q = torch.randn(t, hq * d, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(t, hk * d, device=DEV, dtype=torch.bfloat16)
    pos = torch.randint(0, 500, (3, t), device=DEV, dtype=torch.int32)
    cs = ref.build_cos_sin_cache(d, 512, 10000.0).to(DEV)
    sec = (24, 20, 20)
    qr, kr = ref.rope_qk(q.cpu(), k.cpu(), pos.cpu(), cs.cpu(), d, d, True, sec, interleaved)
    ops.rope_qk_(q, k, pos, cs, d, d, True, sec, interleaved)
    _close(q, qr, 2e-2, 2e-2)
    _close(k, kr, 2e-2, 2e-2)


def _paged_setup(seq_lens, q_lens, hq, hk, d, bs, dv=None, seed=0):
    torch.manual_seed(seed)
    dv = dv or d
    b = len(seq_lens)
    max_blocks = max((s + bs - 1) // bs for s in seq_lens) + 1
    nblocks = b * max_blocks + 3
    perm = torch.randperm(nblocks)[: b * max_blocks].view(b, max_blocks).to(torch.int32)
    k_cache = torch.randn(nblocks, hk, bs, d, dtype=torch.bfloat16)
    v_cache = torch.randn(nblocks, hk, bs, dv, dtype=torch.bfloat16)
    t = sum(q_lens)
    q = torch.randn(t, hq * d, dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    return q, k_cache, v_cache, perm, cu, sl


@pytest.mark.parametrize("tc", [True, False])
@pytest.mark.parametrize("seq_lens,q_lens,hq,hk,bs,causal", [
    ([130, 64, 517, 9], [130, 33, 200, 9], 8, 2, 16, True),        # with cached context, ragged tiles
    ([1000, 1], [1000, 1], 4, 4, 16, True),                        # many key tiles, a one-row sequence
    ([300, 257], [300, 129], 16, 2, 32, True),                     # 8 query heads per kv head, 32-token blocks
    ([200, 77], [200, 40], 8, 2, 16, False),                       # not causal
    ([640], [64], 8, 1, 64, True),                                 # short chunk over a long context, 64-token blocks
])
def test_gqa_prefill_tcgen05_matches_reference(seq_lens, q_lens, hq, hk, bs, causal, tc):
    """Head size 128: the tcgen05 / TMEM kernel and the mma.sync kernel against the fp32 reference."""
    d = 128
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, q_lens, hq, hk, d, bs, seed=31)
    want, lse_want = ref.paged_attention(q, kc, vc, bt, cu, sl, hq, d ** -0.5, causal, 0, True)
    got, lse = ops.gqa_prefill(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), cu.to(DEV), sl.to(DEV),
                               len(seq_lens), max(q_lens), hq, d ** -0.5, causal, 0, True, tcgen05=tc)
    _close(got, want, 2e-2, 2e-2)
    _close(lse, lse_want, 2e-2, 1e-2)
    # q as a column slice of a wider activation (the fused qkv projection's output)
    wide = torch.randn(q.shape[0], q.shape[1] + 512, dtype=torch.bfloat16)
    wide[:, : q.shape[1]] = q
    got2 = ops.gqa_prefill(wide.to(DEV)[:, : q.shape[1]], kc.to(DEV), vc.to(DEV), bt.to(DEV), cu.to(DEV),
                           sl.to(DEV), len(seq_lens), max(q_lens), hq, d ** -0.5, causal, tcgen05=tc)
    _close(got2, want, 2e-2, 2e-2)


@pytest.mark.parametrize("d,bs", [(128, 16), (64, 16), (128, 128)])
def test_gqa_prefill(d, bs):
    seq_lens, q_lens = [130, 64, 517, 9], [130, 33, 200, 9]
    hq, hk = 8, 2
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, q_lens, hq, hk, d, bs)
    want, lse_want = ref.paged_attention(q, kc, vc, bt, cu, sl, hq, d ** -0.5, True, 0, True)
    got, lse = ops.gqa_prefill(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), cu.to(DEV), sl.to(DEV),
                               len(seq_lens), max(q_lens), hq, d ** -0.5, True, 0, True)
    _close(got, want, 2e-2, 2e-2)
    _close(lse, lse_want, 2e-2, 1e-2)


def test_gqa_prefill_window_and_mla_dims():
    seq_lens, q_lens = [300, 77], [300, 40]
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, q_lens, 4, 4, 128, 16, seed=5)
    want = ref.paged_attention(q, kc, vc, bt, cu, sl, 4, 0.1, True, 64)
    got = ops.gqa_prefill(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), cu.to(DEV), sl.to(DEV), 2, 300,
                          4, 0.1, True, 64)
    _close(got, want, 2e-2, 2e-2)
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, q_lens, 4, 4, 192, 16, dv=128, seed=6)
    want = ref.paged_attention(q, kc, vc, bt, cu, sl, 4, 192 ** -0.5, True, 0)
    got = ops.gqa_prefill(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), cu.to(DEV), sl.to(DEV), 2, 300,
                          4, 192 ** -0.5, True, 0)
    _close(got, want, 2e-2, 2e-2)


@pytest.mark.parametrize("persistent", [2, True, False])
@pytest.mark.parametrize("splits", [1, 2, 5])
@pytest.mark.parametrize("hq,hk,d", [(32, 8, 128), (4, 2, 64), (16, 1, 128), (16, 2, 128)])
def test_gqa_decode(splits, hq, hk, d, persistent):
    seq_lens = [1, 17, 64, 65, 1000, 333]
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, [1] * 6, hq, hk, d, 16, seed=7)
    want = ref.paged_attention(q, kc, vc, bt, cu, sl, hq, d ** -0.5, True, 0)
    got = ops.gqa_decode(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), 6, hq, d ** -0.5,
                         splits=splits, persistent=persistent)
    _close(got, want, 2e-2, 2e-2)


def test_gqa_decode_persistent_more_items_than_ctas_twice():
    """More (sequence, kv head, split) items than resident CTAs: every CTA walks several items
    handed out by the device counter; the counter is back at zero afterwards, so a second call
    (as a graph replay would make it) gives the same result."""
    torch.manual_seed(21)
    seq_lens = [int(x) for x in torch.randint(1, 700, (96,))]
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, [1] * 96, 32, 8, 128, 16, seed=22)
    want = ref.paged_attention(q, kc, vc, bt, cu, sl, 32, 128 ** -0.5, True, 0)
    args = (q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), 96, 32, 128 ** -0.5)
    for splits in (1, 2):
        for _ in range(2):
            got = ops.gqa_decode(*args, splits=splits, persistent=True)
            _close(got, want, 2e-2, 2e-2)
    wc = ops.device_state(torch.device("cuda", 0)).work_counter(torch.cuda.current_stream().cuda_stream)
    assert wc.tolist() == [0, 0]
    assert ops.decode_splits_persistent(128, 8, 1296) == 2 and ops.decode_splits_persistent(128, 4, 1296) == 4
    assert ops.decode_splits_persistent(1, 8, 8192) > 8          # few items: split to fill the SMs


@pytest.mark.parametrize("n_seqs,hq,hk,hi", [(96, 32, 8, 700), (300, 8, 2, 150), (3, 16, 1, 5000), (40, 4, 4, 64)])
def test_gqa_decode_balanced_cut(n_seqs, hq, hk, hi):
    """Persistent CTAs over the balanced cut of the key tiles: ranges that hold several whole items,
    items that spread over many CTAs, more CTAs than tiles; twice, as a graph replay would run it."""
    torch.manual_seed(31)
    seq_lens = [int(x) for x in torch.randint(1, hi, (n_seqs,))]
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, [1] * n_seqs, hq, hk, 128, 16, seed=32)
    want = ref.paged_attention(q, kc, vc, bt, cu, sl, hq, 128 ** -0.5, True, 0)
    args = (q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), n_seqs, hq, 128 ** -0.5)
    for _ in range(2):
        got = ops.gqa_decode(*args, persistent=2)
        _close(got, want, 2e-2, 2e-2)
    ops.check_status()


def test_gqa_decode_balanced_cut_multi_token_window_and_sink():
    seq_lens = [40, 130, 7, 900]
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, [3] * 4, 8, 2, 128, 16, seed=33)
    want = ref.paged_attention(q, kc, vc, bt, cu, sl, 8, 0.09, True, 0)
    got = ops.gqa_decode(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), 4, 8, 0.09, q_len=3,
                         persistent=2)
    _close(got, want, 2e-2, 2e-2)
    seq_lens = [1, 17, 64, 65, 1000, 333]
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, [1] * 6, 8, 2, 128, 16, seed=13)
    want = ref.paged_attention(q, kc, vc, bt, cu, sl, 8, 0.1, True, 64, False, 32)
    got = ops.gqa_decode(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), 6, 8, 0.1, window=64,
                         sink=32, persistent=2)
    _close(got, want, 2e-2, 2e-2)
    # head size 64, sixteen query rows per kv head
    seq_lens = [500, 3, 129]
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, [1] * 3, 16, 1, 64, 16, seed=34)
    want = ref.paged_attention(q, kc, vc, bt, cu, sl, 16, 0.125, True, 0)
    got = ops.gqa_decode(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), 3, 16, 0.125, persistent=2)
    _close(got, want, 2e-2, 2e-2)
    ops.check_status()


@pytest.mark.parametrize("persistent", [2, 1, 0])
def test_gqa_decode_two_tokens_eight_rows(persistent):
    """Two new tokens per sequence with a group of four: eight query rows per kv head, the
    transposed-product path of the decode kernels, each query with its own causal limit."""
    seq_lens = [40, 130, 7, 64, 2, 700]
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, [2] * 6, 8, 2, 128, 16, seed=35)
    want = ref.paged_attention(q, kc, vc, bt, cu, sl, 8, 0.09, True, 0)
    for splits in (1, 3):
        got = ops.gqa_decode(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), 6, 8, 0.09, q_len=2,
                             splits=splits, persistent=persistent)
        _close(got, want, 2e-2, 2e-2)
    ops.check_status()


def test_gqa_decode_multi_token():
    seq_lens = [40, 130, 7]
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, [3] * 3, 8, 2, 128, 16, seed=8)
    want = ref.paged_attention(q, kc, vc, bt, cu, sl, 8, 0.09, True, 0)
    got = ops.gqa_decode(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), 3, 8, 0.09, q_len=3,
                         splits=2)
    _close(got, want, 2e-2, 2e-2)


@pytest.mark.parametrize("window,sink", [(64, 32), (16, 16), (200, 48)])
def test_gqa_window_with_sink_tokens(window, sink):
    """Sliding-window attention where the first `sink` cached tokens stay visible."""
    seq_lens, q_lens = [300, 77, 40], [300, 40, 1]
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, q_lens, 8, 2, 128, 16, seed=12)
    want = ref.paged_attention(q, kc, vc, bt, cu, sl, 8, 0.1, True, window, False, sink)
    got = ops.gqa_prefill(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), cu.to(DEV), sl.to(DEV), 3, 300,
                          8, 0.1, True, window, sink=sink)
    _close(got, want, 2e-2, 2e-2)
    # without the sink the result differs (the mask matters) ...
    nosink = ops.gqa_prefill(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), cu.to(DEV), sl.to(DEV), 3, 300,
                             8, 0.1, True, window)
    assert (nosink.float().cpu() - want.float()).abs().max() > 1e-2
    # ... and decode agrees too
    seq_lens = [1, 17, 64, 65, 1000, 333]
    q, kc, vc, bt, cu, sl = _paged_setup(seq_lens, [1] * 6, 8, 2, 128, 16, seed=13)
    want = ref.paged_attention(q, kc, vc, bt, cu, sl, 8, 0.1, True, window, False, sink)
    for splits in (1, 3):
        got = ops.gqa_decode(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), 6, 8, 0.1,
                             window=window, splits=splits, sink=sink)
        _close(got, want, 2e-2, 2e-2)


def test_lse_merge_and_gather_cache():
    torch.manual_seed(14)
    n, t, h, d = 3, 37, 8, 128
    outs = torch.randn(n, t, h, d, device=DEV, dtype=torch.bfloat16)
    lses = torch.randn(n, t, h, device=DEV) * 3
    lses[1, 5] = float("-inf")                      # a partial that saw no key
    lses[:, 9, 2] = float("-inf")                   # nobody saw a key
    got, lse = ops.merge_attn_states(outs, lses)
    want, lse_want = ref.merge_attn_states(outs.cpu(), lses.cpu())
    _close(got, want, 2e-2, 2e-2)
    assert torch.isinf(lse[9, 2]) and float(got[9, 2].abs().sum()) == 0
    fin = ~torch.isinf(lse_want)
    _close(lse.cpu()[fin], lse_want[fin], 1e-3, 1e-3)
    # merging the two halves of a key set reproduces attention over the whole set
    q = torch.randn(4, 64)
    k, v = torch.randn(50, 64), torch.randn(50, 64)
    def part(ks, vs):
        s_ = q @ ks.t()
        l_ = torch.logsumexp(s_, -1)
        return torch.softmax(s_, -1) @ vs, l_
    (o1, l1), (o2, l2) = part(k[:20], v[:20]), part(k[20:], v[20:])
    whole, _ = part(k, v)
    m_out, _ = ops.merge_attn_states(torch.stack([o1, o2]).unsqueeze(2).to(DEV, torch.bfloat16),
                                     torch.stack([l1, l2]).unsqueeze(2).to(DEV))
    _close(m_out[:, 0], whole, 3e-2, 3e-2)
    cache = torch.randn(12, 16, 576, device=DEV, dtype=torch.bfloat16)
    bt = torch.tensor([[3, 7, 1, 0], [11, 2, 0, 0]], dtype=torch.int32, device=DEV)
    sl = torch.tensor([40, 17], dtype=torch.int32)
    assert torch.equal(ops.gather_cache(cache, bt, sl).cpu(), ref.gather_cache(cache.cpu(), bt.cpu(), sl))


def test_rope_cache_gqa_and_cache_write():
    t, hq, hk, d, bs = 29, 8, 2, 128, 16
    qkv = torch.randn(t, (hq + 2 * hk) * d, device=DEV, dtype=torch.bfloat16)
    q, k, v = qkv[:, : hq * d], qkv[:, hq * d: (hq + hk) * d], qkv[:, (hq + hk) * d:]
    pos = torch.randint(0, 1000, (t,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(10 * bs)[:t].to(torch.int32)
    slots[3] = -1
    cs = ref.build_cos_sin_cache(d, 1024, 500000.0).to(DEV)
    kc = torch.zeros(10, hk, bs, d, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kc_ref, vc_ref = kc.cpu().clone(), vc.cpu().clone()
    qr, kr = ref.rope_qk(q.cpu(), k.cpu(), pos.cpu(), cs.cpu(), d, d, True)
    ref.gqa_cache_write(kr, v.cpu(), kc_ref, vc_ref, slots)
    ops.rope_cache_gqa_(q, k, v, kc, vc, pos, slots.to(DEV), cs, d, d, True)
    _close(q, qr, 2e-2, 2e-2)
    _close(kc, kc_ref, 2e-2, 2e-2)
    _close(vc, vc_ref, 0, 0)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    ops.gqa_cache_write(k, v, kc2, vc2, slots.to(DEV))
    kc3, vc3 = torch.zeros_like(kc_ref), torch.zeros_like(vc_ref)
    ref.gqa_cache_write(k.cpu(), v.cpu(), kc3, vc3, slots)
    _close(kc2, kc3, 0, 0)
    _close(vc2, vc3, 0, 0)


def test_mla_kv_rmsnorm_rope_cache():
    t, l, r, bs = 21, 512, 64, 16
    kv = torch.randn(t, l + r, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(l, device=DEV, dtype=torch.bfloat16)
    pos = torch.randint(0, 900, (t,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(4 * bs)[:t].to(torch.int32)
    cs = ref.build_cos_sin_cache(r, 1024, 10000.0).to(DEV)
    cache = torch.zeros(4, bs, l + r, device=DEV, dtype=torch.bfloat16)
    cache_ref = cache.cpu().clone()
    a = ops.mla_kv_rmsnorm_rope_cache(kv[:, :l], kv[:, l:], w, cache, pos, slots.to(DEV), cs, 1e-6, False, True)
    b = ops.mla_kv_rmsnorm_rope_cache(kv[:, :l].cpu(), kv[:, l:].cpu(), w.cpu(), cache_ref, pos.cpu(), slots,
                                      cs.cpu(), 1e-6, False, True)
    _close(cache, cache_ref, 3e-2, 2e-2)
    _close(a[0], b[0], 3e-2, 2e-2)
    _close(a[1], b[1], 3e-2, 2e-2)


# ------------------------------------------------------------------ sampling
def test_argmax_and_greedy_sample():
    torch.manual_seed(0)
    logits = torch.randn(33, 128256, device=DEV, dtype=torch.float32)
    want = logits.argmax(-1).to(torch.int32)
    assert torch.equal(ops.argmax(logits), want)
    assert torch.equal(ops.argmax(logits.bfloat16()), logits.bfloat16().float().argmax(-1).to(torch.int32))
    t = torch.zeros(33, device=DEV)
    got = ops.sample(logits, t, torch.zeros(33, dtype=torch.int32, device=DEV), torch.ones(33, device=DEV),
                     torch.arange(33, device=DEV), torch.zeros(1, dtype=torch.int64, device=DEV))
    assert torch.equal(got, want)


def test_sample_respects_top_k_top_p_and_distribution():
    torch.manual_seed(1)
    v, n = 1000, 4096
    base = torch.randn(v, device=DEV) * 2
    logits = base.unsqueeze(0).repeat(n, 1).contiguous()
    temp = torch.full((n,), 0.8, device=DEV)
    topk = torch.full((n,), 20, dtype=torch.int32, device=DEV)
    topp = torch.full((n,), 0.9, device=DEV)
    seeds = torch.arange(n, device=DEV, dtype=torch.int64) * 7919 + 13
    step = torch.zeros(1, dtype=torch.int64, device=DEV)
    got = ops.sample(logits, temp, topk, topp, seeds, step).long().cpu()
    masked = ref.apply_top_k_top_p((base / 0.8).unsqueeze(0).cpu(), torch.tensor([20]), torch.tensor([0.9]))[0]
    allowed = torch.isfinite(masked)
    assert allowed[got].all(), "sampled a token outside the top-k/top-p set"
    probs = masked.softmax(-1)
    freq = torch.bincount(got, minlength=v).float() / n
    assert (freq - probs).abs().max() < 0.04
    # a different step offset gives different draws; the same offset repeats them
    again = ops.sample(logits, temp, topk, topp, seeds, step).long().cpu()
    assert torch.equal(again, got)
    other = ops.sample(logits, temp, topk, topp, seeds, step + 1).long().cpu()
    assert (other != got).float().mean() > 0.3


# --------------------------------------------------------------------- MoE
@pytest.mark.parametrize("e,k,sigmoid,groups,bias", [(64, 6, False, (1, 1), False), (128, 8, False, (1, 1), False),
                                                      (256, 8, True, (8, 4), True), (8, 2, True, (4, 2), False)])
def test_moe_topk(e, k, sigmoid, groups, bias):
    torch.manual_seed(0)
    t = 77
    logits = torch.randn(t, e, device=DEV)
    b = (torch.randn(e, device=DEV) * 0.1) if bias else None
    ids, w = ops.moe_topk(logits, b, k, sigmoid, groups[0], groups[1], True, 2.5)
    ids_r, w_r = ref.moe_topk(logits.cpu(), b.cpu() if bias else None, k, sigmoid, groups[0], groups[1], True, 2.5)
    # same selected set (order of equal scores may differ) and same weights per expert
    assert torch.equal(ids.cpu().sort(-1).values, ids_r.sort(-1).values)
    got = torch.zeros(t, e).scatter_(1, ids.cpu().long(), w.cpu())
    want = torch.zeros(t, e).scatter_(1, ids_r.long(), w_r)
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-4)


def test_fused_moe_layer_single_gpu_matches_cpu_reference():
    from omni_npu_b200.layers.moe import FusedMoE
    torch.manual_seed(1)
    kw = dict(num_experts=16, top_k=4, hidden_size=256, intermediate_size=128, num_shared_experts=1,
              renormalize=True, max_tokens=512)
    gpu = FusedMoE(dtype=torch.bfloat16, device=DEV, **kw)
    for p in gpu.parameters():
        p.data.normal_(0, 0.05)
    cpu = FusedMoE(dtype=torch.bfloat16, **kw)
    cpu.load_state_dict({k_: v.cpu() for k_, v in gpu.state_dict().items()})
    for t in (1, 37, 300):
        x = torch.randn(t, 256, device=DEV, dtype=torch.bfloat16)
        _close(gpu(x), cpu(x.cpu()), 3e-2, 3e-2)
    # inactive (padded) rows: ids of -1 must contribute nothing and must not fault
    x = torch.randn(8, 256, device=DEV, dtype=torch.bfloat16)
    w = torch.full((8, 4), 0.25, device=DEV)
    ids = torch.randint(0, 16, (8, 4), device=DEV, dtype=torch.int32)
    ids[5:] = -1
    out = gpu._routed(x, w, ids)
    sh = gpu.shared_experts(x)
    _close(out[5:], sh[5:], 2e-2, 2e-2)


# --------------------------------------------------------------------- MLA
@pytest.mark.parametrize("n_heads,splits,q_len", [(16, 1, 1), (16, 3, 1), (128, 2, 1), (8, 2, 2)])
def test_mla_decode(n_heads, splits, q_len):
    torch.manual_seed(3)
    bs, seq_lens = 16, [5, 64, 200, 1031]
    b = len(seq_lens)
    max_blocks = max((s + bs - 1) // bs for s in seq_lens) + 1
    nblocks = b * max_blocks + 2
    bt = torch.randperm(nblocks)[: b * max_blocks].view(b, max_blocks).to(torch.int32)
    cache = torch.randn(nblocks, bs, 576).bfloat16()
    q = (torch.randn(b * q_len, n_heads * 576) * 0.3).bfloat16()
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    want, want_lse = ref.mla_decode(q, cache, bt, sl, b, q_len, n_heads, 0.07, None, True)
    got, lse = ops.mla_decode(q.to(DEV), cache.to(DEV), bt.to(DEV), sl.to(DEV), b, n_heads, 0.07, q_len,
                              splits=splits, return_lse=True)
    _close(got, want, 2e-2, 2e-2)
    _close(lse, want_lse, 2e-2, 2e-2)


def test_mla_decode_sparse_selection():
    torch.manual_seed(4)
    bs, n_heads, topk = 16, 16, 128
    seq_lens = [300, 90]
    b = len(seq_lens)
    max_blocks = 20
    bt = torch.randperm(b * max_blocks)[: b * max_blocks].view(b, max_blocks).to(torch.int32)
    cache = torch.randn(b * max_blocks, bs, 576).bfloat16()
    q = (torch.randn(b, n_heads * 576) * 0.3).bfloat16()
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    sel = torch.full((b, topk), -1, dtype=torch.int32)
    sel[0] = torch.randperm(300)[:topk].to(torch.int32)
    sel[1, :90] = torch.randperm(90).to(torch.int32)
    sel[1, 7] = -1
    want = ref.mla_decode(q, cache, bt, sl, b, 1, n_heads, 0.07, sel)
    got = ops.mla_decode(q.to(DEV), cache.to(DEV), bt.to(DEV), sl.to(DEV), b, n_heads, 0.07, 1, sel.to(DEV), splits=2)
    _close(got, want, 2e-2, 2e-2)


@pytest.mark.parametrize("kind", ["int8", "fp8"])
@pytest.mark.parametrize("add", [False, True])
def test_rms_norm_quant_fused(kind, add):
    torch.manual_seed(11)
    t, h = 37, 4096
    x = torch.randn(t, h, device=DEV, dtype=torch.bfloat16)
    w = (torch.rand(h, device=DEV) + 0.5).bfloat16()
    res = torch.randn(t, h, device=DEV, dtype=torch.bfloat16) if add else None
    res_ref = res.cpu().clone() if add else None
    q, s, y = ops.rms_norm_quant(x, w, 1e-6, res, kind, want_bf16=True)
    q0, s0, y0 = ref.rms_norm_quant(x.cpu(), w.cpu(), 1e-6, res_ref, kind, True)
    if add:
        _close(res, res_ref, 1e-2, 1e-2)
    _close(y, y0, 2e-2, 2e-2)
    _close(s, s0, 1e-6, 2e-2)
    # the quantised row must reproduce the normalised row to within one quantisation step
    deq = q.float().cpu() * s.cpu().unsqueeze(-1)
    step = s.cpu().unsqueeze(-1) * (1.0 if kind == "int8" else 32.0)
    assert ((deq - y.float().cpu()).abs() <= step + 1e-3).all()


@pytest.mark.parametrize("kind", ["int8", "fp8"])
def test_silu_and_mul_quant_fused(kind):
    torch.manual_seed(12)
    t, i = 19, 14336
    x = torch.randn(t, 2 * i, device=DEV, dtype=torch.bfloat16)
    q, s = ops.silu_and_mul_quant(x, kind)
    q0, s0 = ref.silu_and_mul_quant(x.cpu(), kind)
    _close(s, s0, 1e-6, 2e-2)
    y = ops.silu_and_mul(x).float().cpu()
    deq = q.float().cpu() * s.cpu().unsqueeze(-1)
    step = s.cpu().unsqueeze(-1) * (1.0 if kind == "int8" else 32.0)
    assert ((deq - y).abs() <= step + 1e-3).all()


@pytest.mark.parametrize("mode", ["decode", "decode_mtp", "prefill"])
def test_dsa_indexer_scores_and_topk(mode):
    """Indexer on tcgen05 + radix select against the dense fp32 reference: same scores, and the
    selected set is a valid top-k (every selected score >= every unselected one)."""
    torch.manual_seed(21)
    bs, h, topk = 16, 64, 256
    if mode == "prefill":
        ctx, q_lens = [700, 130, 1500], [700, 100, 333]
    elif mode == "decode":
        ctx, q_lens = [5, 257, 900, 2049], [1, 1, 1, 1]
    else:
        ctx, q_lens = [300, 1025, 64], [2, 2, 2]
    b = len(ctx)
    max_blocks = max((c + bs - 1) // bs for c in ctx) + 2
    nblocks = b * max_blocks + 3
    bt = torch.randperm(nblocks)[: b * max_blocks].view(b, max_blocks).to(torch.int32)
    cache = (torch.randn(nblocks, bs, 128) * 0.5).bfloat16()
    t = sum(q_lens)
    q = (torch.randn(t, h, 128) * 0.5).bfloat16()
    w = torch.randn(t, h) * 0.1
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    pos = torch.cat([torch.arange(c - n, c) for c, n in zip(ctx, q_lens)]).to(torch.int32)
    uniform = mode != "prefill"
    want_sel, want_sc = ref.dsa_indexer_topk(q, w, cache, bt, pos, b, topk, None if uniform else cu, q_lens[0], True)
    sel, sc = ops.dsa_indexer_topk(q.to(DEV), w.to(DEV), cache.to(DEV), bt.to(DEV), pos.to(DEV), b, topk,
                                   None if uniform else cu.to(DEV), q_lens[0], max_ctx=max(ctx),
                                   max_q=max(q_lens), return_scores=True)
    sel, sc = sel.cpu(), sc.cpu()
    for i in range(t):
        n = int(pos[i]) + 1
        assert torch.allclose(sc[i, :n], want_sc[i, :n], rtol=2e-2, atol=2e-2), (mode, i)
        got = sel[i][sel[i] >= 0].long()
        assert got.numel() == min(topk, n) and got.unique().numel() == got.numel() and int(got.max()) < n
        if n > topk:
            chosen = torch.zeros(n, dtype=torch.bool)
            chosen[got] = True
            assert sc[i, :n][chosen].min() >= sc[i, :n][~chosen].max()


@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (300, 1000, 1024), (8, 4096, 7168), (2048, 2500, 512)])
def test_gemm_fp8_block_scaled(m, n, k):
    """128 x 128 block-scaled weights, per-token-per-128 activations (DeepSeek-V3 checkpoint format)."""
    from omni_npu_b200.layers.quant_fp8 import fp8_block_gemm, quantize_weight_block
    torch.manual_seed(31)
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.float32) * 0.05
    # per-block magnitudes differ by orders of magnitude, so a missing or misplaced scale shows
    w = w * torch.logspace(-2, 2, (k // 128)).to(DEV).repeat_interleave(128)[None, :]
    wq, ws = quantize_weight_block(w)
    xq, xs = ops.quant_fp8_1x128(x)
    bias = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(m, n, device=DEV, dtype=torch.bfloat16)
    want = ref.gemm_fp8_block(xq.cpu(), xs.cpu(), wq.cpu(), ws.cpu(), bias.cpu(), res.cpu(), torch.float32)
    got = ops.gemm_fp8_block(xq, xs, wq, ws, bias, res, torch.float32)
    _close(got, want, 2e-3 * float(want.abs().max()), 2e-3)
    got16 = fp8_block_gemm(x, wq, ws, bias, res)
    assert got16.dtype == torch.bfloat16
    _close(got16, want, 2e-2 * float(want.abs().max()), 2e-2)


@pytest.mark.parametrize("large", [False, True])
@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_gemm_fp8_block_scaled(swiglu, large):
    """Expert GEMM on block-scaled e4m3 weights; with SwiGLU the gate / up rows are interleaved in groups
    of 8 while their scale blocks stay in checkpoint order (gate blocks, then up blocks)."""
    from omni_npu_b200.layers.quant_fp8 import quantize_weight_block
    torch.manual_seed(41)
    e, k, inter = 4, 512, 256
    n = 2 * inter if swiglu else 384
    counts = [130, 0, 7, 300]
    if large:                       # enough 128 x 256 tiles for the two-warp-group variant
        inter = 512
        n = 2 * inter if swiglu else 1000
        counts = [1300, 0, 700, 3000]
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32)
    rows = int(offs[-1])
    x = torch.randn(rows + 50, k, device=DEV, dtype=torch.bfloat16)          # rows past the last expert are unused
    xq, xs = ops.quant_fp8_1x128(x)
    wq = torch.empty(e, n, k, dtype=torch.float8_e4m3fn, device=DEV)
    up0 = (inter + 127) // 128
    ws = torch.empty(e, (2 * up0) if swiglu else (n + 127) // 128, k // 128, device=DEV)
    for i in range(e):
        w = torch.randn(n, k, device=DEV) * 0.05 * torch.logspace(-1, 1, k // 128, device=DEV).repeat_interleave(128)
        if swiglu:
            qg, sg = quantize_weight_block(w[:inter])
            qu, su = quantize_weight_block(w[inter:])
            j = torch.arange(inter, device=DEV)
            wq[i, (j // 8) * 16 + j % 8] = qg
            wq[i, (j // 8) * 16 + 8 + j % 8] = qu
            ws[i, :up0], ws[i, up0:] = sg, su
        else:
            wq[i], ws[i] = quantize_weight_block(w)
    want = ref.grouped_gemm_fp8_block(xq.cpu(), xs.cpu(), wq.cpu(), ws.cpu(), offs, swiglu, up0 if swiglu else 0)
    got = ops.grouped_gemm_fp8_block(xq, xs, wq, ws, offs.to(DEV), swiglu, up0 if swiglu else 0)
    scale = float(want[:rows].float().abs().max())
    _close(got[:rows], want[:rows], 2e-2 * scale, 2e-2)


def test_fused_moe_layer_with_block_scaled_fp8_experts():
    """MoE layer whose experts stay in block-scaled e4m3 on the GPU (grouped block-scaled kernel with the
    SwiGLU epilogue) against the same layer with the weights expanded to fp32 on the CPU."""
    from omni_npu_b200.layers.moe import FusedMoE
    from omni_npu_b200.layers.quant_fp8 import quantize_weight_block
    torch.manual_seed(2)
    e, k, h, inter = 8, 2, 256, 256
    kw = dict(num_experts=e, top_k=k, hidden_size=h, intermediate_size=inter, renormalize=True, max_tokens=512,
              quant="fp8")
    gpu = FusedMoE(dtype=torch.bfloat16, device=DEV, **kw)
    cpu = FusedMoE(dtype=torch.float32, **kw)
    gate_w = torch.randn(e, h) * 0.3
    gpu.gate.weight.data.copy_(gate_w.to(DEV))
    cpu.gate.weight.data.copy_(gate_w)
    for i in range(e):
        for shard, shape, pname, sname in (("gate", (inter, h), "w13", "w13_scale"), ("up", (inter, h), "w13", "w13_scale"),
                                           ("down", (h, inter), "w2", "w2_scale")):
            wq, ws = quantize_weight_block(torch.randn(*shape) * 0.05 * torch.logspace(-0.5, 0.5, shape[0]).unsqueeze(1))
            for layer in (gpu, cpu):
                layer.weight_loader(getattr(layer, pname), wq, i, shard)
                layer.weight_loader(getattr(layer, sname), ws, i, shard)
    gpu.process_weights_after_loading()
    cpu.process_weights_after_loading()
    assert gpu.w13.dtype == torch.float8_e4m3fn and cpu.w13.dtype == torch.float32
    for t in (3, 200):
        x = torch.randn(t, h, device=DEV, dtype=torch.bfloat16)
        want = cpu(x.cpu().float())
        _close(gpu(x), want, 5e-2 * float(want.abs().max()), 5e-2)


def test_bounded_wait_gives_up_and_leaves_the_context_usable():
    """A flag that nothing sets: the wait runs out after its poll limit, the kernel reports status 5
    and returns; the next kernels run normally.  A flag that is already set returns at once."""
    from omni_npu_b200.parallel.symm_mem import wait_probe
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    polls = wait_probe(flag, want=1, max_polls=20000)
    assert polls == 20001
    with pytest.raises(RuntimeError, match="status 5"):
        ops.check_status()
    ops.check_status()                                   # the status word was cleared by the report
    flag.fill_(3)
    assert wait_probe(flag, want=2, max_polls=20000) == 0
    ops.check_status()
    a = torch.randn(64, 128, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(32, 128, device=DEV, dtype=torch.bfloat16)
    _close(ops.gemm(a, w), a.float().cpu() @ w.float().cpu().t(), 2e-1, 2e-2)


def test_ep_dispatch_quantising_scatter_matches_quantise_after_arrival():
    """Expert-parallel dispatch that quantises the rows to e4m3 (one scale per 128 columns) inside the
    scatter kernel: bit-identical to scattering bf16 rows and quantising them afterwards."""
    from omni_npu_b200.layers.moe import _solo_group
    from omni_npu_b200.layers.moe_dispatch import EpBuffers, ep_dispatch
    torch.manual_seed(41)
    t, h, e, k = 77, 1024, 16, 4
    x = torch.randn(t, h, device=DEV, dtype=torch.bfloat16)
    logits = torch.randn(t, e, device=DEV)
    w, ids = torch.topk(torch.softmax(logits, -1), k)
    ids = ids.to(torch.int32)
    ids[5, 1] = -1                                   # an inactive slot
    dev = torch.device("cuda", 0)
    plain = EpBuffers(_solo_group(), dev, e, h, 128, k)
    quant = EpBuffers(_solo_group(), dev, e, h, 128, k, fp8_dispatch=True)
    rows, offs, _ = ep_dispatch(None, x, ids, w.float(), e, plain)
    (rq, rs), offs_q, _ = ep_dispatch(None, x, ids, w.float(), e, quant, fp8=True)
    torch.cuda.synchronize()
    n = int(offs[-1])
    assert n == t * k - 1 and torch.equal(offs, offs_q)
    # rows of one expert arrive in an order fixed by atomics: compare expert by expert as multisets
    want_q, want_s = ops.quant_fp8_1x128(rows[:n].contiguous())
    for ei in range(e):
        lo, hi = int(offs[ei]), int(offs[ei + 1])
        a = torch.cat([want_q[lo:hi].view(torch.uint8).float(), want_s[lo:hi]], dim=1)
        b = torch.cat([rq[lo:hi].view(torch.uint8).float(), rs[lo:hi]], dim=1)
        assert torch.equal(torch.sort(a, dim=0).values, torch.sort(b, dim=0).values)
    plain.close(), quant.close()
    ops.check_status()


@pytest.mark.parametrize("sink_len,window", [(4, 8), (0, 6), (3, 0)])
def test_sink_window_latent_attention_cuda_matches_the_cpu_path(sink_len, window):
    """Learned sink rows + sliding window on the latent cache, as composed on the GPU (sparse mode of
    the latent-cache kernel with its log-sum-exp, the sink GEMM, the LSE merge kernel), against the
    fp32 CPU path of the same module with the same weights."""
    from omni_npu_b200.attention.metadata import AttentionMetadata, set_forward_context
    from omni_npu_b200.attention.mla import MLABackend, StaticSinkMLAAttention
    from omni_npu_b200.config import ModelConfig
    from omni_npu_b200.models.utils import random_init_
    kw = dict(architecture="DeepseekV3ForCausalLM", model_type="deepseek_v3", hidden_size=512, num_layers=1,
              num_heads=16, num_kv_heads=16, head_dim=192, intermediate_size=1024, vocab_size=512,
              rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512, rope_neox=False,
              use_mla=True, q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
              v_head_dim=128)
    dev = torch.device("cuda", 0)
    gpu = StaticSinkMLAAttention(ModelConfig(dtype=torch.bfloat16, **kw), 0, dev, "model.layers.0.self_attn",
                                 sink_len=sink_len, sliding_window=window)
    random_init_(gpu, seed=3, std=0.05)
    if sink_len:
        gpu.param_sink_kv.data.normal_(0, 0.5)
    cpu = StaticSinkMLAAttention(ModelConfig(dtype=torch.float32, **kw), 0, torch.device("cpu"),
                                 "model.layers.0.self_attn", sink_len=sink_len, sliding_window=window)
    cpu.load_state_dict({k: v.float().cpu() for k, v in gpu.state_dict().items()})
    gpu.process_weights_after_loading(), cpu.process_weights_after_loading()
    bs, nblk, lens = 16, 8, [21, 13]
    T = sum(lens)
    torch.manual_seed(1)
    hidden = (torch.randn(T, 512) * 0.5).to(torch.bfloat16)
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32)
    bt = torch.tensor([[1, 2, 0, 0], [3, 4, 0, 0]], dtype=torch.int32)
    slots = torch.cat([bt[b, torch.arange(n) // bs] * bs + torch.arange(n) % bs for b, n in enumerate(lens)]).to(torch.int32)
    cu = torch.tensor([0, lens[0], T], dtype=torch.int32)
    outs = {}
    for name, mod, d, dt in (("gpu", gpu, dev, torch.bfloat16), ("cpu", cpu, torch.device("cpu"), torch.float32)):
        cache = MLABackend.allocate_kv_cache(nblk, bs, 512, 64, dt, d)
        md = AttentionMetadata(is_prefill=True, num_seqs=2, num_tokens=T, max_q_len=max(lens), max_seq_len=max(lens),
                               q_len=0, positions=pos.to(d), slot_mapping=slots.to(d), block_tables=bt.to(d),
                               seq_lens=torch.tensor(lens, dtype=torch.int32, device=d), cu_q=cu.to(d),
                               num_actual_tokens=T, num_actual_seqs=2)
        with set_forward_context(md, [cache]):
            outs[name] = mod(hidden.to(d, dt)).float().cpu()
    got, want = outs["gpu"], outs["cpu"]
    rel = (got - want).abs().max() / want.abs().max().clamp_min(1e-6)
    assert rel <= 5e-2, float(rel)
    ops.check_status()
