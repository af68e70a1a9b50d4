"""Layer-level unit tests on CPU: rotary-embedding family, norms, activation, embedding sharding."""
import math

import pytest
import torch

from omni_npu_b200.layers.rope import get_rope, yarn_get_mscale


def _rot_ref(x, pos, inv, mscale, neox=True):
    """Explicit complex rotation of [T, D] with frequencies inv [D/2]."""
    ang = pos.float().unsqueeze(1) * inv.unsqueeze(0)
    cos, sin = ang.cos() * mscale, ang.sin() * mscale
    if neox:
        a, b = x[:, : x.shape[1] // 2], x[:, x.shape[1] // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=1)
    a, b = x[:, 0::2], x[:, 1::2]
    out = torch.empty_like(x)
    out[:, 0::2], out[:, 1::2] = a * cos - b * sin, b * cos + a * sin
    return out


@pytest.mark.parametrize("neox", [True, False])
def test_default_rope_rotates_like_the_closed_form(neox):
    d = 16
    rope = get_rope(d, d, 128, 10000.0, neox)
    q, k = torch.randn(5, 2 * d), torch.randn(5, d)
    pos = torch.tensor([0, 1, 7, 100, 127], dtype=torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))
    want_q = torch.cat([_rot_ref(q[:, :d], pos, inv, 1.0, neox), _rot_ref(q[:, d:], pos, inv, 1.0, neox)], 1)
    want_k = _rot_ref(k, pos, inv, 1.0, neox)
    gq, gk = rope(pos, q.clone(), k.clone())
    assert torch.allclose(gq, want_q, atol=1e-5) and torch.allclose(gk, want_k, atol=1e-5)
    cos, sin = rope.get_cos_sin(pos)
    assert cos.shape == (5, d // 2) and torch.allclose(cos[0], torch.ones(d // 2)) and torch.allclose(sin[0], torch.zeros(d // 2))


def test_partial_rotary_leaves_the_tail_dims_alone():
    rope = get_rope(16, 8, 64, 10000.0, True)
    q, k = torch.randn(3, 16), torch.randn(3, 16)
    gq, _ = rope(torch.tensor([1, 2, 3], dtype=torch.int32), q.clone(), k.clone())
    assert torch.equal(gq[:, 8:], q[:, 8:]) and not torch.allclose(gq[:, :8], q[:, :8])


def test_scaled_variants_frequencies_and_amplitudes():
    d, base = 32, 10000.0
    inv0 = 1.0 / (base ** (torch.arange(0, d, 2).float() / d))

    def table(rope):
        # angle of position 1 = inv_freq (while < pi), amplitude = mscale
        cs = rope.cos_sin_cache[1]
        return torch.atan2(cs[d // 2:], cs[: d // 2]), torch.sqrt(cs[: d // 2] ** 2 + cs[d // 2:] ** 2)

    lin = get_rope(d, d, 64, base, True, {"rope_type": "linear", "factor": 4.0})
    ang, amp = table(lin)
    assert torch.allclose(ang, inv0 / 4.0, atol=1e-6) and torch.allclose(amp, torch.ones_like(amp), atol=1e-6)
    assert lin.cos_sin_cache.shape[0] == 256                                # table extended by the factor

    l3 = get_rope(d, d, 64, base, True, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                         "high_freq_factor": 4.0, "original_max_position_embeddings": 64})
    ang, _ = table(l3)
    assert torch.allclose(ang[0], inv0[0], atol=1e-6)                       # short wavelengths untouched
    assert torch.allclose(ang[-1], inv0[-1] / 8.0, atol=1e-7)               # long wavelengths divided by the factor
    assert ((ang <= inv0 + 1e-7) & (ang >= inv0 / 8.0 - 1e-7)).all()

    yarn = get_rope(d, d, 64, base, True, {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64})
    ang, amp = table(yarn)
    assert torch.allclose(amp, torch.full_like(amp, yarn_get_mscale(4.0)), atol=1e-5)
    assert torch.allclose(ang[0], inv0[0], atol=1e-6) and torch.allclose(ang[-1], inv0[-1] / 4.0, atol=1e-7)
    assert yarn.cos_sin_cache.shape[0] == 256

    ds = get_rope(d, d, 64, base, True, {"rope_type": "deepseek_yarn", "factor": 40.0, "mscale": 1.0,
                                         "mscale_all_dim": 1.0, "original_max_position_embeddings": 64})
    _, amp = table(ds)
    assert torch.allclose(amp, torch.ones_like(amp), atol=1e-5)             # mscale / mscale_all_dim cancel

    ntk = get_rope(d, d, 256, base, True, {"rope_type": "ntk", "factor": 2.0, "original_max_position_embeddings": 64})
    ang, _ = table(ntk)
    new_base = base * ((2.0 * 256 / 64) - 1.0) ** (d / (d - 2))
    assert torch.allclose(ang, 1.0 / (new_base ** (torch.arange(0, d, 2).float() / d)), atol=1e-6)

    lr = get_rope(d, d, 256, base, True, {"rope_type": "longrope", "original_max_position_embeddings": 64,
                                          "long_factor": [2.0] * (d // 2), "short_factor": [1.0] * (d // 2)})
    ang, amp = table(lr)
    assert torch.allclose(ang, inv0 / 2.0, atol=1e-6)
    assert torch.allclose(amp, torch.full_like(amp, math.sqrt(1 + math.log(4.0) / math.log(64))), atol=1e-5)
    with pytest.raises(ValueError):
        get_rope(d, d, 64, base, True, {"rope_type": "nope"})


def test_rope_instances_are_cached_per_configuration():
    a = get_rope(16, 16, 64, 10000.0, True, {"rope_type": "linear", "factor": 2.0})
    assert get_rope(16, 16, 64, 10000.0, True, {"rope_type": "linear", "factor": 2.0}) is a
    assert get_rope(16, 16, 64, 10000.0, True, {"rope_type": "linear", "factor": 3.0}) is not a


def test_mrope_sections_take_their_axis_positions():
    """M-RoPE: frequency index i takes the position of the axis its section names (t, h, w)."""
    d = 16
    rope = get_rope(d, d, 64, 10000.0, True, {"rope_type": "mrope", "mrope_section": [4, 2, 2]})
    pos = torch.tensor([[3, 5], [10, 1], [20, 2]], dtype=torch.int32)       # [3 axes, T]
    q, k = torch.randn(2, d), torch.randn(2, d)
    gq, _ = rope(pos, q.clone(), k.clone())
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))
    axis = torch.tensor([0] * 4 + [1] * 2 + [2] * 2)
    per_freq_pos = pos.float()[axis, :].t()                                 # [T, d/2]
    ang = per_freq_pos * inv
    a, b = q[:, : d // 2], q[:, d // 2:]
    want = torch.cat([a * ang.cos() - b * ang.sin(), b * ang.cos() + a * ang.sin()], 1)
    assert torch.allclose(gq, want, atol=1e-5)


def test_norm_and_activation_layers_match_formulas():
    from omni_npu_b200.layers.activation import SiluAndMul
    from omni_npu_b200.layers.norm import LayerNorm, RMSNorm
    x, r = torch.randn(4, 32), torch.randn(4, 32)
    n = RMSNorm(32, 1e-5, torch.float32)
    n.weight.data = torch.rand(32) + 0.5
    want = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * n.weight
    assert torch.allclose(n(x), want, atol=1e-5)
    r0 = r.clone()
    y, res = n(x, r)
    s = x + r0
    assert torch.allclose(res, s) and torch.allclose(y, s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5) * n.weight, atol=1e-5)
    ln = LayerNorm(32, 1e-6, torch.float32, None)
    assert torch.allclose(ln(x), torch.nn.functional.layer_norm(x, (32,), ln.weight, ln.bias, 1e-6), atol=1e-5)
    g = torch.randn(3, 16)
    assert torch.allclose(SiluAndMul()(g), torch.nn.functional.silu(g[:, :8]) * g[:, 8:], atol=1e-6)


def test_rope_factory_alpha_ntk_xdrope_and_aliases():
    import math
    from omni_npu_b200.layers.rope import get_rope
    d, base, alpha = 64, 10000.0, 8.0
    want = 1.0 / ((base * alpha ** (d / (d - 2))) ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    for kind, extra in (("dynamic", {}), ("xdrope", {"xdrope_section": [8, 8, 8, 8]})):
        rope = get_rope(d, d, 256, base, True, {"rope_type": kind, "alpha": alpha, **extra})
        cos, sin = rope.get_cos_sin(torch.tensor([7]))
        assert torch.allclose(cos[0], torch.cos(7 * want), atol=1e-5)
        assert torch.allclose(sin[0], torch.sin(7 * want), atol=1e-5)
    plain = get_rope(d, d, 256, base, False, {"rope_type": "mllama4"})
    assert torch.equal(plain.cos_sin_cache, get_rope(d, d, 256, base, False, None).cos_sin_cache)
    ds = {"factor": 4.0, "original_max_position_embeddings": 64, "mscale": 1.0, "mscale_all_dim": 1.0}
    a = get_rope(d, d, 256, base, False, {"rope_type": "deepseek_yarn", **ds})
    b = get_rope(d, d, 256, base, False, {"rope_type": "deepseek_llama_scaling", **ds})
    assert torch.equal(a.cos_sin_cache, b.cos_sin_cache)
    with pytest.raises(ValueError):
        get_rope(d, d, 256, base, True, {"rope_type": "dynamic"})


def test_xdrope_takes_each_frequency_band_from_its_own_axis():
    """Four position axes, sections (2, 2, 2, 2) of the 8 frequency indices: band b is rotated by
    positions[b]; 1-D positions are the plain rotation."""
    d, alpha, base = 16, 1000.0, 10000.0
    rope = get_rope(d, d, 256, base, True, {"rope_type": "xdrope", "alpha": alpha, "xdrope_section": [2, 2, 2, 2]})
    inv = 1.0 / ((base * alpha ** (d / (d - 2))) ** (torch.arange(0, d, 2).float() / d))
    t = 6
    pos = torch.stack([torch.arange(t) + 3 * a for a in range(4)]).to(torch.int32)      # [4, T]
    q, k = torch.randn(t, 2 * d), torch.randn(t, d)
    gq, gk = rope(pos, q.clone(), k.clone())
    per_freq_pos = pos.long()[torch.tensor([0, 0, 1, 1, 2, 2, 3, 3])].t().float()       # [T, 8]
    ang = per_freq_pos * inv
    cos, sin = ang.cos(), ang.sin()

    def rot(x):
        a, b = x[:, : d // 2], x[:, d // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], 1)
    assert torch.allclose(gq, torch.cat([rot(q[:, :d]), rot(q[:, d:])], 1), atol=1e-5)
    assert torch.allclose(gk, rot(k), atol=1e-5)
    flat = pos[0].contiguous()
    g1, _ = rope(flat, q.clone(), k.clone())
    g4, _ = rope(flat.expand(4, t).contiguous(), q.clone(), k.clone())
    assert torch.allclose(g1, g4, atol=1e-6)


def test_dual_chunk_rope_produces_the_five_query_views():
    """Keys rotate by their offset inside a chunk; the query comes back five times at the remapped
    positions (intra, successor, inter, successor-critical, inter-critical)."""
    d, base, chunk, local = 16, 10000.0, 32, 8
    rope = get_rope(d, d, 4096, base, True, None, None, {"chunk_size": chunk, "local_size": local})
    clen = chunk - local
    inv = 1.0 / (base ** (torch.arange(0, d, 2).float() / d))
    pos = torch.tensor([0, 5, 23, 24, 47, 1000], dtype=torch.int32)
    q, k = torch.randn(6, d), torch.randn(6, d)
    qs, gk = rope(pos, q.clone(), k.clone())
    assert qs.shape == (6, 5 * d)
    r = pos.long() % clen
    want_pos = [r, torch.clamp(r + clen, max=chunk), torch.full_like(r, min(2 * clen - 1, chunk)), r + clen, r + chunk]
    for i, wp in enumerate(want_pos):
        assert torch.allclose(qs[:, i * d:(i + 1) * d], _rot_ref(q, wp, inv, 1.0), atol=1e-5), i
    assert torch.allclose(gk, _rot_ref(k, r, inv, 1.0), atol=1e-5)
