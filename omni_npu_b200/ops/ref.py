"""Plain PyTorch reference implementations (fp32 math) of every device op.

They serve two purposes: the CPU execution path (gloo / no-GPU plumbing runs)
and the oracle the CUDA kernels are tested against.  Shapes and semantics are
identical to the CUDA entry points in ``omni_npu_b200.ops``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def gemm(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
         swiglu: bool = False) -> torch.Tensor:
    """``a @ w.T`` with fp32 accumulation.  With ``swiglu`` the N columns are
    interpreted as interleaved groups of 8 gate / 8 up columns."""
    out = a.float() @ w.float().t()
    if swiglu:
        n = out.shape[-1]
        g = out.view(*out.shape[:-1], n // 16, 2, 8)
        out = (F.silu(g[..., 0, :]) * g[..., 1, :]).reshape(*out.shape[:-1], n // 2)
    if bias is not None:
        out = out + bias.float()
    if residual is not None:
        out = out + residual.float()
    if out_dtype is None:
        out_dtype = torch.bfloat16 if a.dtype.itemsize == 1 else a.dtype
    return out.to(out_dtype)


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """Row layout the fused SwiGLU epilogue expects: 8 gate rows, the 8 matching
    up rows, 8 gate rows, ...  ([I,K],[I,K]) -> [2I,K]."""
    i, k = w_gate.shape[-2:]
    lead = w_gate.shape[:-2]
    g = w_gate.reshape(*lead, i // 8, 1, 8, k)
    u = w_up.reshape(*lead, i // 8, 1, 8, k)
    return torch.cat([g, u], dim=-3).reshape(*lead, 2 * i, k)


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, expert_offsets: torch.Tensor,
                 swiglu: bool = False) -> torch.Tensor:
    e = w.shape[0]
    offs = expert_offsets.tolist()
    n_out = w.shape[1] // 2 if swiglu else w.shape[1]
    out = torch.zeros(a.shape[0], n_out, dtype=torch.bfloat16 if a.dtype.itemsize == 1 else a.dtype,
                      device=a.device)
    for i in range(e):
        lo, hi = offs[i], offs[i + 1]
        if hi > lo:
            out[lo:hi] = gemm(a[lo:hi], w[i], swiglu=swiglu, out_dtype=out.dtype)
    return out


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(x.dtype)


def fused_add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor,
                       eps: float) -> torch.Tensor:
    """residual <- x + residual (in place, rounded to its dtype); returns norm(residual)*w."""
    residual.copy_((x.float() + residual.float()).to(residual.dtype))
    return rms_norm(residual, w, eps)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    i = x.shape[-1] // 2
    return (F.silu(x[..., :i].float()) * x[..., i:].float()).to(x.dtype)


def quant_fp8_1x128(x: torch.Tensor, ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    t, h = x.shape
    xf = x.float().view(t, h // 128, 128)
    amax = xf.abs().amax(-1).clamp_min(1e-10)
    scale = amax / 448.0
    if ue8m0:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    q = (xf / scale.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.view(t, h), scale


def dequant_fp8_block(wq: torch.Tensor, scale: torch.Tensor, block: Tuple[int, int] = (128, 128)) -> torch.Tensor:
    """Weights [.., N, K] in e4m3 with one fp32 scale per (128 x 128) block."""
    n, k = wq.shape[-2:]
    bn, bk = block
    s = scale.repeat_interleave(bn, dim=-2)[..., :n, :].repeat_interleave(bk, dim=-1)[..., :k]
    return wq.float() * s


def build_cos_sin_cache(rot_dim: int, max_pos: int, base: float = 10000.0,
                        inv_freq: Optional[torch.Tensor] = None, mscale: float = 1.0,
                        device=None) -> torch.Tensor:
    """[max_pos, rot_dim] fp32: cos in the first half, sin in the second."""
    if inv_freq is None:
        inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    t = torch.arange(max_pos, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq.float().cpu())
    cache = torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1)
    return cache.to(device) if device is not None else cache


def mrope_axis_of_freq(i: torch.Tensor, half: int, sec_t: int, sec_h: int,
                       interleaved: bool) -> torch.Tensor:
    """Which of the (t, h, w) position rows frequency index ``i`` reads."""
    if not interleaved:
        return torch.where(i < sec_t, 0, torch.where(i < sec_t + sec_h, 1, 2))
    sec_w = half - sec_t - sec_h
    m = i % 3
    axis = torch.zeros_like(i)
    axis = torch.where((m == 1) & (i < 3 * sec_h), torch.ones_like(i), axis)
    axis = torch.where((m == 2) & (i < 3 * sec_w), torch.full_like(i, 2), axis)
    return axis


def _rope_one(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot_dim: int,
              neox: bool) -> torch.Tensor:
    """x [T, H, D]; cos/sin [T, rot/2]."""
    xf = x.float()
    rot, rest = xf[..., :rot_dim], xf[..., rot_dim:]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    if neox:
        x0, x1 = rot[..., : rot_dim // 2], rot[..., rot_dim // 2:]
        y = torch.cat([x0 * c - x1 * s, x1 * c + x0 * s], dim=-1)
    else:
        x0, x1 = rot[..., 0::2], rot[..., 1::2]
        y = torch.stack([x0 * c - x1 * s, x1 * c + x0 * s], dim=-1).flatten(-2)
    return torch.cat([y, rest], dim=-1).to(x.dtype)


def rope_qk(q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
            head_dim: int, rot_dim: int, neox: bool = True,
            mrope_section: Optional[Tuple[int, int, int]] = None,
            mrope_interleaved: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [T, Hq*D], k [T, Hk*D]; returns rotated copies."""
    half = rot_dim // 2
    if mrope_section is None:
        cs = cos_sin[positions.long()]
        cos, sin = cs[:, :half], cs[:, half:]
    else:
        idx = torch.arange(half, device=q.device)
        axis = mrope_axis_of_freq(idx, half, mrope_section[0], mrope_section[1], mrope_interleaved)
        pos = positions.long()[axis, :]            # [half, T] -> pick per frequency
        pos = pos.t()                              # [T, half]
        cos = cos_sin[:, :half][pos, idx]
        sin = cos_sin[:, half:][pos, idx]
    t = q.shape[0]
    qo = _rope_one(q.view(t, -1, head_dim), cos, sin, rot_dim, neox).reshape(q.shape)
    ko = _rope_one(k.view(t, -1, head_dim), cos, sin, rot_dim, neox).reshape(k.shape)
    return qo, ko


def gqa_cache_write(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    slot_mapping: torch.Tensor) -> None:
    """k [T, Hk*D] -> k_cache [blocks, Hk, bs, D] at slot (block*bs + off); negative slots skipped."""
    nb, hk, bs, d = k_cache.shape
    dv = v_cache.shape[-1]
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    blk, off = slots // bs, slots % bs
    k_cache[blk, :, off, :] = k[valid].view(-1, hk, d).to(k_cache.dtype)
    v_cache[blk, :, off, :] = v[valid].view(-1, hk, dv).to(v_cache.dtype)


def paged_scatter_rows(dst: torch.Tensor, src: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    valid = slot_mapping >= 0
    dst.view(-1, dst.shape[-1])[slot_mapping[valid].long(), : src.shape[1]] = src[valid].to(dst.dtype)


def _gather_kv(cache: torch.Tensor, block_table: torch.Tensor, n: int) -> torch.Tensor:
    """cache [blocks, Hk, bs, D] -> [n, Hk, D] for one sequence."""
    bs = cache.shape[2]
    nblk = (n + bs - 1) // bs
    x = cache[block_table[:nblk].long()]          # [nblk, Hk, bs, D]
    return x.permute(0, 2, 1, 3).reshape(nblk * bs, cache.shape[1], cache.shape[3])[:n]


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_tables: torch.Tensor, cu_q: torch.Tensor, seq_lens: torch.Tensor,
                    num_q_heads: int, scale: float, causal: bool = True, window: int = 0,
                    return_lse: bool = False, sink: int = 0):
    """Variable-length attention over the paged cache.  q [T, Hq*Dqk]; the queries of
    sequence b are rows cu_q[b]:cu_q[b+1] and sit at the END of its seq_lens[b] cached tokens.
    ``sink`` leading keys stay visible to every query whatever the sliding window."""
    hk, dqk, dv = k_cache.shape[1], k_cache.shape[3], v_cache.shape[3]
    hq = num_q_heads
    g = hq // hk
    t = q.shape[0]
    out = torch.zeros(t, hq * dv, dtype=q.dtype, device=q.device)
    lse = torch.full((t, hq), float("-inf"), dtype=torch.float32, device=q.device)
    cu = cu_q.tolist()
    sl = seq_lens.tolist()
    for b in range(len(sl)):
        qs, qe = cu[b], cu[b + 1]
        ql, n = qe - qs, sl[b]
        if ql == 0:
            continue
        kk = _gather_kv(k_cache, block_tables[b], n).float().repeat_interleave(g, dim=1)  # [n,Hq,D]
        vv = _gather_kv(v_cache, block_tables[b], n).float().repeat_interleave(g, dim=1)
        qq = q[qs:qe].view(ql, hq, dqk).float()
        s = torch.einsum("qhd,khd->hqk", qq, kk) * scale
        pos_q = torch.arange(n - ql, n, device=q.device).view(1, ql, 1)
        pos_k = torch.arange(n, device=q.device).view(1, 1, n)
        mask = torch.ones(1, ql, n, dtype=torch.bool, device=q.device)
        if causal:
            mask &= pos_k <= pos_q
        if window > 0:
            mask &= (pos_k > pos_q - window) | (pos_k < sink)
        s = s.masked_fill(~mask, float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l.unsqueeze(-1))
        p = torch.nan_to_num(p, nan=0.0)
        o = torch.einsum("hqk,khd->qhd", p, vv)
        out[qs:qe] = o.reshape(ql, hq * dv).to(q.dtype)
        lse[qs:qe] = l.t()
    return (out, lse) if return_lse else out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    return logits.float().argmax(dim=-1).to(torch.int32)


def apply_top_k_top_p(logits: torch.Tensor, top_k: Optional[torch.Tensor],
                      top_p: Optional[torch.Tensor]) -> torch.Tensor:
    """Mask (to -inf) everything outside the top-k / nucleus set; ties at the
    k-th value are kept.  logits [B,V] fp32."""
    logits = logits.float().clone()
    b, v = logits.shape
    if top_k is not None:
        k = top_k.clamp(min=1, max=v).long()
        k = torch.where(top_k.long() <= 0, torch.full_like(k, v), k)
        srt = logits.sort(dim=-1, descending=True).values
        kth = srt.gather(1, (k - 1).unsqueeze(1))
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p is not None:
        probs = logits.softmax(dim=-1)
        srt, idx = probs.sort(dim=-1, descending=True)
        csum = srt.cumsum(dim=-1)
        # keep the smallest prefix whose mass reaches p (always at least one token)
        drop = (csum - srt) >= top_p.unsqueeze(1)
        drop[:, 0] = False
        thr = torch.where(drop, torch.full_like(srt, 2.0), srt).amin(dim=-1, keepdim=True)
        logits = logits.masked_fill(probs < thr, float("-inf"))
    return logits


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], generator: Optional[torch.Generator] = None,
           seeds: Optional[torch.Tensor] = None, step_offset: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exponential-race sampling.  With ``seeds`` (int64 per row) every row draws from its own stream,
    keyed by its seed and the step offset, as the CUDA kernel does (not the same numbers: the same
    dependence on the seed)."""
    logits = logits.float()
    greedy = argmax(logits)
    if temperature is None:
        temperature = torch.ones(logits.shape[0], device=logits.device)
    t = temperature.clamp_min(1e-5).unsqueeze(1)
    masked = apply_top_k_top_p(logits / t, top_k, top_p)
    probs = masked.softmax(dim=-1)
    if seeds is not None:
        off = int(step_offset.flatten()[0]) if step_offset is not None else 0
        e = torch.empty_like(probs)
        g = torch.Generator(device="cpu")
        for i, sd in enumerate(seeds[: probs.shape[0]].tolist()):
            g.manual_seed((int(sd) * 0x2545F4914F6CDD1D + off) & 0x7FFFFFFFFFFFFFFF)
            e[i] = torch.empty(probs.shape[1]).exponential_(1.0, generator=g)
    else:
        e = torch.empty_like(probs).exponential_(1.0, generator=generator)
    tok = (probs / e).argmax(dim=-1).to(torch.int32)
    return torch.where(temperature < 1e-5, greedy, tok)


def moe_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], k: int, sigmoid: bool = False,
             n_group: int = 1, topk_group: int = 1, renorm: bool = False,
             scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Router reference.  logits [T,E] -> (ids int32 [T,k], weights fp32 [T,k]).
    Selection uses the bias-corrected scores, the returned weights the unbiased
    ones (DeepSeek-V3 "noaux_tc"); with groups, a group's score is the sum of its
    two best corrected scores when a bias is present, else its best score."""
    lf = logits.float()
    scores = torch.sigmoid(lf) if sigmoid else torch.softmax(lf, dim=-1)
    choice = scores + bias.float() if bias is not None else scores.clone()
    t, e = scores.shape
    if n_group > 1:
        grp = choice.view(t, n_group, e // n_group)
        gscore = grp.topk(2, dim=-1).values.sum(-1) if bias is not None else grp.max(-1).values
        gi = _stable_topk(gscore, topk_group)
        gmask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, gi, True)
        choice = choice.masked_fill(~gmask.unsqueeze(-1).expand(t, n_group, e // n_group).reshape(t, e),
                                    float("-inf"))
    ids = _stable_topk(choice, k)
    w = scores.gather(1, ids)
    if renorm:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return ids.to(torch.int32), (w * scale).float()


def _stable_topk(x: torch.Tensor, k: int) -> torch.Tensor:
    """top-k indices, lowest index first among equal values (the CUDA kernel's tie rule)."""
    order = torch.sort(x, dim=-1, descending=True, stable=True).indices
    return order[:, :k]


def moe_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_ids: torch.Tensor,
                topk_w: torch.Tensor, swiglu_interleaved: bool = True) -> torch.Tensor:
    """Dense reference of the routed experts: out[t] = sum_j w[t,j] * MLP_{id[t,j]}(x[t])."""
    t, h = x.shape
    out = torch.zeros(t, h, dtype=torch.float32, device=x.device)
    for e in topk_ids.unique().tolist():
        if e < 0:
            continue
        rows, js = (topk_ids == e).nonzero(as_tuple=True)
        xe = x[rows]
        hmid = gemm(xe, w13[e], swiglu=swiglu_interleaved, out_dtype=x.dtype)
        if not swiglu_interleaved:
            hmid = silu_and_mul(hmid)
        ye = gemm(hmid, w2[e], out_dtype=x.dtype)
        out.index_add_(0, rows, ye.float() * topk_w[rows, js].unsqueeze(1))
    return out.to(x.dtype)


def mla_decode(q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
               num_seqs: int, q_len: int, num_heads: int, scale: float,
               topk_indices: Optional[torch.Tensor] = None, return_lse: bool = False):
    """Absorbed MLA reference.  q [T, N*576], cache [blocks, bs, 576] -> [T, N*512].
    Query token i of a sequence sees keys 0 .. seq_len - q_len + i; with
    ``topk_indices`` [T, topk] only those positions (negative = hole)."""
    bs = cache.shape[1]
    out = torch.zeros(q.shape[0], num_heads * 512, dtype=q.dtype, device=q.device)
    lse = torch.full((q.shape[0], num_heads), float("-inf"), dtype=torch.float32, device=q.device)
    flat = cache.view(-1, 576)
    for b in range(num_seqs):
        n = int(seq_lens[b])
        for i in range(q_len):
            t = b * q_len + i
            if topk_indices is not None:
                pos = topk_indices[t]
                pos = pos[pos >= 0].long()
            else:
                pos = torch.arange(max(0, n - q_len + i + 1), device=q.device)
            if pos.numel() == 0:
                continue
            rows = block_tables[b][pos // bs].long() * bs + pos % bs
            kv = flat[rows].float()                                   # [L, 576]
            qq = q[t].view(num_heads, 576).float()
            sc = qq @ kv.t() * scale
            p = torch.softmax(sc, dim=-1)
            lse[t] = torch.logsumexp(sc, dim=-1)
            out[t] = (p @ kv[:, :512]).reshape(-1).to(q.dtype)
    return (out, lse) if return_lse else out


def spec_verify(draft: torch.Tensor, target: torch.Tensor, bonus: torch.Tensor, cu: torch.Tensor,
                max_spec: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """draft/target [T] tokens at the draft positions (request b owns cu[b]:cu[b+1]),
    bonus [B].  Row b of the result: target tokens up to and including the first
    mismatch with the draft, plus the bonus token when every draft matched; -1 padded."""
    b = cu.numel() - 1
    out = torch.full((b, max_spec + 1), -1, dtype=torch.int32, device=draft.device)
    num = torch.zeros(b, dtype=torch.int32, device=draft.device)
    cul = cu.tolist()
    d, t, bo = draft.tolist(), target.tolist(), bonus.tolist()
    for r in range(b):
        emitted, ok = 0, True
        for i in range(cul[r], min(cul[r + 1], cul[r] + max_spec)):
            out[r, emitted] = t[i]
            emitted += 1
            if t[i] != d[i]:
                ok = False
                break
        if ok:
            out[r, emitted] = bo[r]
            emitted += 1
        num[r] = emitted
    return out, num


def quant_int8_per_token(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    xf = x.float()
    scale = xf.abs().amax(dim=-1).clamp_min(1e-10) / 127.0
    q = torch.round(xf / scale.unsqueeze(-1)).clamp_(-127, 127).to(torch.int8)
    return q, scale


def gemm_scaled(a_q: torch.Tensor, w_q: torch.Tensor, a_scale: torch.Tensor, w_scale: torch.Tensor,
                bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    acc = a_q.double() @ w_q.double().t()          # exact for int8 products
    out = acc.float() * a_scale.float().reshape(-1, 1) * w_scale.float().reshape(1, -1)
    if bias is not None:
        out = out + bias.float()
    if residual is not None:
        out = out + residual.float()
    return out.to(out_dtype or torch.bfloat16)


def merge_attn_states(outs: torch.Tensor, lses: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """outs [N,T,H,D], lses [N,T,H] -> (out [T,H,D], lse [T,H]); -inf partials are ignored."""
    l = lses.float()
    m = l.max(dim=0).values
    w = torch.exp(l - torch.where(torch.isinf(m), torch.zeros_like(m), m))
    w = torch.where(torch.isinf(l), torch.zeros_like(w), w)
    denom = w.sum(0)
    out = (outs.float() * (w / denom.clamp_min(1e-38)).unsqueeze(-1)).sum(0)
    lse = torch.where(denom > 0, m + torch.log(denom.clamp_min(1e-38)), torch.full_like(m, float("-inf")))
    return out.to(outs.dtype), lse


def gather_cache(cache: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor) -> torch.Tensor:
    bs = cache.shape[1]
    parts = []
    for b, n in enumerate(seq_lens.tolist()):
        pos = torch.arange(n, device=cache.device)
        rows = block_tables[b][pos // bs].long() * bs + pos % bs
        parts.append(cache.reshape(-1, *cache.shape[2:])[rows])
    return torch.cat(parts) if parts else cache.new_zeros(0, *cache.shape[2:])


def quant_per_token(y: torch.Tensor, kind: str):
    """Per-row symmetric dynamic quantisation: int8 (amax/127, round to nearest even) or e4m3 (amax/448)."""
    yf = y.float()
    amax = yf.abs().amax(dim=-1).clamp_min(1e-10)
    if kind == "fp8":
        scale = amax / 448.0
        q = (yf / scale.unsqueeze(-1)).to(torch.float8_e4m3fn)
    else:
        scale = amax / 127.0
        q = torch.round(yf * (1.0 / scale).unsqueeze(-1)).clamp_(-127, 127).to(torch.int8)
    return q, scale


def rms_norm_quant(x, weight, eps, residual=None, kind="int8", want_bf16=False):
    if residual is not None:
        s = (x.float() + residual.float()).to(x.dtype)
        residual.copy_(s)
        x = s
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)
    q, scale = quant_per_token(y, kind)
    return q, scale, (y if want_bf16 else None)


def silu_and_mul_quant(x, kind="int8"):
    i = x.shape[-1] // 2
    y = (torch.nn.functional.silu(x[..., :i].float()) * x[..., i:].float()).to(x.dtype)
    return quant_per_token(y, kind)


def dsa_indexer_topk(q, w, index_cache, block_tables, positions, num_seqs, topk, cu_q=None, q_len=1,
                     return_scores=False):
    """Dense reference of the sparse-attention indexer (see ``ops.dsa_indexer_topk``)."""
    t, h, d = q.shape
    bs = index_cache.shape[1]
    flat = index_cache.reshape(-1, d).float()
    out = torch.full((t, topk), -1, dtype=torch.int32, device=q.device)
    ld = (block_tables.shape[1] * bs + 127) // 128 * 128
    scores = torch.full((t, ld), float("-inf"), dtype=torch.float32, device=q.device)
    cu = cu_q.tolist() if cu_q is not None else [i * q_len for i in range(num_seqs + 1)]
    for b in range(num_seqs):
        qs, qe = cu[b], cu[b + 1]
        if qe <= qs or int(positions[qs]) < 0:
            continue
        n = int(positions[qe - 1]) + 1
        pos = torch.arange(n, device=q.device)
        rows = block_tables[b][pos // bs].long() * bs + pos % bs
        keys = flat[rows]
        logits = torch.einsum("thd,ld->thl", q[qs:qe].float(), keys).relu_()
        sc = (logits * w[qs:qe].float().unsqueeze(-1)).sum(1)
        mask = pos.unsqueeze(0) > positions[qs:qe].long().unsqueeze(1)
        sc = sc.masked_fill(mask, float("-inf"))
        scores[qs:qe, :n] = sc
        k = min(topk, n)
        vals, idx = sc.topk(k, dim=-1)
        idx = torch.where(torch.isinf(vals), torch.full_like(idx, -1), idx)
        out[qs:qe, :k] = idx.to(torch.int32)
    return (out, scores) if return_scores else out


def gemm_fp8_block(a_q, a_scale, w_q, w_scale, bias=None, residual=None, out_dtype=None):
    """fp32 reference of the block-scaled e4m3 product (scales: a [M, K/128], w [N/128, K/128])."""
    m, k = a_q.shape
    a = a_q.float() * a_scale.float().repeat_interleave(128, dim=1)[:, :k]
    w = dequant_fp8_block(w_q, w_scale)
    y = a @ w.t()
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or torch.bfloat16)


def grouped_gemm_fp8_block(a_q, a_scale, w_q, w_scale, expert_offsets, swiglu=False, up_scale_row0=0):
    """fp32 reference of the grouped block-scaled product (see ``ops.grouped_gemm_fp8_block``)."""
    e, n, k = w_q.shape
    a = a_q.float() * a_scale.float().repeat_interleave(128, dim=1)[:, :k]
    out = torch.zeros(a.shape[0], n // 2 if swiglu else n, dtype=torch.float32, device=a.device)
    offs = expert_offsets.tolist()
    r = torch.arange(n, device=a.device)
    for i in range(e):
        if swiglu:
            half = n // 2
            src = (r // 16) * 8 + r % 8
            blk = src // 128 + ((r // 8) % 2) * up_scale_row0
        else:
            blk = r // 128
        s = w_scale[i][blk].float().repeat_interleave(128, dim=1)[:, :k]
        w = w_q[i].float() * s
        y = a[offs[i]: offs[i + 1]] @ w.t()
        if swiglu:
            y = y.view(-1, n // 16, 2, 8)
            y = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(-1, half)
        out[offs[i]: offs[i + 1]] = y
    return out.to(torch.bfloat16)
