"""A deliberately plain PyTorch Llama (no paging, no fusion) used as the oracle
for end-to-end token equality tests."""
import torch
import torch.nn.functional as F


def rope(x, pos, theta, rot_dim):
    # x [T, H, D] neox style
    d = rot_dim
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = pos.float()[:, None] * inv[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x0, x1 = x[..., : d // 2].float(), x[..., d // 2: d].float()
    out = torch.cat([x0 * c - x1 * s, x1 * c + x0 * s, x[..., d:].float()], dim=-1)
    return out.to(x.dtype)


def rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


@torch.no_grad()
def forward(weights, cfg, tokens):
    """tokens: list[int]; returns logits [T, V] of a full causal forward pass."""
    T = len(tokens)
    ids = torch.tensor(tokens)
    pos = torch.arange(T)
    h = weights["model.embed_tokens.weight"][ids]
    H, Hk, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        x = rms(h, weights[p + "input_layernorm.weight"], cfg.rms_norm_eps)
        q = (x @ weights[p + "self_attn.q_proj.weight"].t()).view(T, H, D)
        k = (x @ weights[p + "self_attn.k_proj.weight"].t()).view(T, Hk, D)
        v = (x @ weights[p + "self_attn.v_proj.weight"].t()).view(T, Hk, D)
        q, k = rope(q, pos, cfg.rope_theta, D), rope(k, pos, cfg.rope_theta, D)
        k = k.repeat_interleave(H // Hk, dim=1)
        v = v.repeat_interleave(H // Hk, dim=1)
        s = torch.einsum("qhd,khd->hqk", q.float(), k.float()) * D ** -0.5
        s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)), float("-inf"))
        a = torch.einsum("hqk,khd->qhd", s.softmax(-1), v.float()).reshape(T, H * D).to(h.dtype)
        h = h + a @ weights[p + "self_attn.o_proj.weight"].t()
        x = rms(h, weights[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        g = x @ weights[p + "mlp.gate_proj.weight"].t()
        u = x @ weights[p + "mlp.up_proj.weight"].t()
        h = h + (F.silu(g.float()).to(h.dtype) * u) @ weights[p + "mlp.down_proj.weight"].t()
    h = rms(h, weights["model.norm.weight"], cfg.rms_norm_eps)
    return h.float() @ weights["lm_head.weight"].float().t()


def make_weights(cfg, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    w = {}

    def r(*shape):
        return (torch.randn(*shape, generator=g) * 0.02).to(dtype)

    H, Hk, D, hid, I, V = (cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.hidden_size,
                           cfg.intermediate_size, cfg.vocab_size)
    w["model.embed_tokens.weight"] = r(V, hid)
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = torch.ones(hid, dtype=dtype)
        w[p + "post_attention_layernorm.weight"] = torch.ones(hid, dtype=dtype)
        w[p + "self_attn.q_proj.weight"] = r(H * D, hid)
        w[p + "self_attn.k_proj.weight"] = r(Hk * D, hid)
        w[p + "self_attn.v_proj.weight"] = r(Hk * D, hid)
        w[p + "self_attn.o_proj.weight"] = r(hid, H * D)
        w[p + "mlp.gate_proj.weight"] = r(I, hid)
        w[p + "mlp.up_proj.weight"] = r(I, hid)
        w[p + "mlp.down_proj.weight"] = r(hid, I)
    w["model.norm.weight"] = torch.ones(hid, dtype=dtype)
    w["lm_head.weight"] = r(V, hid)
    return w


@torch.no_grad()
def greedy_generate(weights, cfg, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        logits = forward(weights, cfg, toks)
        toks.append(int(logits[-1].argmax()))
    return toks[len(prompt):]
