"""Unfolded, unsharded, autograd-differentiated fp32 model used as the oracle for the
engine: same maths as ``dhellam_b200.models`` written the plain PyTorch way."""
import math

import torch
import torch.nn.functional as F


def _norm(cfg, x, w, b):
    if cfg.norm == "rmsnorm":
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * w
    return F.layer_norm(x, (x.shape[-1],), w, b, cfg.norm_eps)


def _rope(x, pos, theta):
    # x [S, B, H, d]
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    ang = pos.double()[:, None] * inv[None, :]
    c, s = ang.cos().float()[:, None, None, :], ang.sin().float()[:, None, None, :]
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)


def layer_forward(cfg, w, x, B, pos_seq, moe_aux=None):
    """x [S*B, h] sequence-first rows; ``pos_seq [S]`` positions."""
    T, h = x.shape
    S = T // B
    nq, nkv, d = cfg.num_attention_heads, cfg.num_query_groups, cfg.head_dim
    y = _norm(cfg, x, w["ln_attn_weight"], w.get("ln_attn_bias"))
    qkv = y @ w["column_attn_weight"].t()
    q = qkv[:, : nq * d].view(S, B, nq, d)
    k = qkv[:, nq * d:(nq + nkv) * d].view(S, B, nkv, d)
    v = qkv[:, (nq + nkv) * d:].view(S, B, nkv, d)
    if cfg.position == "rope":
        q, k = _rope(q, pos_seq, cfg.rope_theta), _rope(k, pos_seq, cfg.rope_theta)
    g = nq // nkv
    qh = q.permute(1, 2, 0, 3)
    kh = k.permute(1, 2, 0, 3).repeat_interleave(g, 1)
    vh = v.permute(1, 2, 0, 3).repeat_interleave(g, 1)
    s = qh @ kh.transpose(-1, -2) / math.sqrt(d)
    order = pos_seq[:, None] >= pos_seq[None, :]
    s = s.masked_fill(~order, float("-inf"))
    o = (torch.softmax(s, -1) @ vh).permute(2, 0, 1, 3).reshape(T, nq * d)
    h1 = x + o @ w["linear_attn_weight"].t()
    y2 = _norm(cfg, h1, w["ln_mlp_weight"], w.get("ln_mlp_bias"))
    if cfg.is_moe:
        logits = y2 @ w["router_weight"].t()
        probs = torch.softmax(logits, -1)
        topv, topi = probs.topk(cfg.moe_top_k, -1)
        gates = topv / topv.sum(-1, keepdim=True)
        out = torch.zeros_like(y2)
        for e in range(cfg.num_experts):
            sel = (topi == e)
            rows = sel.any(-1).nonzero().squeeze(1)
            if rows.numel() == 0:
                continue
            gw = (gates * sel)[rows].sum(-1, keepdim=True)
            z = y2[rows] @ w["expert_column_weight"][e].t()
            f = z.shape[-1] // 2
            a = F.silu(z[:, :f]) * z[:, f:]
            out = out.index_add(0, rows, gw * (a @ w["expert_linear_weight"][e].t()))
        if moe_aux is not None:
            frac = torch.zeros(cfg.num_experts)
            frac = frac.index_add(0, topi.reshape(-1), torch.ones(topi.numel())) / topi.numel()
            moe_aux.append(cfg.num_experts * (frac * probs.mean(0)).sum())
        return h1 + out
    z = y2 @ w["column_mlp_weight"].t()
    if cfg.gated:
        f = z.shape[-1] // 2
        a = F.silu(z[:, :f]) * z[:, f:]
    else:
        a = F.gelu(z, approximate="tanh")
    return h1 + a @ w["linear_mlp_weight"].t()


def model_loss(cfg, layers, head, sample, moe_aux_coeff=0.0):
    """``sample [B, S+1]`` token ids -> mean next-token loss (fp32)."""
    B = sample.shape[0]
    tok = sample[:, :-1].t().reshape(-1)
    lab = sample[:, 1:].t().reshape(-1)
    S = sample.shape[1] - 1
    pos = torch.arange(S)
    x = head["word_embeddings"][tok]
    if cfg.position == "learned":
        x = x + head["position_embeddings"][pos[:, None].expand(-1, B).reshape(-1)]
    aux = []
    for w in layers:
        x = layer_forward(cfg, w, x, B, pos, aux)
    y = _norm(cfg, x, head["final_ln_weight"], head.get("final_ln_bias"))
    wout = head.get("output_weight", head["word_embeddings"])
    logits = y @ wout.t()
    loss = F.cross_entropy(logits, lab)
    if aux and moe_aux_coeff:
        loss = loss + moe_aux_coeff * torch.stack(aux).sum()
    return loss
