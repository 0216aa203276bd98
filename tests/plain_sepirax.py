"""A plain, slow statement of the Sepirax decoder, one function per mechanism, written from the
design's equations and sharing no code with the package.  Everything is a whole-sequence
computation on the CPU in the dtype of the weights it is given (float64 in the tests): no
cache, no state carried between calls, no batch.  ``forward`` returns the logits of every
position and, on request, the residual stream after every layer.

Conventions: a linear map is stored [out, in] and applied as ``x @ W.T``; positions count
from 0; ``w`` maps tensor names of a model folder to tensors.
"""
from __future__ import annotations

import math

import torch


# ---------------------------------------------------------------- norms
def dynamic_tanh(x, weight, bias, alpha):
    """y = tanh(alpha x) * weight + bias; no statistics of the row are taken."""
    return torch.tanh(alpha * x) * weight + bias


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ---------------------------------------------------------------- rotary frequencies with YaRN
def yarn_frequencies(dims, base, factor, original, fast, slow):
    """The dims/2 angular frequencies and the magnitude that multiplies cos and sin.

    g_i = base^(-2i/dims).  The pair index at which a wave makes t turns over ``original``
    positions is d(t) = dims ln(original / (2 pi t)) / (2 ln base); between lo = floor(d(fast))
    and hi = ceil(d(slow)) (clamped to 0 and dims - 1) a ramp goes from 0 to 1; a pair keeps g_i
    where the ramp is 0 and gets g_i / factor where it is 1."""
    def d(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(d(fast)), 0)
    hi = min(math.ceil(d(slow)), dims - 1)
    out = []
    for i in range(dims // 2):
        g = base ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(g / factor * ramp + g * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_half_pairs(x, positions, freqs, magnitude, dims):
    """x [T, ..., R]: the first ``dims`` entries of the last axis are rotated, entry i with entry
    i + dims/2, by the angle position * freqs[i]; cos and sin are scaled by ``magnitude``."""
    half = dims // 2
    ang = positions.to(x.dtype)[:, None] * torch.tensor(freqs, dtype=x.dtype)[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c = (torch.cos(ang) * magnitude).reshape(shape)
    s = (torch.sin(ang) * magnitude).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------- latent attention
def latent_attention(h, w, p, mx, eps):
    """Queries and keys/values through low-rank latents; one rotated key part shared by all heads."""
    T = h.shape[0]
    H, dn, dr, dv, rk = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    rot = mx["rot"]
    sc = rot.get("scaling")
    if sc:
        freqs, mag = yarn_frequencies(rot["dims"], rot["base"], sc["factor"], sc["original"], sc["fast"], sc["slow"])
    else:
        freqs, mag = [rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], 1.0
    pos = torch.arange(T)
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_half_pairs(q[..., dn:], pos, freqs, mag, rot["dims"])
    kv = h @ w[p + "dkv"].T
    c = unit_rms(kv[:, :rk], eps) * w[p + "dkv.norm"]
    k_rot = rotate_half_pairs(kv[:, rk:], pos, freqs, mag, rot["dims"])             # [T, dr], one for all heads
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * mx["scale"]
    visible = pos[None, :] <= pos[:, None]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    o = torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v).reshape(T, H * dv)
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# ---------------------------------------------------------------- matrix memory (mLSTM)
def mlstm(h, w, p, mx, eps):
    """Token by token: a matrix S [dim, vdim] and a vector n [dim] per head, kept relative to a
    running maximum m of the accumulated log gates (m starts at 0)."""
    T = h.shape[0]
    H, dk, dv, cap = mx["heads"], mx["dim"], mx["vdim"], mx["gate_cap"]
    q = (h @ w[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    gi = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                                  # log input gate
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))  # log forget gate
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    n = torch.zeros(H, dk, dtype=h.dtype)
    m = torch.zeros(H, dtype=h.dtype)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        m_new = torch.maximum(gf[t] + m, gi[t])
        keep = torch.exp(gf[t] + m - m_new)
        take = torch.exp(gi[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        num = torch.einsum("hkv,hk->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    o = unit_rms(out, eps).reshape(T, H * dv) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# ---------------------------------------------------------------- routed feed-forward
def route(z, top, n_groups, keep_groups):
    """z [T, E] router logits -> (chosen experts [T, top], their weights [T, top]).  Scores are a
    softmax over all experts; a group of neighbours counts by its best score; experts outside the
    best ``keep_groups`` groups cannot be chosen; the weights are the chosen scores over their sum."""
    T, E = z.shape
    s = torch.softmax(z, dim=-1)
    per = E // n_groups
    gscore = s.reshape(T, n_groups, per).max(-1).values
    best = torch.topk(gscore, keep_groups, dim=-1).indices
    allowed = torch.zeros(T, n_groups, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    masked = torch.where(allowed[:, :, None].expand(T, n_groups, per).reshape(T, E), s, torch.full_like(s, -1.0))
    idx = torch.topk(masked, top, dim=-1).indices
    chosen = torch.gather(s, 1, idx)
    return idx, chosen / (chosen.sum(-1, keepdim=True) + 1e-20)


def routed_experts(h, w, p, ml):
    r = ml["router"]
    idx, wt = route(h @ w[p + "router"].T, r["top"], r["groups"]["count"], r["groups"]["keep"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            a = h[t] @ w[f"{p}e{e}.gate"].T
            y = (a * torch.sigmoid(a) * (h[t] @ w[f"{p}e{e}.up"].T)) @ w[f"{p}e{e}.down"].T
            out[t] += wt[t, j] * y
    return out


# ---------------------------------------------------------------- the decoder
def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of every position of one sequence; ``layers_out`` (a list) receives the
    residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    mult = cfg["residual_mult"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]

    def norm(name, v):
        return dynamic_tanh(v, w[name], w[name + ".b"], w[name + ".alpha"])

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        hin = norm(p + "norm1", x)
        if layer["type"] == "latent_attention":
            y = latent_attention(hin, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "mlstm":
            y = mlstm(hin, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + mult * y
        if layer.get("mlp") is not None:
            x = x + mult * routed_experts(norm(p + "norm2", x), w, p + "mlp.", layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = norm("final.norm", x) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
