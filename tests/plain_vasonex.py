"""A plain, slow statement of the Vasonex decoder, one function per mechanism, written from the
design's equations and sharing no code with the package.  Everything is a whole-sequence
computation on the CPU in the dtype of the weights it is given (float64 in the tests): no
cache, no batch, nothing carried between calls.  ``forward`` returns the logits of every
position and, on request, the residual stream after every layer run.

Conventions: a linear map is stored [out, in] and applied as ``x @ W.T``; positions count
from 0; ``w`` maps tensor names of a model folder to tensors.

The design in short.  Every layer is a sandwich,

    x <- x + N1b(mixer(N1(x)));   x <- x + N2b(ff(N2(x)))        N = RMS norm with a weight,

the mixer is grouped-query attention with an interleaved rotation of the first ``rot.dims``
entries of every query and key head (frequencies stretched as in Llama 3.1), a sliding window
that also keeps the first ``keep_first`` positions visible, value heads of a size of their own
and one sigmoid output gate per head; the feed-forward is a SiLU-gated one with biases, or a
mixture of experts with sigmoid scores whose weight multiplies an expert's INPUT, plus a shared
expert behind a sigmoid gate of its own, or missing.  A layer may borrow another layer's tensors.
"""
from __future__ import annotations

import math

import torch


# ---------------------------------------------------------------- norm
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


# ---------------------------------------------------------------- rotation
def stretched_frequencies(dims, base, scaling):
    """f_i = base^(-2i/dims) for the dims/2 pairs; with ``scaling`` {factor, low, high, original}
    a wave longer than original/low is slowed down by ``factor``, one shorter than original/high
    is kept, and in between the two are blended linearly in s = (original/wavelength - low) /
    (high - low)."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            F, lo, hi, L = scaling["factor"], scaling["low"], scaling["high"], scaling["original"]
            wavelength = 2.0 * math.pi / f
            if wavelength > L / lo:
                f = f / F
            elif wavelength >= L / hi:
                s = (L / wavelength - lo) / (hi - lo)
                f = (1.0 - s) * f / F + s * f
        out.append(f)
    return out


def rotate_neighbour_pairs(x, positions, freqs, dims, angle_dtype=None):
    """x [T, heads, D]: entries (2i, 2i+1), i < dims/2, of the last axis are turned by the angle
    position * freqs[i]; entries from ``dims`` on pass unchanged."""
    adt = angle_dtype or x.dtype
    ang = positions.to(adt)[:, None] * torch.tensor(freqs, dtype=adt)[None, :]          # [T, dims/2]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).reshape(*x.shape[:-1], dims)
    return torch.cat([turned, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------- who sees whom
def visible(n, size, keep_first):
    """[n, n] booleans: query i sees key j iff j <= i and (i - j < size or j < keep_first);
    ``size`` None: every earlier key."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    near = (i - j < size) if size is not None else torch.ones(n, n, dtype=torch.bool)
    return (j <= i) & (near | (j < keep_first))


# ---------------------------------------------------------------- attention
def attention(h, w, p, mx, angle_dtype=None):
    """The mixer on a whole sequence h [T, W]; ``p`` is the prefix of its tensors."""
    T = h.shape[0]
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, dk)
    k = (h @ w[p + "k"].T).reshape(T, G, dk)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    rot = mx.get("rot")
    if rot and rot.get("dims"):
        freqs = stretched_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        pos = torch.arange(T)
        q = rotate_neighbour_pairs(q, pos, freqs, rot["dims"], angle_dtype)
        k = rotate_neighbour_pairs(k, pos, freqs, rot["dims"], angle_dtype)
    mask = mx.get("mask") or {}
    see = visible(T, mask.get("size"), mask.get("keep_first", 0))
    rep = H // G
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        s = (q[:, a] @ k[:, a // rep].T) * mx["scale"]
        s = s.masked_fill(~see, float("-inf"))
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, a // rep]
    gate = torch.sigmoid(h @ w[p + "g"].T)                                   # [T, H], one number per head
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ---------------------------------------------------------------- feed-forwards
def gated_ff(h, w, p):
    """down(silu(gate h + b) * (up h + b)) + b."""
    g = h @ w[p + "gate"].T + w[p + "gate.b"]
    u = h @ w[p + "up"].T + w[p + "up.b"]
    return (g * torch.sigmoid(g) * u) @ w[p + "down"].T + w[p + "down.b"]


def gelu(z):
    """The exact form: z Phi(z)."""
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def small_ff(x, w, p):
    """down(gelu(up x)), no biases: an expert."""
    return gelu(x @ w[p + "up"].T) @ w[p + "down"].T


def mixture(h, w, p, mlp, forced=None):
    """Every token goes to its ``top`` best experts by sigmoid score; the score multiplies what the
    expert reads; a shared expert, if there is one, is added behind a sigmoid gate per token.
    ``forced`` [T, top]: the experts to take instead of the best ones (to follow an implementation
    through a close call between two scores)."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    score = torch.sigmoid(h @ w[p + "router"].T)                             # [T, E]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(score[t, e]), e))[:top]
        if forced is not None:
            order = [int(e) for e in forced[t]]
        for e in order:
            out[t] += small_ff(score[t, e] * h[t], w, f"{p}e{e}.")
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * small_ff(h, w, p + "shared.")
    return out


def router_margin(h, w, p, mlp):
    """Per token: how far the last chosen expert's router logit lies above the first one not chosen, as a
    fraction of the token's largest |logit| (infinite when every expert is chosen)."""
    z = h @ w[p + "router"].T
    top = mlp["router"]["top"]
    if top >= z.shape[1]:
        return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    best = z.sort(-1, descending=True).values
    return (best[:, top - 1] - best[:, top]) / z.abs().max(-1).values


# ---------------------------------------------------------------- the model
def forward(tokens, cfg, w, want_layers=False, angle_dtype=None, want_margins=False, forced=None):
    """logits [T, vocab] of the token list; with ``want_layers`` also the residual stream after
    every layer run, [runs, T, width]; with ``want_margins`` also, per position, the smallest
    ``router_margin`` over the layer runs with a mixture (a close call there means that an
    implementation with other roundings may send the token to another expert).  ``forced``
    {layer run: [T, top] expert ids}: the choices to take in those runs."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    streams = []
    margins = torch.full((len(tokens),), float("inf"), dtype=x.dtype)
    for i, ly in enumerate(cfg["layers"]):
        src = ly.get("weights_of", i)
        src = i if src is None else src
        p = f"l{src}."
        y = attention(rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", ly["mixer"], angle_dtype)
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        mlp = ly.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] != "dense" and want_margins:
                margins = torch.minimum(margins, router_margin(h, w, p + "mlp.", mlp))
            y = gated_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else \
                mixture(h, w, p + "mlp.", mlp, forced[i] if forced is not None else None)
            x = x + rms_norm(y, w[p + "norm2b"], eps)
        streams.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    if want_layers or want_margins:
        return (logits,) + ((torch.stack(streams),) if want_layers else ()) + ((margins,) if want_margins else ())
    return logits
