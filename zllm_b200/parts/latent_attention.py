"""Attention whose keys and values are linear maps of a small cached latent.

Per position the mixer computes, from its input h (width W):
    query latent   cq = rmsnorm(Wdq h) * gq                      [q_rank]
    queries        q  = Wuq cq, head by head [dim plain | rot_dim rotated]
    latent         c  = rmsnorm((Wdkv h)[:kv_rank]) * gc          [kv_rank]
    rotated key    kr = rotate((Wdkv h)[kv_rank:])                [rot_dim], one for all heads
and per head k = Uk c (plain part), v = Uv c.  The score of query i and key j is
scale * (q_plain . k_plain + rotate(q_rot) . kr), softmax over j <= i, the heads'
outputs concatenated, multiplied by sigmoid(Wg h), then Wo.

Only [c | kr] is cached (one row per position, no value rows).  The kernels never expand
it: Uk moves to the query side (q_lat = Uk_h^T q_plain) and Uv behind the weighted sum, so
decode reads kv_rank + rot_dim numbers per position instead of heads * (dim + vdim).

The three projections of h (Wdq, Wdkv, Wg) are stacked into one matrix at load.
``residual_scale`` multiplies the mixer's output on its way into the residual stream; it is
applied where the gate is, before the output product, so that product's epilogue can still
add into the float32 residual.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from .base import KVCacheSpec, Mixer, WeightSpec, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    capturable = True
    KERNELS = ("latent_attention", "gemm_grouped")

    def __init__(self, hidden_size: int, n_heads: int, head_dim: int, rot_dim: int, value_dim: int, q_rank: int,
                 kv_rank: int, scale: float, eps: float, position_encoding=None, residual_scale: float = 1.0,
                 init_std: float = 0.02):
        self.W = int(hidden_size)
        self.H = int(n_heads)
        self.dn, self.dr, self.dv = int(head_dim), int(rot_dim), int(value_dim)
        self.q_rank, self.kv_rank = int(q_rank), int(kv_rank)
        self.scale = float(scale)
        self.eps = float(eps)
        self.position_encoding = position_encoding
        self.residual_scale = float(residual_scale)
        self.init_std = init_std
        if min(self.H, self.dn, self.dv, self.q_rank, self.kv_rank) <= 0 or self.dr < 0:
            raise ConfigError("latent attention: sizes must be positive")
        if self.dr and position_encoding is None:
            raise ConfigError("latent attention: a rotated part needs a position encoding")
        if position_encoding is not None and getattr(position_encoding, "interleaved", False):
            raise ConfigError("latent attention rotates half-split pairs only")
        if position_encoding is not None and position_encoding.dims > self.dr:
            raise ConfigError(f"latent attention: {position_encoding.dims} rotated dimensions exceed rot_dim {self.dr}")

    def weight_specs(self):
        s = ("normal", self.init_std)
        H, W = self.H, self.W
        return {
            "dq": WeightSpec((self.q_rank, W), "matrix", s),
            "dq_norm": WeightSpec((self.q_rank,), "vector", ("one_plus_normal", 0.0)),
            "uq": WeightSpec((H * (self.dn + self.dr), self.q_rank), "matrix", s),
            "dkv": WeightSpec((self.kv_rank + self.dr, W), "matrix", s),
            "dkv_norm": WeightSpec((self.kv_rank,), "vector", ("one_plus_normal", 0.0)),
            "uk": WeightSpec((H * self.dn, self.kv_rank), "matrix", s),
            "uv": WeightSpec((H * self.dv, self.kv_rank), "matrix", s),
            "g": WeightSpec((H * self.dv, W), "matrix", s),
            "o": WeightSpec((W, H * self.dv), "matrix", s),
        }

    def cache_spec(self):
        return KVCacheSpec(1, self.kv_rank + self.dr, None, values=False)

    def bind(self, rt):
        super().bind(rt)
        if self.position_encoding is not None and self.position_encoding.rt is None:
            self.position_encoding.bind(rt)
        prepare = getattr(rt.ops, "prepare", None)
        if prepare is not None:
            mma = rt.dtype == torch.bfloat16 and self.kv_rank in getattr(rt.ops, "LATENT_MMA_RANKS", ()) and self.dr % 16 == 0
            prepare(self.KERNELS + (("latent_attention_mma",) if mma else ())
                    + (("gemm_grouped_mma",) if rt.dtype == torch.bfloat16 and self.dn % 32 == 0 else ()))

    def load(self, tensors):
        H = self.H
        # one product for everything that reads h: [query latent | latent, key part | gate]
        self.w_in = torch.cat([tensors["dq"], tensors["dkv"], tensors["g"]], dim=0).contiguous()
        self.off_kv = self.q_rank
        self.off_g = self.q_rank + self.kv_rank + self.dr
        self.w_uq = tensors["uq"].contiguous()
        # Uk per head, transposed so that it maps a head's plain query to the latent side: [H, kv_rank, dim]
        self.w_uk_t = tensors["uk"].reshape(H, self.dn, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv"].reshape(H, self.dv, self.kv_rank).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.q_norm = tensors["dq_norm"].to(torch.float32).contiguous()
        self.c_norm = tensors["dkv_norm"].to(torch.float32).contiguous()
        if self.position_encoding is None:
            dev = self.w_o.device
            self._freqs = (torch.zeros(1, dtype=torch.float32, device=dev)[:0], 1.0, 0)
        else:
            self._freqs = self.position_encoding.frequencies().as_tuple()

    def forward(self, h, residual, ctx, cache, write_cache: bool = True):
        ops, dt = self.rt.ops, self.rt.dtype
        T = h.shape[0]
        H, dn, dr, dv, rk = self.H, self.dn, self.dr, self.dv, self.kv_rank
        proj = ctx.ws.get("latent_in", (T, self.w_in.shape[0]), dt)
        ops.linear(h, self.w_in, proj, "store")
        cq = ctx.ws.get("latent_cq", (T, self.q_rank), dt)
        ops.latent_prepare(proj, 0, self.q_rank, self.off_kv, rk, dr, self.q_norm, self.c_norm, self.eps, self._freqs, cq,
                           ctx, cache, write_cache)
        q = ctx.ws.get("latent_q", (T, H * (dn + dr)), dt)
        ops.linear(cq, self.w_uq, q, "store")
        q_lat = ctx.ws.get("latent_qlat", (T, H * rk), torch.float32)
        ops.linear_heads(q, dn + dr, self.w_uk_t, q_lat)
        o_lat = ctx.ws.get("latent_olat", (T, H * rk), dt)
        ops.latent_attention(q_lat, q, dn + dr, o_lat, ctx, cache, H, rk, dr, self._freqs, self.scale)
        # values out of the latent, times the output gate and the residual scale
        og = ctx.ws.get("latent_og", (T, H * dv), dt)
        ops.linear_heads(o_lat, rk, self.w_uv, og, gate=(proj, self.off_g), out_scale=self.residual_scale)
        ops.linear(og, self.w_o, residual, "add")
