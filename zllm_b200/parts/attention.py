"""Grouped-query attention over the paged cache.

q = Wq h, k = Wk h, v = Wv h without biases (zllm
src/backend/candle/quantized_llama_fork.rs:462-473); head ``i`` is columns
i*hd..(i+1)*hd-1 (fork.rs:475-487); q and k are rotated, v is not
(fork.rs:489-490); the new k and v go to the cache at their positions
(fork.rs:495-496) before any row attends; scores q.k / sqrt(hd), query head h
reads kv head h // (nh/nkv), key j visible to a query at position p iff j <= p
(and j > p - window when a window is set), softmax and the weighted sum in
float32 (fork.rs:518-533; src/backend/gpu/shaders.rs:703-723); heads concatenated
to [T, nh*hd], which may differ from the width (fork.rs:514-516); output
projection added to the residual (fork.rs:535,945).

The three projections are stacked into one matrix at load, as the reference's
Vulkan path concatenates weights to save a pass (src/backend/vulkan/mod.rs:1141-1181).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..errors import ConfigError
from .base import KVCacheSpec, Mixer, WeightSpec, register_mixer


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position_encoding=None, window: Optional[int] = None, scale: Optional[float] = None,
                 init_std: float = 0.02):
        if n_heads % n_kv_heads:
            raise ConfigError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        if head_dim % 16:
            raise ConfigError(f"attention: head_dim {head_dim} must be a multiple of 16")
        self.hidden_size = int(hidden_size)
        self.n_heads = int(n_heads)
        self.n_kv_heads = int(n_kv_heads)
        self.head_dim = int(head_dim)
        self.position_encoding = position_encoding
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.init_std = init_std
        self.w_qkv = None
        self.w_o = None

    def weight_specs(self):
        H, hd = self.hidden_size, self.head_dim
        s = ("normal", self.init_std)
        return {
            "q_proj": WeightSpec((self.n_heads * hd, H), "matrix", s),
            "k_proj": WeightSpec((self.n_kv_heads * hd, H), "matrix", s),
            "v_proj": WeightSpec((self.n_kv_heads * hd, H), "matrix", s),
            "o_proj": WeightSpec((H, self.n_heads * hd), "matrix", s),
        }

    def cache_spec(self):
        return KVCacheSpec(self.n_kv_heads, self.head_dim, self.window)

    def bind(self, rt):
        super().bind(rt)
        if self.position_encoding is not None and self.position_encoding.rt is None:
            self.position_encoding.bind(rt)
        prepare = getattr(rt.ops, "prepare", None)
        if prepare is not None:                     # the attention kernels of this precision, built together
            prepare(rt.ops.PAGED_ATTENTION_KERNELS[rt.dtype])

    def load(self, tensors):
        self.w_qkv = torch.cat([tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]], dim=0).contiguous()
        self.w_o = tensors["o_proj"].contiguous()

    accepts_input_norm = True
    capturable = True

    def step_planner(self):
        # the tiled attention kernels want each portion cut into query tiles of their own size
        return getattr(self.rt.ops, "plan_query_tiles", None)

    def forward(self, h, residual, ctx, cache, write_cache: bool = True, input_norm=None):
        """``input_norm`` None: h is the normed input.  Otherwise h is the float32 residual and
        ``input_norm`` = (weight, eps) of the RMS norm to apply to it inside the QKV product."""
        ops = self.rt.ops
        T = h.shape[0]
        nq, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        qkv = ctx.ws.get("qkv", (T, (nq + 2 * nkv) * hd), self.rt.dtype)
        rot = self.position_encoding.rotary() if self.position_encoding is not None else None
        ops.qkv_rope_store(h, input_norm, self.w_qkv, qkv, ctx, rot, cache, nq, nkv, hd, write_cache, ctx.ws)
        att = ctx.ws.get("attn_out", (T, nq * hd), self.rt.dtype)
        ops.paged_attention(qkv, att, ctx, cache, nq, nkv, hd, self.scale, self.window)
        ops.linear(att, self.w_o, residual, "add")


@register_mixer("window_attention")
class WindowAttention(Mixer):
    """Grouped-query attention whose mask, value size and output gate are parameters.

    q = Wq h [H heads of ``head_dim``], k = Wk h [G heads], v = Wv h [G heads of ``value_dim``], no
    biases; query head a reads key/value head a // (H / G).  q and k are rotated by the mixer's
    position encoding (frequencies only: the angle position * f is formed in float32 in the kernel).
    Query i sees key j iff j <= i and (i - j < window or j < keep_first); ``window`` None: every
    earlier key.  The kept first positions keep their own positions for the rotation.  Softmax
    over the visible keys in float32.  With ``head_gate`` a head's output is multiplied by
    sigmoid(Wg h) (one number per head, from the same input as the projections) before Wo.

    Everything that reads h is ONE product: the rows of Wq, Wk, Wv and Wg are stacked (and padded
    with zero rows to a multiple of 8 so that the tensor-core products take the matrix).  The cache
    holds key rows of ``head_dim`` and value rows of ``value_dim`` entries; pages that the window has
    passed go back to the pool, those of the first ``keep_first`` positions stay.
    """

    accepts_input_norm = True
    can_overwrite = True
    capturable = True
    KERNELS = ("attention_window",)

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int, value_dim: Optional[int] = None,
                 position_encoding=None, window: Optional[int] = None, keep_first: int = 0, scale: Optional[float] = None,
                 head_gate: bool = False, init_std: float = 0.02):
        if n_heads <= 0 or n_kv_heads <= 0 or n_heads % n_kv_heads:
            raise ConfigError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        self.hidden_size = int(hidden_size)
        self.n_heads, self.n_kv_heads = int(n_heads), int(n_kv_heads)
        self.head_dim = int(head_dim)
        self.value_dim = int(value_dim) if value_dim else self.head_dim
        self.position_encoding = position_encoding
        self.window = int(window) if window else None
        self.keep_first = int(keep_first or 0) if self.window else 0
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.head_gate = bool(head_gate)
        self.init_std = init_std
        if self.head_dim <= 0 or self.value_dim <= 0 or self.keep_first < 0:
            raise ConfigError("attention: sizes must be positive")
        if position_encoding is not None and position_encoding.dims > self.head_dim:
            raise ConfigError(f"attention: {position_encoding.dims} rotated entries exceed the head size {self.head_dim}")
        H, G, dk, dv = self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim
        # columns of the stacked product: queries, keys, values, gates
        self.off_k = H * dk
        self.off_v = self.off_k + G * dk
        self.off_g = self.off_v + G * dv
        self.n_proj = -(-(self.off_g + (H if self.head_gate else 0)) // 8) * 8
        self.w_in = self.w_o = None

    def weight_specs(self):
        W = self.hidden_size
        s = ("normal", self.init_std)
        out = {"q": WeightSpec((self.n_heads * self.head_dim, W), "matrix", s),
               "k": WeightSpec((self.n_kv_heads * self.head_dim, W), "matrix", s),
               "v": WeightSpec((self.n_kv_heads * self.value_dim, W), "matrix", s),
               "o": WeightSpec((W, self.n_heads * self.value_dim), "matrix", s)}
        if self.head_gate:
            out["g"] = WeightSpec((self.n_heads, W), "matrix", s)
        return out

    def cache_spec(self):
        return KVCacheSpec(self.n_kv_heads, self.head_dim, self.window, True,
                           self.value_dim if self.value_dim != self.head_dim else None, self.keep_first)

    def bind(self, rt):
        super().bind(rt)
        if self.position_encoding is not None and self.position_encoding.rt is None:
            self.position_encoding.bind(rt)
        prepare = getattr(rt.ops, "prepare", None)
        if prepare is not None:
            prepare(self.KERNELS)

    def load(self, tensors):
        rows = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if self.head_gate else [])
        w = torch.cat(rows, dim=0)
        pad = self.n_proj - w.shape[0]
        if pad:
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
        self.w_in = w.contiguous()
        self.w_o = tensors["o"].contiguous()

    def step_planner(self):
        return getattr(self.rt.ops, "plan_query_tiles", None)

    def forward(self, h, out, ctx, cache, write_cache: bool = True, input_norm=None, accumulate: bool = True):
        """``input_norm`` as for ``paged_attention``; ``accumulate`` False: ``out`` is written, not added to."""
        ops = self.rt.ops
        T = h.shape[0]
        proj = ctx.ws.get("attn_proj", (T, self.n_proj), self.rt.dtype)
        if input_norm is not None:
            ops.linear_normed(h, input_norm[0], input_norm[1], self.w_in, proj, "store", ctx.ws)
        else:
            ops.linear(h, self.w_in, proj, "store")
        freqs = self.position_encoding.frequencies() if self.position_encoding is not None else None
        ops.rotate_store_kv(proj, self.off_k, self.off_v, ctx, freqs, cache, self.n_heads, self.n_kv_heads, self.head_dim,
                            self.value_dim, write_cache)
        att = ctx.ws.get("attn_out", (T, self.n_heads * self.value_dim), self.rt.dtype)
        ops.window_attention(proj, self.off_g if self.head_gate else -1, att, ctx, cache, self.n_heads, self.n_kv_heads,
                             self.head_dim, self.value_dim, self.scale, self.window, self.keep_first)
        ops.linear(att, self.w_o, out, "add" if accumulate else "store")
