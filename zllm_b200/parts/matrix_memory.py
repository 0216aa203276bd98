"""A matrix memory with exponential gates (the mLSTM layer of xLSTM) as a mixer with state.

Per head, from the mixer's input h: q = Wq h * dk^(-1/2), k = Wk h [dk], v = Wv h [dv], and two
scalar log gates, i = cap tanh((Wi h + bi) / cap) and f = logsigmoid(cap tanh((Wf h + bf) / cap)).
The head keeps a matrix S [dk, dv], a vector n [dk] and a running maximum m (all zero at the
start of a sequence, m too):
    m' = max(f + m, i);  S' = exp(f + m - m') S + exp(i - m') k v^T;  n' likewise with k alone
    out = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
Each head's out is divided by its root mean square, the heads are concatenated and multiplied by
a learned vector and by sigmoid(Wg h), then Wo.

The state lives in the request's state slot as float32 [heads * (dk*dv + dk + 1)], is read and
written by device-side slot indices only, and walks token by token whatever the step's cut, so
a position's result does not depend on how its prompt was divided.  The gate projections are a
product of their own with a float32 result; gates, decays and the recurrence are float32.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from .base import Mixer, StateSpec, WeightSpec, register_mixer


@register_mixer("matrix_memory")
class MatrixMemory(Mixer):
    capturable = True
    KERNELS = ("mlstm",)
    FEW_ROWS = 16

    def __init__(self, hidden_size: int, n_heads: int, head_dim: int, value_dim: int, gate_cap: float, eps: float,
                 residual_scale: float = 1.0, init_std: float = 0.02):
        self.W, self.H, self.dk, self.dv = int(hidden_size), int(n_heads), int(head_dim), int(value_dim)
        self.cap, self.eps = float(gate_cap), float(eps)
        self.residual_scale = float(residual_scale)
        self.init_std = init_std
        if min(self.H, self.dk, self.dv) <= 0 or not self.cap > 0:
            raise ConfigError("matrix memory: sizes and the gate cap must be positive")

    def weight_specs(self):
        s = ("normal", self.init_std)
        H, W = self.H, self.W
        return {
            "q": WeightSpec((H * self.dk, W), "matrix", s),
            "k": WeightSpec((H * self.dk, W), "matrix", s),
            "v": WeightSpec((H * self.dv, W), "matrix", s),
            "g": WeightSpec((H * self.dv, W), "matrix", s),
            "o": WeightSpec((W, H * self.dv), "matrix", s),
            "norm": WeightSpec((H * self.dv,), "vector", ("one_plus_normal", 0.0)),
            "i": WeightSpec((H, W), "matrix", s),
            "i_bias": WeightSpec((H,), "vector", ("normal", 0.0)),
            "f": WeightSpec((H, W), "matrix", s),
            "f_bias": WeightSpec((H,), "vector", ("normal", 0.0)),
        }

    def cache_spec(self):
        return StateSpec((self.H * (self.dk * self.dv + self.dk + 1),), "float32")

    def bind(self, rt):
        super().bind(rt)
        prepare = getattr(rt.ops, "prepare", None)
        if prepare is not None:
            prepare(self.KERNELS)

    def step_planner(self):
        # the recurrence walks each request's rows in order: it wants the step's runs of rows
        return getattr(self.rt.ops, "plan_row_segments", None)

    def load(self, tensors):
        H = self.H
        self.w_in = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0).contiguous()
        self.oq, self.ok, self.ov, self.og = 0, H * self.dk, 2 * H * self.dk, 2 * H * self.dk + H * self.dv
        self.w_gates = torch.cat([tensors["i"], tensors["f"]], dim=0).contiguous()
        self.b_i = tensors["i_bias"].to(torch.float32).contiguous()
        self.b_f = tensors["f_bias"].to(torch.float32).contiguous()
        self.norm = tensors["norm"].to(torch.float32).contiguous()
        self.w_o = tensors["o"].contiguous()

    def forward(self, h, residual, ctx, cache, write_cache: bool = True):
        ops, dt = self.rt.ops, self.rt.dtype
        T = h.shape[0]
        qkvg = ctx.ws.get("mm_in", (T, self.w_in.shape[0]), dt)
        ops.linear(h, self.w_in, qkvg, "store")
        z = ctx.ws.get("mm_gates", (T, 2 * self.H), torch.float32)
        # 2 * heads outputs, float32: the few-row product for decode steps, the plain product otherwise
        # (the tiled tensor-core products are made for matrices with many rows)
        if T <= self.FEW_ROWS:
            ops.linear(h, self.w_gates, z, "store")
        else:
            ops.linear_plain(h, self.w_gates, z, "store")
        out = ctx.ws.get("mm_out", (T, self.H * self.dv), dt)
        ops.matrix_memory(qkvg, self.oq, self.ok, self.ov, self.og, z, self.b_i, self.b_f, self.cap, self.norm, self.eps,
                          self.residual_scale, out, ctx, cache, self.H, self.dk, self.dv)
        ops.linear(out, self.w_o, residual, "add")
