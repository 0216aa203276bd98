"""A mixture of experts as a feed-forward: a router chooses ``top`` of ``n_experts`` small
SiLU-gated feed-forwards per token and sums their outputs with the router's weights.

Router: z = Wr h in float32, scores s = softmax(z) over all experts.  The experts form
``n_groups`` equal groups of neighbours; a group counts by its largest score and only the experts
of the ``keep_groups`` best groups can be chosen (one group of everything: no restriction).  The
``top`` largest scores are chosen; the weights are those scores divided by their sum (+ 1e-20).
Expert e: Wdown_e (silu(Wgate_e h) * (Wup_e h)), no biases.

On the device the (token, choice) pairs are sorted by expert and each expert's rows go through
its matrices in tiles of one launch: no host decision, so a step can be captured as a graph.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from .base import FeedForward, WeightSpec, register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    capturable = True
    KERNELS = ("moe", "gemm_grouped")

    def __init__(self, hidden_size: int, expert_size: int, n_experts: int, top: int, n_groups: int = 1,
                 keep_groups: int = 1, residual_scale: float = 1.0, init_std: float = 0.02):
        self.W, self.F, self.E = int(hidden_size), int(expert_size), int(n_experts)
        self.top, self.n_groups, self.keep_groups = int(top), int(n_groups), int(keep_groups)
        self.residual_scale = float(residual_scale)
        self.init_std = init_std
        if min(self.W, self.F, self.E, self.top, self.n_groups, self.keep_groups) <= 0:
            raise ConfigError("routed experts: sizes must be positive")
        if self.E % self.n_groups or self.keep_groups > self.n_groups:
            raise ConfigError(f"routed experts: {self.E} experts in {self.n_groups} groups, {self.keep_groups} kept")
        if self.top > self.keep_groups * (self.E // self.n_groups):
            raise ConfigError(f"routed experts: {self.top} choices among {self.keep_groups} groups of "
                              f"{self.E // self.n_groups} experts")

    def weight_specs(self):
        s = ("normal", self.init_std)
        out = {"router": WeightSpec((self.E, self.W), "matrix", s)}
        for e in range(self.E):
            out[f"gate.{e}"] = WeightSpec((self.F, self.W), "matrix", s)
            out[f"up.{e}"] = WeightSpec((self.F, self.W), "matrix", s)
            out[f"down.{e}"] = WeightSpec((self.W, self.F), "matrix", s)
        return out

    def bind(self, rt):
        super().bind(rt)
        prepare = getattr(rt.ops, "prepare", None)
        if prepare is not None:
            prepare(self.KERNELS + (("gemm_grouped_mma",) if rt.dtype == torch.bfloat16 else ()))

    def load(self, tensors):
        self.w_router = tensors["router"].contiguous()
        self.w_gate = torch.stack([tensors[f"gate.{e}"] for e in range(self.E)]).contiguous()
        self.w_up = torch.stack([tensors[f"up.{e}"] for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([tensors[f"down.{e}"] for e in range(self.E)]).contiguous()

    def forward(self, h, residual, ctx):
        ops = self.rt.ops
        T = h.shape[0]
        idx = ctx.ws.get("moe_choice", (T, self.top), torch.int32)
        wts = ctx.ws.get("moe_weight", (T, self.top), torch.float32)
        ops.moe_route(h, self.w_router, self.top, self.n_groups, self.keep_groups, idx, wts)
        ops.moe_experts(h, idx, wts, self.w_gate, self.w_up, self.w_down, residual, self.residual_scale, ctx.ws)
