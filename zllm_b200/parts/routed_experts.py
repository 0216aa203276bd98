"""A mixture of experts as a feed-forward: a router chooses ``top`` of ``n_experts`` small
feed-forwards per token and sums their outputs.

Router: z = Wr h in float32.  Scores: s = softmax(z) over all experts, or s = sigmoid(z) each by
itself (``score``).  The experts form ``n_groups`` equal groups of neighbours; a group counts by
its largest score and only the experts of the ``keep_groups`` best groups can be chosen (one group
of everything: no restriction).  The ``top`` largest scores are chosen (lowest index on ties); the
weights are those scores, divided by their sum (+ 1e-20) when ``normalise`` is set.  A weight
multiplies the expert's output (``weight_on`` "output") or what the expert reads ("input").
Expert e: Wdown_e (silu(Wgate_e x) * (Wup_e x)) when ``gated``, else Wdown_e f(Wup_e x) with
f = ``activation`` (silu, gelu in its exact erf form, gelu_tanh); no biases.

A shared expert of ``shared_size`` inner entries (0: none), of the same form, is visited by every
token and added, multiplied by sigmoid(w_sg . h) when ``shared_gate`` is set (one number per token).
It rides in the same launches: its matrices are cut into pieces of ``expert_size`` inner entries
(the last one filled up with zero rows, which contribute nothing) and appended to the experts'
stacks as experts E, E+1, ...; the router kernel gives every token those choices with the gate's
value as their output weight, and the gate's vector is one more row of the router matrix.

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
    can_overwrite = True
    KERNELS = ("moe", "gemm_grouped")
    # a list, when somebody wants to know what was chosen: every call then appends (slots of the rows, their
    # positions, the chosen experts [rows, top]) as copies on the device.  Only outside captured graphs.
    record = None

    def __init__(self, hidden_size: int, expert_size: int, n_experts: int, top: int, n_groups: int = 1,
                 keep_groups: int = 1, residual_scale: float = 1.0, init_std: float = 0.02, score: str = "softmax",
                 normalise: bool = True, weight_on: str = "output", gated: bool = True, activation: str = "silu",
                 shared_size: int = 0, shared_gate: bool = False):
        self.W, self.F, self.E = int(hidden_size), int(expert_size), int(n_experts)
        self.top, self.n_groups, self.keep_groups = int(top), int(n_groups), int(keep_groups)
        self.residual_scale = float(residual_scale)
        self.init_std = init_std
        self.score, self.normalise, self.weight_on = str(score), bool(normalise), str(weight_on)
        self.gated, self.activation = bool(gated), str(activation)
        self.shared_size, self.shared_gate = int(shared_size or 0), bool(shared_gate) and bool(shared_size)
        if min(self.W, self.F, self.E, self.top, self.n_groups, self.keep_groups) <= 0 or self.shared_size < 0:
            raise ConfigError("routed experts: sizes must be positive")
        if self.E % self.n_groups or self.keep_groups > self.n_groups:
            raise ConfigError(f"routed experts: {self.E} experts in {self.n_groups} groups, {self.keep_groups} kept")
        if self.top > self.keep_groups * (self.E // self.n_groups):
            raise ConfigError(f"routed experts: {self.top} choices among {self.keep_groups} groups of "
                              f"{self.E // self.n_groups} experts")
        if self.score not in ("softmax", "sigmoid") or self.weight_on not in ("output", "input"):
            raise ConfigError(f"routed experts: score {self.score!r} / weight_on {self.weight_on!r}")
        if self.activation not in ("silu", "gelu", "gelu_tanh") or (self.gated and self.activation != "silu"):
            raise ConfigError(f"routed experts: activation {self.activation!r} (gated experts use silu)")
        self.n_shared = -(-self.shared_size // self.F)        # pieces of the shared expert, each one more choice per token

    def weight_specs(self):
        s = ("normal", self.init_std)
        out = {"router": WeightSpec((self.E, self.W), "matrix", s)}
        for e in range(self.E):
            if self.gated:
                out[f"gate.{e}"] = WeightSpec((self.F, self.W), "matrix", s)
            out[f"up.{e}"] = WeightSpec((self.F, self.W), "matrix", s)
            out[f"down.{e}"] = WeightSpec((self.W, self.F), "matrix", s)
        if self.shared_size:
            if self.gated:
                out["shared.gate"] = WeightSpec((self.shared_size, self.W), "matrix", s)
            out["shared.up"] = WeightSpec((self.shared_size, self.W), "matrix", s)
            out["shared.down"] = WeightSpec((self.W, self.shared_size), "matrix", s)
            if self.shared_gate:
                out["shared.sg"] = WeightSpec((1, self.W), "matrix", s)
        return out

    def bind(self, rt):
        super().bind(rt)
        prepare = getattr(rt.ops, "prepare", None)
        if prepare is not None:
            prepare(self.KERNELS + (("gemm_grouped_mma",) if rt.dtype == torch.bfloat16 else ()))

    def _pieces(self, m, rows: bool):
        """The shared expert's matrix ``m`` cut into ``n_shared`` pieces of F inner entries (rows of an
        up matrix, columns of a down matrix), the last filled up with zeros."""
        F, n = self.F, self.n_shared
        pad = n * F - self.shared_size
        if rows:
            if pad:
                m = torch.cat([m, torch.zeros((pad, m.shape[1]), dtype=m.dtype, device=m.device)], dim=0)
            return [m[c * F:(c + 1) * F] for c in range(n)]
        if pad:
            m = torch.cat([m, torch.zeros((m.shape[0], pad), dtype=m.dtype, device=m.device)], dim=1)
        return [m[:, c * F:(c + 1) * F] for c in range(n)]

    def load(self, tensors):
        router = [tensors["router"]] + ([tensors["shared.sg"].reshape(1, self.W)] if self.shared_gate else [])
        self.w_router = torch.cat(router, dim=0).contiguous()
        sh = bool(self.shared_size)
        self.w_gate = None
        if self.gated:
            self.w_gate = torch.stack([tensors[f"gate.{e}"] for e in range(self.E)]
                                      + (self._pieces(tensors["shared.gate"], True) if sh else [])).contiguous()
        self.w_up = torch.stack([tensors[f"up.{e}"] for e in range(self.E)]
                                + (self._pieces(tensors["shared.up"], True) if sh else [])).contiguous()
        self.w_down = torch.stack([tensors[f"down.{e}"] for e in range(self.E)]
                                  + (self._pieces(tensors["shared.down"], False) if sh else [])).contiguous()

    def forward(self, h, residual, ctx, accumulate: bool = True):
        ops = self.rt.ops
        T = h.shape[0]
        cols = self.top + self.n_shared
        idx = ctx.ws.get("moe_choice", (T, cols), torch.int32)
        wts = ctx.ws.get("moe_weight", (T, cols), torch.float32)
        ops.moe_route(h, self.w_router, self.top, self.n_groups, self.keep_groups, idx, wts, score=self.score,
                      normalise=self.normalise, n_shared=self.n_shared, shared_gate=self.shared_gate)
        if self.record is not None:
            self.record.append((ctx.row_slot.clone(), ctx.positions.clone(), idx[:, :self.top].clone()))
        ops.moe_experts(h, idx, wts, self.w_gate, self.w_up, self.w_down, residual, self.residual_scale, ctx.ws,
                        n_input_weighted=self.top if self.weight_on == "input" else 0, activation=self.activation,
                        accumulate=accumulate)
        return None
