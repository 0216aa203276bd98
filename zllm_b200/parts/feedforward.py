"""SiLU-gated feed-forward (SwiGLU), dense.

x <- x + Wdown( silu(Wgate h) * (Wup h) ), silu(g) = g / (1 + exp(-g)), no
biases (zllm src/backend/candle/quantized_llama_fork.rs:394-400,956-958;
src/backend/gpu/shaders.rs:984-988).  Gate and up are stored as one matrix so a
single product serves both, as the reference's Vulkan path does
(src/backend/vulkan/mod.rs:1141-1167); rows are interleaved in groups of eight
(eight gate rows, then the eight up rows of the same outputs) so that the
product's epilogue holds a gate value and its up value in the same thread and
writes silu(gate)*up directly.  An intermediate size that is no multiple of
eight keeps the two matrices apart and uses the stand-alone SiLU-mul kernel.

With ``bias`` every projection has a bias vector: Wdown(silu(Wgate h + bg) * (Wup h + bu)) + bd.
Gate and up are then one plain stack [gate rows; up rows] whose product is followed by a
kernel that adds both biases and forms silu(gate) * up; the down bias is added to the float32
result, or handed to the caller when it asks to add it itself (an output norm does it in its pass).
"""
from __future__ import annotations

import torch

from .base import FeedForward, WeightSpec, register_feed_forward

GATE_UP_GROUP = 8


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, group: int = GATE_UP_GROUP) -> torch.Tensor:
    """[I,K],[I,K] -> [2I,K]: rows g*2*group .. : ``group`` gate rows then their ``group`` up rows."""
    I, K = gate.shape
    assert I % group == 0
    g = gate.reshape(I // group, group, K)
    u = up.reshape(I // group, group, K)
    return torch.stack([g, u], dim=1).reshape(2 * I, K).contiguous()


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, init_std: float = 0.02, bias: bool = False):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.init_std = init_std
        self.bias = bool(bias)
        self.fused = self.intermediate_size % GATE_UP_GROUP == 0 and not self.bias
        self.b_gate_up = self.b_down = None
        self.w_gate_up = None
        self.w_gate = None
        self.w_up = None
        self.w_down = None

    def weight_specs(self):
        H, I = self.hidden_size, self.intermediate_size
        s = ("normal", self.init_std)
        out = {
            "gate_proj": WeightSpec((I, H), "matrix", s),
            "up_proj": WeightSpec((I, H), "matrix", s),
            "down_proj": WeightSpec((H, I), "matrix", s),
        }
        if self.bias:
            out.update({"gate_bias": WeightSpec((I,), "vector", s), "up_bias": WeightSpec((I,), "vector", s),
                        "down_bias": WeightSpec((H,), "vector", s)})
        return out

    def load(self, tensors):
        if self.bias:
            # one stack [gate; up], padded with zero rows to a multiple of 8 (the tensor-core products' row rule)
            w = torch.cat([tensors["gate_proj"], tensors["up_proj"]], dim=0)
            pad = -w.shape[0] % 8
            if pad:
                w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
            self.w_gate_up = w.contiguous()
            self.b_gate_up = torch.cat([tensors["gate_bias"], tensors["up_bias"]]).to(torch.float32).contiguous()
            self.b_down = tensors["down_bias"].to(torch.float32).contiguous()
        elif self.fused:
            self.w_gate_up = interleave_gate_up(tensors["gate_proj"], tensors["up_proj"])
        else:
            self.w_gate = tensors["gate_proj"].contiguous()
            self.w_up = tensors["up_proj"].contiguous()
        self.w_down = tensors["down_proj"].contiguous()

    accepts_input_norm = True
    can_overwrite = True
    capturable = True

    def forward(self, h, residual, ctx, input_norm=None, accumulate: bool = True):
        """``input_norm`` as for the attention mixer: (weight, eps) when h is the float32 residual.
        ``accumulate`` False: the result is written to ``residual`` instead of added, and a down bias
        is RETURNED for the caller to add (None otherwise)."""
        ops = self.rt.ops
        T = h.shape[0]
        act = ctx.ws.get("ffn_act", (T, self.intermediate_size), self.rt.dtype)
        if self.bias:
            gu = ctx.ws.get("ffn_gate_up", (T, self.w_gate_up.shape[0]), self.rt.dtype)
            if input_norm is not None:
                ops.linear_normed(h, input_norm[0], input_norm[1], self.w_gate_up, gu, "store", ctx.ws)
            else:
                ops.linear(h, self.w_gate_up, gu, "store")
            ops.bias_silu_mul(gu, self.b_gate_up, act)
            ops.linear(act, self.w_down, residual, "add" if accumulate else "store")
            if not accumulate:
                return self.b_down
            ops.add_bias(residual, self.b_down)
            return None
        if self.fused and input_norm is not None:
            ops.linear_normed(h, input_norm[0], input_norm[1], self.w_gate_up, act, "swiglu", ctx.ws)
        elif self.fused:
            ops.linear(h, self.w_gate_up, act, "swiglu")
        else:
            if input_norm is not None:
                hn = ctx.ws.get("normed", tuple(h.shape), self.rt.dtype)
                ops.rmsnorm(h, input_norm[0], input_norm[1], hn)
                h = hn
            up = ctx.ws.get("ffn_up", (T, self.intermediate_size), self.rt.dtype)
            ops.linear(h, self.w_gate, act, "store")
            ops.linear(h, self.w_up, up, "store")
            ops.silu_mul(act, up, act)
        ops.linear(act, self.w_down, residual, "add" if accumulate else "store")
        return None
