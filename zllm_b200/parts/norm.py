"""Norms of the residual stream: RMSNorm and Dynamic Tanh.

y = x * rsqrt(mean_i(x_i^2) + eps) * w, the mean over the row, eps inside the
root, the weight applied after normalisation, no bias and no ``1 + w``
(zllm src/backend/gpu/shaders.rs:555-562; placement before attention, before the
feed-forward and before the head: quantized_llama_fork.rs:943,956,971).  Input is
the float32 residual stream; sums and the root are float32 in every path.
"""
from __future__ import annotations

import torch

from .base import Norm, WeightSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    capturable = True

    def __init__(self, size: int, eps: float):
        self.size = int(size)
        self.eps = float(eps)
        self.weight = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.size,), "vector", ("one_plus_normal", 0.0))}

    def forward(self, x, out, ctx):
        self.rt.ops.rmsnorm(x, self.weight, self.eps, out)
        return out

    def as_prologue(self):
        """(weight, eps): what a product needs to apply this norm to its own input rows."""
        return (self.weight, self.eps)

    def forward_add(self, y, residual, ctx, bias=None):
        """residual += rmsnorm(y + bias) * weight in one pass, all float32."""
        self.rt.ops.rmsnorm_add(y, bias, self.weight, self.eps, residual)


@register_norm("dynamic_tanh")
class DynamicTanh(Norm):
    """y = tanh(alpha x) * weight + bias, element by element: no mean, no variance, no epsilon.
    ``alpha`` is one learned number stored beside the weight.  It cannot ride in a product's
    prologue the way an RMS norm does (``as_prologue`` stays None): it runs as a kernel of its own
    from the float32 residual into the compute dtype."""

    capturable = True

    def __init__(self, size: int, init_alpha: float = 0.5):
        self.size = int(size)
        self.init_alpha = float(init_alpha)
        self.weight = self.bias = self.alpha = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.size,), "vector", ("one_plus_normal", 0.0)),
                "bias": WeightSpec((self.size,), "vector", ("normal", 0.0)),
                "alpha": WeightSpec((), "vector", ("constant", self.init_alpha))}

    def load(self, tensors):
        # three small tensors: kept in float32 whatever they were stored in (the norm is 32-bit arithmetic)
        self.weight = tensors["weight"].to(torch.float32).contiguous()
        self.bias = tensors["bias"].to(torch.float32).contiguous()
        self.alpha = tensors["alpha"].to(torch.float32).reshape(1).contiguous()

    def forward(self, x, out, ctx):
        self.rt.ops.dynamic_tanh(x, self.alpha, self.weight, self.bias, out)
        return out
