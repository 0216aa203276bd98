"""Arrangements: the order in which a layer's norms, mixer and feed-forward act
on the residual stream.

``pre_norm`` is the Llama block: x <- x + mixer(norm1(x)); x <- x + ffn(norm2(x))
(zllm src/backend/candle/quantized_llama_fork.rs:943-958).  The residual stream
``x`` is float32; mixer and feed-forward add into it themselves so that a
product's epilogue can do the addition.

``sandwich_norm`` norms every branch on both sides: x <- x + norm1b(mixer(norm1(x)));
x <- x + norm2b(ffn(norm2(x))).  The branch writes its float32 output into a scratch array
and the output norm adds the normed rows to the residual in the same pass.
"""
from __future__ import annotations

from .base import register_arrangement


class Layer:
    """A built layer: its parts and its arrangement function."""

    def __init__(self, norm1, mixer, norm2, ffn, arrangement, norm1_post=None, norm2_post=None):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.norm1_post, self.norm2_post = norm1_post, norm2_post
        self.arrangement = arrangement

    def parts(self):
        """The layer's parts by role; a layer without a feed-forward has neither ``ffn`` nor ``norm2``;
        the output norms (``norm1b``, ``norm2b``) are there when the layer's spec names them."""
        out = {"norm1": self.norm1, "mixer": self.mixer}
        if self.norm1_post is not None:
            out["norm1b"] = self.norm1_post
        if self.ffn is not None:
            out["norm2"] = self.norm2
            out["ffn"] = self.ffn
            if self.norm2_post is not None:
                out["norm2b"] = self.norm2_post
        return out

    def run(self, x, ctx, cache, write_cache=True):
        self.arrangement(self, x, ctx, cache, write_cache)


@register_arrangement("pre_norm")
def pre_norm(layer: Layer, x, ctx, cache, write_cache):
    rt = layer.mixer.rt
    pro1 = layer.norm1.as_prologue() if layer.mixer.accepts_input_norm else None
    if pro1 is not None:
        layer.mixer.forward(x, x, ctx, cache, write_cache, input_norm=pro1)   # the norm runs inside the mixer's product
    else:
        h = ctx.ws.get("normed", tuple(x.shape), rt.dtype)
        layer.norm1.forward(x, h, ctx)
        layer.mixer.forward(h, x, ctx, cache, write_cache)
    if layer.ffn is None:
        return
    pro2 = layer.norm2.as_prologue() if layer.ffn.accepts_input_norm else None
    if pro2 is not None:
        layer.ffn.forward(x, x, ctx, input_norm=pro2)
    else:
        h = ctx.ws.get("normed", tuple(x.shape), rt.dtype)
        layer.norm2.forward(x, h, ctx)
        layer.ffn.forward(h, x, ctx)


def _branch(part, norm_in, norm_out, x, ctx, *cache_args):
    """x += norm_out(part(norm_in(x))): the branch's output goes to a float32 scratch array, which
    the output norm reads, norms and adds to the residual.  A part that cannot overwrite its
    target adds into zeros.  What the part returns (None, or a bias vector it left for the sum)
    is handed to the output norm, which adds it to the rows before it norms them."""
    rt = part.rt
    y = ctx.ws.get("branch_out", tuple(x.shape), x.dtype)
    kw = {}
    if part.can_overwrite:
        kw["accumulate"] = False
    else:
        y.zero_()
    pro = norm_in.as_prologue() if part.accepts_input_norm else None
    if pro is not None:
        left = part.forward(x, y, ctx, *cache_args, input_norm=pro, **kw)
    else:
        h = ctx.ws.get("normed", tuple(x.shape), rt.dtype)
        norm_in.forward(x, h, ctx)
        left = part.forward(h, y, ctx, *cache_args, **kw)
    norm_out.forward_add(y, x, ctx, bias=left)


@register_arrangement("sandwich_norm")
def sandwich_norm(layer: Layer, x, ctx, cache, write_cache):
    if layer.norm1_post is None or (layer.ffn is not None and layer.norm2_post is None):
        raise ValueError("the sandwich arrangement needs an output norm for every branch")
    _branch(layer.mixer, layer.norm1, layer.norm1_post, x, ctx, cache, write_cache)
    if layer.ffn is not None:
        _branch(layer.ffn, layer.norm2, layer.norm2_post, x, ctx)
