"""Vasonex: a decoder whose layers are listed one by one in its configuration, each a sandwich of
RMS norms around an attention mixer and around a feed-forward,

    x = embed[token]
    per layer:  x += norm1b(mixer(norm1(x)));  x += norm2b(ff(norm2(x)))
    logits = head . final_norm(x)

The mixer is grouped-query attention with value heads of a size of their own, a rotation of the
first entries of every head (neighbour pairs, long waves stretched), a sliding window that keeps
the first positions, and a sigmoid gate per head; the feed-forward is a SiLU-gated one with
biases, a mixture of experts (sigmoid scores, the weight on the expert's input, exact GELU, a
shared expert behind a gate of its own), or missing.  A layer may run with another layer's
tensors (``weights_of``): it is then one more entry of the run order that names that layer, with
a cache of its own.

This file only lists parts and tensor names; the mechanisms are the registered kinds
``window_attention``, ``swiglu``, ``routed_experts``, ``rmsnorm``, ``rotary_on_the_fly`` and the
arrangement ``sandwich_norm``.  Tensor names: ``embed``, ``head``, ``final.norm`` and per layer i
with tensors of its own ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.q|k|v|g|o``,
``l<i>.mlp.gate|up|down[.b]`` or ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.up|down``,
``l<i>.mlp.shared.up|down|sg``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.vasonex_config import VasonexConfig
from ..errors import ConfigError
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunEntry


def _layer_spec(cfg: VasonexConfig, i: int) -> LayerSpec:
    ly = cfg.layers[i]
    W, p, mx = cfg.width, f"l{i}.", ly.mixer
    norm = PartSpec("rmsnorm", {"size": W, "eps": cfg.norm_eps})
    rot, mask = mx.get("rot"), mx.get("mask")
    pe = None
    if rot and rot["dims"]:
        pe = PartSpec("rotary_on_the_fly", {"dims": rot["dims"], "base": rot["base"], "scaling": rot.get("scaling") or None,
                                            "interleaved": True})
    mixer = PartSpec("window_attention", {
        "hidden_size": W, "n_heads": mx["heads"], "n_kv_heads": mx["kv_heads"], "head_dim": mx["dim"], "value_dim": mx["vdim"],
        "position_encoding": pe, "window": mask["size"] if mask else None, "keep_first": mask.get("keep_first", 0) if mask else 0,
        "scale": mx["scale"], "head_gate": True})
    names = {"norm1.weight": p + "norm1", "norm1b.weight": p + "norm1b"}
    names.update({f"mixer.{k}": p + "mix." + k for k in ("q", "k", "v", "g", "o")})
    ffn = norm2 = norm2b = None
    if ly.mlp is not None:
        norm2 = norm2b = norm
        names.update({"norm2.weight": p + "norm2", "norm2b.weight": p + "norm2b"})
        if ly.mlp["kind"] == "dense":
            ffn = PartSpec("swiglu", {"hidden_size": W, "intermediate_size": ly.mlp["ff"], "bias": True})
            for k in ("gate", "up", "down"):
                names[f"ffn.{k}_proj"] = f"{p}mlp.{k}"
                names[f"ffn.{k}_bias"] = f"{p}mlp.{k}.b"
        else:
            r, shared = ly.mlp["router"], ly.mlp.get("shared")
            ffn = PartSpec("routed_experts", {
                "hidden_size": W, "expert_size": ly.mlp["expert"]["ff"], "n_experts": r["experts"], "top": r["top"],
                "score": "sigmoid", "normalise": False, "weight_on": "input", "gated": False, "activation": "gelu",
                "shared_size": shared["ff"] if shared else 0, "shared_gate": bool(shared)})
            names["ffn.router"] = p + "mlp.router"
            for e in range(r["experts"]):
                for k in ("up", "down"):
                    names[f"ffn.{k}.{e}"] = f"{p}mlp.e{e}.{k}"
            if shared:
                names.update({f"ffn.shared.{k}": f"{p}mlp.shared.{k}" for k in ("up", "down", "sg")})
    return LayerSpec(mixer, ffn, norm, norm2, "sandwich_norm", names, norm1_post=norm, norm2_post=norm2b)


def build_vasonex_spec(cfg: VasonexConfig) -> ModelSpec:
    # layers with tensors of their own become the model's layers; every configured layer is an entry of the
    # run order that names one of them (its own, or the one whose tensors it borrows)
    own = [i for i, ly in enumerate(cfg.layers) if ly.weights_of is None]
    index = {i: n for n, i in enumerate(own)}
    layers = [_layer_spec(cfg, i) for i in own]
    run = []
    for i, ly in enumerate(cfg.layers):
        src = i if ly.weights_of is None else ly.weights_of
        if src not in index:
            raise ConfigError(f"layers[{i}].weights_of names layer {src}, which has no tensors of its own")
        a, b = cfg.layers[src], ly
        if ly.weights_of is not None and (a.mixer != b.mixer or a.mlp != b.mlp or a.type != b.type):
            raise ConfigError(f"layers[{i}] borrows the tensors of layer {src} but its sizes differ")
        run.append(RunEntry(index[src]))
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps})
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_position=None,
        layers=layers,
        run_order=run,
        final_norm=norm,
        embedding_name="embed",
        final_norm_names={"weight": "final.norm"},
        head_name="head",
    )


register_architecture("Vasonex", VasonexConfig.from_dict, build_vasonex_spec)
