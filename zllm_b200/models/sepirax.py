"""Sepirax: a decoder whose layers are listed one by one in its configuration, each with a
latent-attention or a matrix-memory (mLSTM) mixer and a routed mixture of experts, Dynamic Tanh
norms, a scaled embedding, a scaled residual and soft-capped logits.

    x = embed[token] * embedding.scale
    per layer:  x += m * mixer(norm1(x));  x += m * experts(norm2(x))      (m = residual_mult)
    logits = cap * tanh((head . final_norm(x)) / cap)

This file only lists parts and tensor names; the mechanisms are the registered kinds
``latent_attention``, ``matrix_memory``, ``routed_experts``, ``dynamic_tanh`` and
``rotary_on_the_fly``.  Tensor names: ``embed``, ``head``, ``final.norm[.b|.alpha]``, and per
layer i ``l<i>.norm1|norm2[.b|.alpha]``, ``l<i>.mix.<name>``, ``l<i>.mlp.router``,
``l<i>.mlp.e<j>.gate|up|down``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sepirax_config import SepiraxConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunEntry


def _norm_names(part: str, name: str) -> dict:
    return {f"{part}.weight": name, f"{part}.bias": name + ".b", f"{part}.alpha": name + ".alpha"}


def build_sepirax_spec(cfg: SepiraxConfig) -> ModelSpec:
    W = cfg.width
    norm = PartSpec("dynamic_tanh", {"size": W})
    layers = []
    for i, ly in enumerate(cfg.layers):
        p = f"l{i}."
        mx = ly.mixer
        names = _norm_names("norm1", p + "norm1")
        if ly.type == "latent_attention":
            pe = None
            if mx["rot_dim"]:
                rot = mx["rot"]
                pe = PartSpec("rotary_on_the_fly", {"dims": rot["dims"], "base": rot["base"], "scaling": rot.get("scaling") or None})
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "n_heads": mx["heads"], "head_dim": mx["dim"], "rot_dim": mx["rot_dim"],
                "value_dim": mx["vdim"], "q_rank": mx["q_rank"], "kv_rank": mx["kv_rank"], "scale": mx["scale"],
                "eps": cfg.norm_eps, "position_encoding": pe, "residual_scale": cfg.residual_mult})
            names.update({f"mixer.{k}": p + "mix." + k for k in ("dq", "uq", "dkv", "uk", "uv", "g", "o")})
            names.update({"mixer.dq_norm": p + "mix.dq.norm", "mixer.dkv_norm": p + "mix.dkv.norm"})
        else:
            mixer = PartSpec("matrix_memory", {
                "hidden_size": W, "n_heads": mx["heads"], "head_dim": mx["dim"], "value_dim": mx["vdim"],
                "gate_cap": mx["gate_cap"], "eps": cfg.norm_eps, "residual_scale": cfg.residual_mult})
            names.update({f"mixer.{k}": p + "mix." + k for k in ("q", "k", "v", "g", "o", "norm", "i", "f")})
            names.update({"mixer.i_bias": p + "mix.i.b", "mixer.f_bias": p + "mix.f.b"})
        ffn = norm2 = None
        if ly.mlp is not None:
            r = ly.mlp["router"]
            groups = r.get("groups") or {"count": 1, "keep": 1}
            ffn = PartSpec("routed_experts", {
                "hidden_size": W, "expert_size": ly.mlp["expert"]["ff"], "n_experts": r["experts"], "top": r["top"],
                "n_groups": groups["count"], "keep_groups": groups["keep"], "residual_scale": cfg.residual_mult})
            norm2 = norm
            names.update(_norm_names("norm2", p + "norm2"))
            names["ffn.router"] = p + "mlp.router"
            for e in range(r["experts"]):
                for k in ("gate", "up", "down"):
                    names[f"ffn.{k}.{e}"] = f"{p}mlp.e{e}.{k}"
        layers.append(LayerSpec(mixer, ffn, norm, norm2, "pre_norm", names))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=W,
        max_position=None,
        layers=layers,
        run_order=[RunEntry(i) for i in range(len(layers))],
        final_norm=norm,
        embedding_name="embed",
        final_norm_names={"weight": "final.norm", "bias": "final.norm.b", "alpha": "final.norm.alpha"},
        head_name="head",
        embedding_scale=cfg.embedding_scale,
        logit_softcap=cfg.logit_softcap,
    )


register_architecture("Sepirax", SepiraxConfig.from_dict, build_sepirax_spec)
