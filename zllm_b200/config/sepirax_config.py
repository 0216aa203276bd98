"""Typed configuration of the Sepirax decoder, read from its ``config.json``.

The file names the architecture with the key ``architecture`` and lists its layers one by
one: ``layers[i] = {"type": mixer kind, "mixer": {sizes...}, "mlp": {...} | null}``.  Every
size and constant comes from the file; a missing key is an error that names it, as for the
other architectures.  The file sets no largest position.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional, Tuple

from ..errors import ConfigError

MIXER_KINDS = ("latent_attention", "mlstm")


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} is missing key {key!r}")
    return d[key]


def _pos(d: dict, key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, found {v!r}")
    return v


@dataclass(frozen=True)
class SepiraxLayer:
    type: str
    mixer: dict
    mlp: Optional[dict]


@dataclass(frozen=True)
class SepiraxConfig:
    architecture: str
    vocab: int
    width: int
    layers: Tuple[SepiraxLayer, ...]
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    logit_softcap: Optional[float]
    extra: dict = field(default_factory=dict, compare=False)

    @staticmethod
    def from_dict(d: dict) -> "SepiraxConfig":
        layers: List[SepiraxLayer] = []
        raw_layers = _need(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, ly in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(ly, "type", where)
            if kind not in MIXER_KINDS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {MIXER_KINDS}")
            mx = _need(ly, "mixer", where)
            for k in (("heads", "dim", "vdim") + (("rot_dim", "kv_rank", "q_rank") if kind == "latent_attention" else ())):
                _pos(mx, k, where + ".mixer") if k != "rot_dim" else _need(mx, k, where + ".mixer")
            if kind == "latent_attention":
                _need(mx, "scale", where + ".mixer")
                if mx["rot_dim"]:
                    rot = _need(mx, "rot", where + ".mixer")
                    _pos(rot, "dims", where + ".mixer.rot")
                    _need(rot, "base", where + ".mixer.rot")
                    if rot.get("scaling"):
                        for k in ("factor", "original", "fast", "slow"):
                            _need(rot["scaling"], k, where + ".mixer.rot.scaling")
            else:
                _need(mx, "gate_cap", where + ".mixer")
            mlp = ly.get("mlp")
            if mlp is not None:
                kind_ff = _need(mlp, "kind", where + ".mlp")
                if kind_ff != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind {kind_ff!r} is not supported (moe)")
                _pos(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert")
                r = _need(mlp, "router", where + ".mlp")
                _pos(r, "experts", where + ".mlp.router")
                _pos(r, "top", where + ".mlp.router")
                if r.get("groups"):
                    _pos(r["groups"], "count", where + ".mlp.router.groups")
                    _pos(r["groups"], "keep", where + ".mlp.router.groups")
            layers.append(SepiraxLayer(kind, dict(mx), dict(mlp) if mlp is not None else None))
        cap = d.get("logit_softcap")
        known = {"architecture", "vocab", "width", "layers", "norm", "residual_mult", "embedding", "logit_softcap"}
        return SepiraxConfig(
            architecture=str(_need(d, "architecture", "the model")),
            vocab=_pos(d, "vocab", "the model"),
            width=_pos(d, "width", "the model"),
            layers=tuple(layers),
            norm_eps=float(_need(_need(d, "norm", "the model"), "eps", "norm")),
            residual_mult=float(_need(d, "residual_mult", "the model")),
            embedding_scale=float(_need(_need(d, "embedding", "the model"), "scale", "embedding")),
            logit_softcap=float(cap) if cap else None,
            extra={k: v for k, v in d.items() if k not in known},
        )

    def to_dict(self) -> dict:
        return {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": ly.type, "mixer": dict(ly.mixer), "mlp": dict(ly.mlp) if ly.mlp is not None else None}
                       for ly in self.layers],
            "logit_softcap": self.logit_softcap,
            "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult,
            "vocab": self.vocab,
            "width": self.width,
        }
