"""Typed configuration of the Vasonex decoder, read from its ``config.json``.

The file names the architecture with the key ``architecture`` and lists its layers one by
one: ``layers[i] = {"type": "attention", "mixer": {sizes...}, "mlp": {...} | null}``, optionally
with ``"weights_of": j``: the layer then has no tensors of its own and runs with those of layer
j (which has its own), with a cache of its own.  Every size and constant comes from the file; a
missing key is an error that names it.  The file sets no largest position.

    mixer: heads, kv_heads, dim, vdim, scale,
           rot  {dims, base, scaling {factor, low, high, original} | null} | null,
           mask {size, keep_first} | null
    mlp:   {"kind": "dense", "ff"}   or
           {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}, "shared": {"ff"} | null}
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

from ..errors import ConfigError
from .sepirax_config import _need, _pos

MIXER_KINDS = ("attention",)
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class VasonexLayer:
    type: str
    mixer: dict
    mlp: Optional[dict]
    weights_of: Optional[int] = None


def _check_mixer(mx: dict, where: str) -> None:
    for k in ("heads", "kv_heads", "dim", "vdim"):
        _pos(mx, k, where)
    if mx["heads"] % mx["kv_heads"]:
        raise ConfigError(f"config.json: {where}: {mx['heads']} heads are not a multiple of {mx['kv_heads']} kv_heads")
    _need(mx, "scale", where)
    rot = mx.get("rot")
    if rot:
        _need(rot, "base", where + ".rot")
        dims = _need(rot, "dims", where + ".rot")
        if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > mx["dim"]:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim, found {dims!r}")
        if rot.get("scaling"):
            for k in ("factor", "low", "high", "original"):
                _need(rot["scaling"], k, where + ".rot.scaling")
    mask = mx.get("mask")
    if mask:
        _pos(mask, "size", where + ".mask")
        kf = mask.get("keep_first", 0)
        if isinstance(kf, bool) or not isinstance(kf, int) or kf < 0:
            raise ConfigError(f"config.json: {where}.mask.keep_first must be a count, found {kf!r}")


def _check_mlp(mlp: dict, where: str) -> None:
    kind = _need(mlp, "kind", where)
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not one of {MLP_KINDS}")
    if kind == "dense":
        _pos(mlp, "ff", where)
        return
    _pos(_need(mlp, "expert", where), "ff", where + ".expert")
    r = _need(mlp, "router", where)
    _pos(r, "experts", where + ".router")
    _pos(r, "top", where + ".router")
    if r["top"] > r["experts"]:
        raise ConfigError(f"config.json: {where}.router: {r['top']} choices among {r['experts']} experts")
    if mlp.get("shared"):
        _pos(mlp["shared"], "ff", where + ".shared")


@dataclass(frozen=True)
class VasonexConfig:
    architecture: str
    vocab: int
    width: int
    layers: Tuple[VasonexLayer, ...]
    norm_eps: float
    extra: dict = field(default_factory=dict, compare=False)

    @staticmethod
    def from_dict(d: dict) -> "VasonexConfig":
        raw_layers = _need(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[VasonexLayer] = []
        for i, ly in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(ly, "type", where)
            if kind not in MIXER_KINDS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {MIXER_KINDS}")
            mx = _need(ly, "mixer", where)
            _check_mixer(mx, where + ".mixer")
            mlp = ly.get("mlp")
            if mlp is not None:
                _check_mlp(mlp, where + ".mlp")
            src = ly.get("weights_of")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(raw_layers) or src == i:
                    raise ConfigError(f"config.json: {where}.weights_of must name another layer, found {src!r}")
                if raw_layers[src].get("weights_of") is not None:
                    raise ConfigError(f"config.json: {where}.weights_of names layer {src}, which has no tensors of its own")
            layers.append(VasonexLayer(kind, dict(mx), dict(mlp) if mlp is not None else None, src))
        known = {"architecture", "vocab", "width", "layers", "norm"}
        return VasonexConfig(
            architecture=str(_need(d, "architecture", "the model")),
            vocab=_pos(d, "vocab", "the model"),
            width=_pos(d, "width", "the model"),
            layers=tuple(layers),
            norm_eps=float(_need(_need(d, "norm", "the model"), "eps", "norm")),
            extra={k: v for k, v in d.items() if k not in known},
        )

    def to_dict(self) -> dict:
        out_layers = []
        for ly in self.layers:
            e = {"type": ly.type, "mixer": dict(ly.mixer), "mlp": dict(ly.mlp) if ly.mlp is not None else None}
            if ly.weights_of is not None:
                e["weights_of"] = ly.weights_of
            out_layers.append(e)
        return {"architecture": self.architecture, "layers": out_layers, "norm": {"eps": self.norm_eps},
                "vocab": self.vocab, "width": self.width}
