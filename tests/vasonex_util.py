"""Small Vasonex configurations of the test-suite, model folders with random weights, and
helpers that read such a folder for the plain implementation.

The configurations differ in every size and option: head counts (kv heads equal to the heads, fewer,
one), key and value sizes (larger, smaller, equal), rotated entries (a part of the head, all of it,
none), stretched frequencies or plain ones, windows (shorter and longer than the kept first
positions, kept positions of 0, no mask at all), dense feed-forwards whose size is no multiple of
eight, experts with one choice and several, a shared expert smaller or larger than the experts (cut
into pieces, the last one filled up) or none, a layer without feed-forward, layers that borrow
another layer's tensors, page sizes of 16, 8 and 4.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from zllm_b200.config import VasonexConfig


def _mixer(heads, kv, dim, vdim, rot, mask, scale=None):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": rot, "mask": mask,
            "scale": scale if scale is not None else dim ** -0.5}


def _moe(ff, experts, top, shared):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top},
            "shared": {"ff": shared} if shared else None}


_MA = _mixer(4, 2, 16, 24, {"dims": 8, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}},
             {"size": 24, "keep_first": 5}, 0.3)
VAS_A = {
    "architecture": "Vasonex", "vocab": 211, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _MA, "mlp": {"kind": "dense", "ff": 48}},
        {"type": "attention", "mixer": _MA, "mlp": _moe(32, 6, 2, 40)},
        {"type": "attention", "mixer": _MA, "mlp": {"kind": "dense", "ff": 48}, "weights_of": 0},
        {"type": "attention", "mixer": _MA, "mlp": _moe(32, 6, 2, 40), "weights_of": 1},
    ],
}
VAS_B = {
    "architecture": "Vasonex", "vocab": 160, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _mixer(3, 3, 32, 16, {"dims": 32, "base": 500.0, "scaling": None}, {"size": 40, "keep_first": 0}),
         "mlp": _moe(24, 5, 1, None)},
        {"type": "attention", "mixer": _mixer(6, 1, 16, 16, None, None), "mlp": None},
        {"type": "attention", "mixer": _mixer(3, 3, 24, 40, {"dims": 8, "base": 500.0, "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 16}},
                                              {"size": 7, "keep_first": 9}, 0.25),
         "mlp": {"kind": "dense", "ff": 37}},
        {"type": "attention", "mixer": _mixer(3, 3, 32, 16, {"dims": 32, "base": 500.0, "scaling": None}, {"size": 40, "keep_first": 0}),
         "mlp": _moe(24, 5, 1, None), "weights_of": 0},
    ],
}
# sizes that the tensor-core kernels take (head sizes and inner sizes that are multiples of 32 and 64)
_MC = _mixer(4, 2, 64, 32, {"dims": 32, "base": 100000.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256}},
             {"size": 64, "keep_first": 16})
VAS_C = {
    "architecture": "Vasonex", "vocab": 264, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _MC, "mlp": _moe(64, 8, 2, 128)},
        {"type": "attention", "mixer": _MC, "mlp": {"kind": "dense", "ff": 192}},
        {"type": "attention", "mixer": _MC, "mlp": _moe(64, 8, 2, 128), "weights_of": 0},
    ],
}
# sizes that are multiples of nothing: every kernel's general path
VAS_D = {
    "architecture": "Vasonex", "vocab": 101, "width": 76, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _mixer(5, 5, 12, 18, {"dims": 6, "base": 50.0, "scaling": None}, {"size": 13, "keep_first": 3}, 0.4),
         "mlp": _moe(22, 7, 3, 30)},
        {"type": "attention", "mixer": _mixer(6, 2, 10, 6, {"dims": 10, "base": 1000.0, "scaling": {"factor": 3.0, "low": 0.5, "high": 4.0, "original": 32}},
                                              {"size": 30, "keep_first": 1}),
         "mlp": {"kind": "dense", "ff": 23}},
    ],
}
# name -> (configuration, page size, weight seed, std of matrices)
VASONEX = {"A": (VAS_A, 16, 21, 0.1), "B": (VAS_B, 8, 22, 0.1), "C": (VAS_C, 16, 23, 0.08), "D": (VAS_D, 4, 24, 0.15)}


def make_vasonex_dir(tmp_path, name, dtype="float32", std=None, edit=None):
    """Write the model ``name`` under ``tmp_path`` (random weights from the engine's random-weights
    mode); ``edit(tensors)`` may change tensors before they are stored.  Returns the folder."""
    from zllm_b200.weights import write_random_model
    from zllm_b200.weights.safetensors_io import open_model_files, write_safetensors

    cfg, _, seed, s = VASONEX[name]
    d = Path(tmp_path) / f"vasonex{name}_{dtype}{'_edited' if edit else ''}"
    if not (d / "model.safetensors").exists():
        write_random_model(d, VasonexConfig.from_dict(cfg), seed, dtype, std=std if std is not None else s, norm_std=0.1)
        if edit is not None:
            where = open_model_files(d)
            tensors = {n: f.tensor(n).clone() for n, f in where.items()}
            for f in {id(f): f for f in where.values()}.values():
                f.close()
            edit(tensors)
            write_safetensors(d / "model.safetensors", tensors, {"format": "pt"})
    return d


def read_dir(model_dir, dtype=torch.float64):
    """(raw configuration, {tensor name: tensor in ``dtype``}) of a model folder."""
    from zllm_b200.weights.safetensors_io import open_model_files

    cfg = json.loads((Path(model_dir) / "config.json").read_text())
    where = open_model_files(model_dir)
    w = {n: f.tensor(n).to(dtype) for n, f in where.items()}
    for f in {id(f): f for f in where.values()}.values():
        f.close()
    return cfg, w
