"""Small Sepirax configurations of the test-suite, model folders with random weights, and
helpers that read such a folder for the plain implementation.

The first two configurations differ in every size and option: layer order (which mixer comes first, a
mixer twice in a row), head counts (also odd ones), head sizes that differ from value sizes, a
rotated part whose first half only is rotated, YaRN scaling or none, expert counts and groups
(also no groups and a single choice), a layer without a feed-forward, the residual factor, the
embedding scale, a soft cap or none.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from zllm_b200.config import SepiraxConfig


def _latent(heads, dim, rot_dim, dims, vdim, q_rank, kv_rank, scaling):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
            "scale": (dim + rot_dim) ** -0.5, "rot": {"base": 10000.0, "dims": dims, "scaling": scaling}}


def _moe(ff, experts, top, count, keep):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


SEP_A = {
    "architecture": "Sepirax", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
    "embedding": {"scale": 4.0}, "logit_softcap": 20.0,
    "layers": [
        {"type": "latent_attention", "mlp": _moe(32, 8, 2, 4, 2),
         "mixer": _latent(4, 16, 8, 8, 24, 40, 48, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0})},
        {"type": "mlstm", "mlp": _moe(32, 8, 2, 4, 2), "mixer": {"heads": 2, "dim": 16, "vdim": 24, "gate_cap": 10.0}},
        {"type": "latent_attention", "mlp": _moe(32, 8, 2, 4, 2),
         "mixer": _latent(4, 16, 8, 8, 24, 40, 48, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0})},
        {"type": "mlstm", "mlp": _moe(32, 8, 2, 4, 2), "mixer": {"heads": 2, "dim": 16, "vdim": 24, "gate_cap": 10.0}},
    ],
}
SEP_B = {
    "architecture": "Sepirax", "vocab": 333, "width": 96, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
    "embedding": {"scale": 1.0}, "logit_softcap": None,
    "layers": [
        {"type": "mlstm", "mlp": _moe(40, 6, 1, 1, 1), "mixer": {"heads": 3, "dim": 40, "vdim": 16, "gate_cap": 6.0}},
        {"type": "latent_attention", "mlp": None, "mixer": _latent(3, 24, 16, 8, 16, 56, 72, None)},
        {"type": "latent_attention", "mlp": _moe(24, 6, 3, 3, 2), "mixer": _latent(5, 8, 16, 16, 40, 32, 40, None)},
    ],
}
# Sizes that the tensor-core kernels take (a latent of 64 with a rotated part of 16, inner sizes that are
# multiples of 32 and 64, a memory whose rows fill the registers exactly), so that those kernels also run
# inside the whole-model tests in bfloat16
SEP_C = {
    "architecture": "Sepirax", "vocab": 264, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.8,
    "embedding": {"scale": 2.0}, "logit_softcap": 25.0,
    "layers": [
        {"type": "latent_attention", "mlp": _moe(64, 8, 2, 2, 1),
         "mixer": _latent(4, 32, 16, 16, 32, 64, 64, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0})},
        {"type": "mlstm", "mlp": _moe(64, 8, 2, 2, 1), "mixer": {"heads": 2, "dim": 32, "vdim": 64, "gate_cap": 12.0}},
        {"type": "latent_attention", "mlp": None,
         "mixer": _latent(4, 32, 16, 16, 32, 64, 64, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0})},
    ],
}
# Sizes that are multiples of nothing: no vector load, no tensor-core tile and no 16-byte boundary fits, so every
# kernel's general path runs (a width of 76, a cache row of 42 numbers, 9 experts in 3 groups, 5 heads of 12 x 18)
SEP_D = {
    "architecture": "Sepirax", "vocab": 101, "width": 76, "norm": {"eps": 1e-5}, "residual_mult": 0.9,
    "embedding": {"scale": 3.0}, "logit_softcap": 15.0,
    "layers": [
        {"type": "mlstm", "mlp": _moe(22, 9, 4, 3, 2), "mixer": {"heads": 5, "dim": 12, "vdim": 18, "gate_cap": 9.0}},
        {"type": "latent_attention", "mlp": _moe(22, 9, 4, 3, 2),
         "mixer": _latent(3, 10, 6, 4, 14, 20, 36, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5})},
    ],
}
# name -> (configuration, page size, weight seed, std of matrices)
SEPIRAX = {"A": (SEP_A, 16, 11, 0.08), "B": (SEP_B, 8, 12, 0.1), "C": (SEP_C, 16, 13, 0.08), "D": (SEP_D, 16, 16, 0.15)}


def make_sepirax_dir(tmp_path, name, dtype="float32", std=None, edit=None):
    """Write the model ``name`` under ``tmp_path`` (random weights from the engine's random-weights
    mode); ``edit(tensors)`` may change tensors before they are stored.  Returns the folder."""
    from zllm_b200.weights import write_random_model
    from zllm_b200.weights.safetensors_io import open_model_files, write_safetensors

    cfg, _, seed, s = SEPIRAX[name]
    d = Path(tmp_path) / f"sepirax{name}_{dtype}{'_edited' if edit else ''}"
    if not (d / "model.safetensors").exists():
        write_random_model(d, SepiraxConfig.from_dict(cfg), seed, dtype, std=std if std is not None else s, norm_std=0.1)
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
