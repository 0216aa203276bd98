"""Sepirax on the CPU: the plain implementation's mechanisms against closed forms, the typed
configuration, and the engine's host side (cache pages, state slots, row segments, step
function, scheduler) driving the model with the plain torch statements of the kernels
(``ref_ops``) -- four ways of cutting a request must reproduce the plain whole-sequence logits.
"""
import math

import pytest
import torch

import plain_sepirax as PS
import traces as TR
from configs import random_prompt
from ref_ops import RefOps
from sepirax_util import SEPIRAX, SEP_A, make_sepirax_dir, read_dir
from zllm_b200 import Engine, EngineConfig, ModelRunner, SamplingParams, StepEntry
from zllm_b200.config import SepiraxConfig, architecture_of
from zllm_b200.errors import ConfigError
from zllm_b200.parts.rotary import yarn_frequencies


def cpu_runner(model_dir, name, num_blocks, max_rows=256, slots=4):
    return ModelRunner(model_dir, ops=RefOps(), engine_config=EngineConfig(
        dtype="float32", device="cpu", cuda_graphs=False, block_size=SEPIRAX[name][1], num_blocks=num_blocks,
        max_num_seqs=slots, max_num_batched_tokens=max_rows))


# ---- the plain mechanisms against closed forms --------------------------------------------------
def test_plain_route_respects_groups_and_normalises():
    z = torch.tensor([[5.0, 0.1, 0.2, 0.3, 4.0, 3.9, 0.0, 0.0, 4.5, 0.0, 0.0, 0.0]], dtype=torch.float64)
    idx, wt = PS.route(z, 3, 3, 2)              # groups {0..3}, {4..7}, {8..11}: the best two are 0 and 2
    assert sorted(idx[0].tolist()) == [0, 3, 8]  # 4.0 and 3.9 sit in the group that is struck out
    assert abs(float(wt.sum()) - 1.0) < 1e-12
    idx1, _ = PS.route(z, 3, 1, 1)               # one group: no restriction
    assert sorted(idx1[0].tolist()) == [0, 4, 8]


def test_plain_matrix_memory_first_token_and_decay():
    torch.manual_seed(0)
    W, H, dk, dv = 8, 1, 4, 3
    w = {"q": torch.randn(H * dk, W), "k": torch.randn(H * dk, W), "v": torch.randn(H * dv, W), "g": torch.zeros(H * dv, W),
         "o": torch.eye(W)[:, :H * dv].clone(), "norm": torch.ones(H * dv), "i": torch.zeros(H, W), "i.b": torch.zeros(H),
         "f": torch.zeros(H, W), "f.b": torch.full((H,), -30.0)}
    w = {"m." + k: v.double() for k, v in w.items()}
    h = torch.randn(5, W).double()
    y = PS.mlstm(h, w, "m.", {"heads": H, "dim": dk, "vdim": dv, "gate_cap": 40.0}, 1e-6)
    # a forget gate of ~e^-30 forgets everything: every token sees only itself, out ~ v (k.q) / max(|k.q|, e^-m),
    # then unit RMS and the gate sigmoid(0) = 1/2
    for t in range(5):
        k, q, v = w["m.k"] @ h[t], (w["m.q"] @ h[t]) * dk ** -0.5, w["m.v"] @ h[t]
        raw = v * (k @ q) / (max(abs(float(k @ q)), 1.0) + 1e-6)
        want = raw / torch.sqrt((raw * raw).mean() + 1e-6) * 0.5
        assert torch.allclose(y[t, :dv], want, atol=1e-6), t


def test_yarn_frequencies_match_the_plain_statement():
    for dims, base, sc in ((8, 10000.0, (8.0, 64, 16.0, 1.0)), (16, 50000.0, (4.0, 2048, 32.0, 1.0)), (6, 100.0, (2.0, 16, 4.0, 0.5))):
        f, mag = yarn_frequencies(dims, base, *sc)
        pf, pmag = PS.yarn_frequencies(dims, base, *sc)
        assert torch.allclose(f.double(), torch.tensor(pf, dtype=torch.float64), rtol=1e-6)
        assert abs(mag - pmag) < 1e-12 and abs(mag - (0.1 * math.log(sc[0]) + 1.0)) < 1e-12
    # fast pairs keep their frequency, the slowest are divided by the factor
    f, _ = yarn_frequencies(16, 10000.0, 8.0, 64, 16.0, 1.0)
    assert abs(float(f[0]) - 1.0) < 1e-7 and abs(float(f[7]) - 10000.0 ** (-14 / 16) / 8.0) < 1e-9


# ---- configuration ------------------------------------------------------------------------------
def test_configuration_is_read_and_round_trips():
    cfg = SepiraxConfig.from_dict(SEP_A)
    assert SepiraxConfig.from_dict(cfg.to_dict()) == cfg
    assert architecture_of(SEP_A).name == "Sepirax"
    assert [ly.type for ly in cfg.layers] == ["latent_attention", "mlstm", "latent_attention", "mlstm"]
    bad = {k: v for k, v in SEP_A.items() if k != "residual_mult"}
    with pytest.raises(ConfigError, match="residual_mult"):
        SepiraxConfig.from_dict(bad)
    bad = dict(SEP_A, layers=[dict(SEP_A["layers"][0], type="conv")])
    with pytest.raises(ConfigError, match="conv"):
        SepiraxConfig.from_dict(bad)


# ---- the engine's host side with the plain statements of the kernels -----------------------------
@pytest.mark.parametrize("name", ["A", "B"])
def test_four_ways_of_cutting_agree_with_plain(tmp_path, name):
    d = make_sepirax_dir(tmp_path, name)
    cfg, w = read_dir(d)
    V = cfg["vocab"]
    reqs = [(f"r{i}", random_prompt(V, n, 20 + i)) for i, n in enumerate((5, 41, 33, 58, 1, 17))]
    ref = {rid: PS.forward(cfg, w, toks).float() for rid, toks in reqs}
    max_tokens = 192
    steps = (TR.family_whole(reqs, "w.") + TR.family_tail(reqs, 12, "t.") + TR.family_portions(reqs, prefix="p.")
             + TR.family_mixed(reqs, max_tokens, 4, 1, "m."))
    assert TR.live_tokens_needed(steps) <= max_tokens
    runner = cpu_runner(d, name, max_tokens // SEPIRAX[name][1])
    got = TR.replay_inprocess(runner, steps)
    for prefix in ("w.", "t.", "p.", "m."):
        TR.compare(got, ref, reqs, prefix, 3e-4, 0.0, f"sepirax {name} {prefix}")
    assert all(f == max_tokens // SEPIRAX[name][1] for f in runner.cache.free_pages())
    assert len(runner.cache.free_slots) == 4


def test_a_slot_used_again_starts_from_an_empty_state(tmp_path):
    d = make_sepirax_dir(tmp_path, "A")
    cfg, w = read_dir(d)
    r = cpu_runner(d, "A", 8, slots=1)
    a, b = random_prompt(cfg["vocab"], 30, 1), random_prompt(cfg["vocab"], 9, 2)
    s = r.admit()
    r.step([StepEntry(s, a, ())])
    r.release(s)
    s2 = r.admit()
    assert s2 == s                                   # the same slot, and pages 0.. again
    got = r.step([StepEntry(s2, b, tuple(range(len(b))))]).clone()
    assert float((got - PS.forward(cfg, w, b).float()).abs().max()) < 3e-4


def test_greedy_generation_through_the_scheduler(tmp_path):
    d = make_sepirax_dir(tmp_path, "B", std=0.2)
    cfg, w = read_dir(d)
    prompts = [random_prompt(cfg["vocab"], n, 40 + n) for n in (3, 19, 8)]
    eng = Engine(str(d), ops=RefOps(), dtype="float32", device="cpu", cuda_graphs=False, block_size=8, num_blocks=12,
                 max_num_seqs=2, max_num_batched_tokens=16)
    got = eng.generate(prompts, SamplingParams.greedy(max_tokens=6))
    for p, o in zip(prompts, got):
        toks = list(p)
        for t in o:
            lg = PS.forward(cfg, w, toks)[-1]
            assert t == int(lg.argmax()), (p, o)
            toks.append(t)
