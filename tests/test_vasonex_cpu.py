"""Vasonex on the CPU: the plain implementation's mechanisms against closed forms, the typed
configuration, the cache manager's window that keeps the first pages, and the engine's host side
(cache pages, step function, scheduler) driving the model with the plain torch statements of the
kernels (``ref_ops``): four ways of cutting a request must reproduce the plain whole-sequence logits.
"""
import math

import pytest
import torch

import plain_vasonex as PV
import traces as TR
from configs import random_prompt
from ref_ops import RefOps
from vasonex_util import VASONEX, VAS_A, VAS_B, make_vasonex_dir, read_dir
from zllm_b200 import Engine, EngineConfig, ModelRunner, SamplingParams, StepEntry
from zllm_b200.cache import CacheManager
from zllm_b200.config import VasonexConfig, architecture_of
from zllm_b200.errors import ConfigError
from zllm_b200.parts import KVCacheSpec
from zllm_b200.parts.rotary import stretched_frequencies


def cpu_runner(model_dir, name, num_blocks, max_rows=256, slots=4):
    return ModelRunner(model_dir, ops=RefOps(), engine_config=EngineConfig(
        dtype="float32", device="cpu", cuda_graphs=False, block_size=VASONEX[name][1], num_blocks=num_blocks,
        max_num_seqs=slots, max_num_batched_tokens=max_rows))


# ---- the plain mechanisms against closed forms --------------------------------------------------
def test_plain_mask_keeps_the_first_positions_and_the_window():
    see = PV.visible(12, 4, 2)
    assert see[11].nonzero().flatten().tolist() == [0, 1, 8, 9, 10, 11]      # two kept, four in the window
    assert see[3].nonzero().flatten().tolist() == [0, 1, 2, 3]
    assert see[5].nonzero().flatten().tolist() == [0, 1, 2, 3, 4, 5]          # 2 is the oldest of the window, 0 and 1 are kept
    assert see[6].nonzero().flatten().tolist() == [0, 1, 3, 4, 5, 6]          # 2 has just fallen out
    assert PV.visible(5, None, 0).tolist() == torch.tril(torch.ones(5, 5, dtype=torch.bool)).tolist()
    assert PV.visible(6, 2, 0)[5].nonzero().flatten().tolist() == [4, 5]


def test_plain_rotation_turns_neighbours_and_leaves_the_rest():
    x = torch.arange(1.0, 13.0, dtype=torch.float64).reshape(1, 2, 6).repeat(3, 1, 1)
    f = [0.5, 0.25]
    y = PV.rotate_neighbour_pairs(x, torch.tensor([0, 1, 7]), f, 4)
    assert torch.equal(y[0], x[0])                                             # position 0: nothing turns
    assert torch.equal(y[..., 4:], x[..., 4:])                                 # entries beyond dims pass unchanged
    a = 7 * 0.25
    assert abs(float(y[2, 0, 2]) - (3 * math.cos(a) - 4 * math.sin(a))) < 1e-12
    assert abs(float(y[2, 0, 3]) - (4 * math.cos(a) + 3 * math.sin(a))) < 1e-12
    # a rotation keeps the length of every pair
    assert torch.allclose((y[..., :4] ** 2).reshape(3, 2, 2, 2).sum(-1), (x[..., :4] ** 2).reshape(3, 2, 2, 2).sum(-1))


def test_stretched_frequencies():
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    f = PV.stretched_frequencies(16, 10000.0, sc)
    g = [10000.0 ** (-2.0 * i / 16) for i in range(8)]
    assert f[0] == g[0]                                                         # wavelength 6.3 < 64 / 4: kept
    assert abs(f[7] - g[7] / 8.0) < 1e-15                                       # wavelength 19,869 > 64: slowed down
    mid = [i for i in range(8) if 16 <= 2 * math.pi / g[i] <= 64]
    assert mid and all(g[i] / 8.0 < f[i] < g[i] for i in mid)                   # blended in between
    assert PV.stretched_frequencies(8, 100.0, None) == [100.0 ** (-2.0 * i / 8) for i in range(4)]
    for dims, base, s in ((16, 10000.0, sc), (8, 500.0, {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 16}),
                          (10, 1000.0, {"factor": 3.0, "low": 0.5, "high": 4.0, "original": 32})):
        ours = stretched_frequencies(dims, base, s["factor"], s["original"], s["low"], s["high"])
        assert torch.allclose(ours.double(), torch.tensor(PV.stretched_frequencies(dims, base, s), dtype=torch.float64), rtol=1e-6)


def test_plain_mixture_weights_the_input_and_gates_the_shared_expert():
    torch.manual_seed(0)
    W, F = 6, 4
    w = {"m.router": torch.tensor([[9.0, 0, 0, 0, 0, 0], [0.0, 0, 0, 0, 0, 0], [-9.0, 0, 0, 0, 0, 0]], dtype=torch.float64)}
    for e in range(3):
        w[f"m.e{e}.up"], w[f"m.e{e}.down"] = torch.randn(F, W).double(), torch.randn(W, F).double()
    w["m.shared.up"], w["m.shared.down"] = torch.randn(5, W).double(), torch.randn(W, 5).double()
    w["m.shared.sg"] = torch.zeros(1, W, dtype=torch.float64)
    h = torch.randn(2, W).double()
    h[0, 0], h[1, 0] = 1.0, -1.0                           # token 0 prefers expert 0, token 1 expert 2
    mlp = {"router": {"experts": 3, "top": 1}, "shared": {"ff": 5}}
    y = PV.mixture(h, w, "m.", mlp)
    s = 1.0 / (1.0 + math.exp(-9.0))
    for t, e in ((0, 0), (1, 2)):
        want = PV.gelu((s * h[t]) @ w[f"m.e{e}.up"].T) @ w[f"m.e{e}.down"].T \
            + 0.5 * (PV.gelu(h[t] @ w["m.shared.up"].T) @ w["m.shared.down"].T)
        assert torch.allclose(y[t], want, atol=1e-12)
    assert abs(float(PV.gelu(torch.tensor(1.0, dtype=torch.float64))) - 0.5 * (1 + math.erf(2 ** -0.5))) < 1e-15


# ---- configuration ------------------------------------------------------------------------------
def test_configuration_is_read_and_round_trips():
    cfg = VasonexConfig.from_dict(VAS_A)
    assert VasonexConfig.from_dict(cfg.to_dict()) == cfg
    arch = architecture_of(VAS_A)
    assert arch.name == "Vasonex"
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 2 and [e.layer for e in spec.run_order] == [0, 1, 0, 1]    # borrowed tensors: run entries
    spec_b = arch.build_spec(VasonexConfig.from_dict(VAS_B))
    assert [e.layer for e in spec_b.run_order] == [0, 1, 2, 0] and spec_b.layers[1].ffn is None
    with pytest.raises(ConfigError, match="vdim"):
        VasonexConfig.from_dict(dict(VAS_A, layers=[dict(VAS_A["layers"][0], mixer={k: v for k, v in VAS_A["layers"][0]["mixer"].items() if k != "vdim"})]))
    with pytest.raises(ConfigError, match="conv"):
        VasonexConfig.from_dict(dict(VAS_A, layers=[dict(VAS_A["layers"][0], type="conv")]))
    with pytest.raises(ConfigError, match="weights_of"):
        VasonexConfig.from_dict(dict(VAS_A, layers=VAS_A["layers"][:2] + [dict(VAS_A["layers"][2], weights_of=2)]))
    with pytest.raises(ConfigError, match="weights_of"):       # the lender must have tensors of its own
        VasonexConfig.from_dict(dict(VAS_A, layers=VAS_A["layers"][:3] + [dict(VAS_A["layers"][3], weights_of=2)]))


# ---- the cache: a window that keeps the first pages ---------------------------------------------
def test_window_gives_pages_back_but_keeps_the_first_ones():
    cm = CacheManager([(KVCacheSpec(2, 8, window=10, value_dim=12, keep_first=5), None)], 4, 12, 2, 64, torch.float32, "cpu")
    v = cm.view(0)
    assert tuple(v.k_pages.shape) == (12, 2, 4, 8) and tuple(v.v_pages.shape) == (12, 2, 4, 12)
    s = cm.admit()
    n = 0
    for step in (7, 1, 1, 9, 2, 1, 1, 1, 6):
        assert cm.ensure(s, n + step)
        n += step
        cm.advance(s, n)
        cm.check_integrity()
        g = cm.groups[0]
        held = [b for b in range(g.max_blocks) if g.table[s, b] >= 0]
        first_needed = max(0, n - 10 + 1) // 4
        assert held == sorted(set([0, 1]) | set(range(first_needed, -(-n // 4)))), (n, held)
    assert cm.free_pages() == [12 - len(held)]
    cm.free_slot(s)
    cm.check_integrity()
    assert cm.free_pages() == [12]
    # a second request gets the pages again, the kept ones included
    s2 = cm.admit()
    assert cm.ensure(s2, 30)
    cm.advance(s2, 30)
    cm.check_integrity()
    cm.truncate(s2, 0)
    assert cm.free_pages() == [12]


# ---- the engine's host side with the plain statements of the kernels -----------------------------
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_four_ways_of_cutting_agree_with_plain(tmp_path, name):
    d = make_vasonex_dir(tmp_path, name)
    cfg, w = read_dir(d)
    V = cfg["vocab"]
    reqs = [(f"r{i}", random_prompt(V, n, 20 + i)) for i, n in enumerate((5, 41, 33, 58, 1, 17))]
    ref = {rid: PV.forward(toks, cfg, w).float() for rid, toks in reqs}
    max_tokens = 192
    steps = (TR.family_whole(reqs, "w.") + TR.family_tail(reqs, 12, "t.") + TR.family_portions(reqs, prefix="p.")
             + TR.family_mixed(reqs, max_tokens, 4, 1, "m."))
    assert TR.live_tokens_needed(steps) <= max_tokens
    bs = VASONEX[name][1]
    runner = cpu_runner(d, name, max_tokens // bs)
    got = TR.replay_inprocess(runner, steps)
    for prefix in ("w.", "t.", "p.", "m."):
        TR.compare(got, ref, reqs, prefix, 3e-4, 0.0, f"vasonex {name} {prefix}")
    assert all(f == max_tokens // bs for f in runner.cache.free_pages())
    assert len(runner.cache.free_slots) == 4
    runner.cache.check_integrity()


def test_layers_that_borrow_tensors_have_caches_of_their_own(tmp_path):
    d = make_vasonex_dir(tmp_path, "A")
    cfg, w = read_dir(d)
    r = cpu_runner(d, "A", 8)
    assert len(r.model.layers) == 2 and len(r.spec.run_order) == 4
    views = [r.cache.view(i) for i in range(4)]
    assert len({v.k_pages.data_ptr() for v in views}) == 4
    toks = random_prompt(cfg["vocab"], 40, 3)
    _, streams = PV.forward(toks, cfg, w, want_layers=True)
    assert streams.shape[0] == 4 and float((streams[2] - streams[0]).abs().max()) > 1e-3


def test_greedy_generation_through_the_scheduler(tmp_path):
    d = make_vasonex_dir(tmp_path, "B", std=0.2)
    cfg, w = read_dir(d)
    prompts = [random_prompt(cfg["vocab"], n, 40 + n) for n in (3, 19, 8)]
    eng = Engine(str(d), ops=RefOps(), dtype="float32", device="cpu", cuda_graphs=False, block_size=8, num_blocks=12,
                 max_num_seqs=2, max_num_batched_tokens=16)
    got = eng.generate(prompts, SamplingParams.greedy(max_tokens=6))
    for p, o in zip(prompts, got):
        toks = list(p)
        for t in o:
            lg = PV.forward(toks, cfg, w)[-1]
            assert t == int(lg.argmax()), (p, o)
            toks.append(t)
