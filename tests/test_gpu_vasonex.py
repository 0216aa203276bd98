"""Vasonex on the GPU: every new kernel alone against its plain torch statement (``ref_ops``),
with inputs made so that one key stands out where a fault would hide among random ones, then the
whole model through the engine's step function, cache and scheduler against the plain
whole-sequence implementation (``plain_vasonex``), cut in every way, in both precisions.
"""
import copy

import pytest
import torch

import plain_vasonex as PV
import traces as TR
from configs import random_prompt
from gpu_util import DEV, check_greedy_stream
from ref_ops import RefOps
from vasonex_util import VASONEX, make_vasonex_dir, read_dir

pytestmark = pytest.mark.gpu

# bounds of the bfloat16 comparisons, as a fraction of the request's largest |logit|, per test model
BF16_OF_SCALE = {"A": 0.03, "B": 0.03, "C": 0.03, "D": 0.04}
# A router logit that lies closer to the next one than this fraction of the token's largest is a close call:
# an implementation with other roundings (bfloat16) may send the token to the other expert, and its logits (and,
# through attention, those of later positions) are then another function's.  The comparisons therefore follow the
# engine through its choices: the mixture part records what it chose for every row, the plain implementation is run
# with those choices, and wherever the plain scores were NOT a close call the engine must have chosen as the plain
# implementation would.
CLOSE_CALL = 0.01
# the bfloat16 engine's router reads a residual stream that has drifted by a percent or so after a few layers:
# there a margin under 5 % counts as a close call
CLOSE_CALL_BF16 = 0.05


class _Choices:
    """Collects the experts the engine chose, per (request, layer run), while a trace is replayed."""

    def __init__(self, runner, cfg):
        self.runs = [i for i, ly in enumerate(cfg["layers"]) if ly.get("mlp") and ly["mlp"]["kind"] == "moe"]
        self.record = []
        self.seen = {}                        # (request, run) -> {position: [experts]}
        for layer in runner.model.layers:
            if layer.ffn is not None and hasattr(layer.ffn, "record"):
                layer.ffn.record = self.record

    def after_step(self, step, first):
        assert len(self.record) == len(self.runs), "one record per layer run with a mixture"
        for run, (_, _, idx) in zip(self.runs, self.record):
            idx, r = idx.cpu(), 0
            for e in step["entries"]:
                for k in range(len(e["tokens"])):
                    self.seen.setdefault((e["id"], run), {})[first[e["id"]] + k] = idx[r].tolist()
                    r += 1
        self.record.clear()

    def forced(self, rid, n):
        return {run: torch.tensor([self.seen[(rid, run)][p] for p in range(n)]) for run in self.runs}


_FREE = {}                  # (model folder, request) -> (plain logits with the plain choices, router margins)


def _compare_following_the_choices(got, choices, cfg, w, reqs, prefix, atol, bound_of_scale, what, key=None, close=CLOSE_CALL):
    from gpu_util import observe
    for rid, toks in reqs:
        forced = choices.forced(prefix + rid, len(toks)) if choices.runs else None
        ref64 = PV.forward(toks, cfg, w, forced=forced)
        ref = ref64.float()
        scale = float(ref.abs().max())
        for p in range(len(toks)):
            err = float((got[(prefix + rid, p)] - ref[p]).abs().max())
            if bound_of_scale > 0:
                observe(what, err, scale, bound_of_scale)
            assert err <= atol + bound_of_scale * scale, (f"{what}: request {rid} position {p} (first wrong place): "
                                                          f"max abs error {err:.3e} > {atol + bound_of_scale * scale:.3e}")
        if choices.runs:
            # up to the request's first close call the engine chose what the plain implementation chooses by itself
            if (key, rid) not in _FREE:
                _FREE[(key, rid)] = PV.forward(toks, cfg, w, want_margins=True)
            free, margins = _FREE[(key, rid)]
            near = (margins < close).nonzero().flatten()
            first = int(near[0]) if len(near) else len(toks)
            assert first == 0 or float((ref64[:first] - free[:first]).abs().max()) < 1e-9, \
                f"{what}: request {rid}: the engine chose other experts than the plain implementation without a close call"


@pytest.fixture(scope="module")
def ops():
    from zllm_b200.kernels.ops import CudaOps
    o = CudaOps(DEV)
    o.configure(torch.bfloat16)
    return o


def _ctx(cm, entries, max_rows=1024, as_decode=False):
    """A step description for entries [(slot, n_tokens)] appended at each slot's cached length."""
    from zllm_b200.engine.batch import StepBuffers, StepEntry, Workspace, fill_step, make_context
    from zllm_b200.kernels.ops import CudaOps
    buf = StepBuffers(max_rows, max_rows, DEV)
    ents, starts = [], []
    for slot, n in entries:
        start = cm.length[slot]
        assert cm.ensure(slot, start + n)
        ents.append(StepEntry(slot, [0] * n, ()))
        starts.append(start)
    T, R, nd, plans, mc = fill_step(buf, ents, starts, planners=() if as_decode else (CudaOps.plan_query_tiles,))
    buf.upload()
    cm.sync_tables()
    ctx = make_context(buf, T, R, nd, plans, mc, Workspace(max_rows, DEV), None if as_decode else ents, starts)
    return ctx, [(slot, s + n) for (slot, n), s in zip(entries, starts)]


def _cpu(ctx):
    c = copy.copy(ctx)
    for k in ("token_ids", "positions", "row_slot", "want_rows", "decode_rows"):
        setattr(c, k, getattr(ctx, k).cpu())
    c.aux = {k: v.cpu() for k, v in ctx.aux.items()}
    return c


class _CpuCache:
    def __init__(self, view):
        self.k_pages, self.v_pages = view.k_pages.float().cpu(), view.v_pages.float().cpu()
        self.block_table, self.block_size, self.window = view.block_table.cpu(), view.block_size, view.window


def _close(got, want, dtype, what, scale=None):
    got, want = got.float().cpu(), want.float()
    tol = (3e-5 if dtype == torch.float32 else 1.2e-2) * float(scale if scale is not None else want.abs().max().clamp(min=1e-6))
    err = float((got - want).abs().max())
    assert err <= tol, f"{what}: max abs error {err:.3e} > {tol:.3e}"


# ---- small kernels --------------------------------------------------------------------------------
@pytest.mark.parametrize("H", [64, 76, 1536])
def test_output_norm_added_to_the_residual_and_biases(ops, H):
    g = torch.Generator().manual_seed(H)
    T = 37
    y, x = torch.randn(T, H, generator=g) * 3, torch.randn(T, H, generator=g)
    b, w = torch.randn(H, generator=g), 1 + 0.1 * torch.randn(H, generator=g)
    for bias in (None, b):
        for wt in (w, w.to(torch.bfloat16)):
            want = x.clone()
            RefOps().rmsnorm_add(y, bias, wt, 1e-5, want)
            got = x.to(DEV)
            ops.rmsnorm_add(y.to(DEV), bias.to(DEV) if bias is not None else None, wt.to(DEV), 1e-5, got)
            _close(got, want, torch.float32, "rmsnorm_add")
    got = x.to(DEV)
    ops.add_bias(got, b.to(DEV))
    assert torch.equal(got.cpu(), x + b)
    for dtype in (torch.float32, torch.bfloat16):
        I = H // 2 - 3
        gu = torch.randn(T, H, generator=g).to(dtype)
        bb = torch.randn(2 * I, generator=g)
        want = torch.zeros(T, I, dtype=dtype)
        RefOps().bias_silu_mul(gu, bb, want)
        got = torch.zeros(T, I, dtype=dtype, device=DEV)
        ops.bias_silu_mul(gu.to(DEV), bb.to(DEV), got)
        _close(got, want, dtype, "bias_silu_mul")


@pytest.mark.parametrize("E,top,n_shared,gate", [(8, 1, 1, True), (6, 2, 2, True), (7, 3, 0, False), (5, 5, 3, False), (64, 6, 1, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_with_sigmoid_scores_and_shared_choices(ops, dtype, E, top, n_shared, gate):
    g = torch.Generator().manual_seed(E)
    T, H = 50, 96
    h = torch.randn(T, H, generator=g).to(dtype)
    wr = (torch.randn(E + (1 if gate else 0), H, generator=g) * 0.3).to(dtype)
    cols = top + n_shared
    idx, wt = torch.zeros(T, cols, dtype=torch.int32, device=DEV), torch.zeros(T, cols, device=DEV)
    ops.moe_route(h.to(DEV), wr.to(DEV), top, 1, 1, idx, wt, score="sigmoid", normalise=False, n_shared=n_shared, shared_gate=gate)
    ri, rw = torch.zeros(T, cols, dtype=torch.int32), torch.zeros(T, cols)
    RefOps().moe_route(h, wr, top, 1, 1, ri, rw, score="sigmoid", normalise=False, n_shared=n_shared, shared_gate=gate)
    z = h.float() @ wr.float().T
    for t in range(T):
        assert idx[t, top:].tolist() == list(range(E, E + n_shared))            # the shared pieces, in order
        shared_w = float(torch.sigmoid(z[t, E])) if gate else 1.0
        assert all(abs(v - shared_w) < 1e-5 for v in wt[t, top:].tolist())
        a, b = dict(zip(idx[t, :top].tolist(), wt[t, :top].tolist())), dict(zip(ri[t, :top].tolist(), rw[t, :top].tolist()))
        assert len(a) == top
        if set(a) != set(b):             # a close call: the two scores must be as good as equal
            only_a, only_b = sorted(set(a) - set(b)), sorted(set(b) - set(a))
            assert len(only_a) == len(only_b) == 1 and abs(float(z[t, only_a[0]] - z[t, only_b[0]])) < 1e-3, (t, a, b)
            continue
        assert all(abs(a[k] - b[k]) < 1e-5 for k in a)                          # the scores themselves, not normalised
        assert all(abs(a[k] - float(torch.sigmoid(z[t, k]))) < 1e-5 for k in a)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", ["gelu", "gelu_tanh", "silu"])
# widths and expert sizes that are multiples of 32 reach the tensor-core kernel in bfloat16, the others the CUDA-core one
@pytest.mark.parametrize("T,H,F,E,top,n_in", [(1, 64, 32, 8, 2, 1), (70, 96, 40, 6, 3, 2), (300, 64, 24, 5, 1, 1), (300, 128, 160, 4, 3, 2),
                                               (9, 256, 96, 16, 4, 0), (700, 96, 72, 3, 2, 2)])
def test_experts_without_a_gate_matrix_weighted_on_their_input(ops, dtype, act, T, H, F, E, top, n_in):
    from zllm_b200.engine.batch import Workspace
    g = torch.Generator().manual_seed(T)
    h = torch.randn(T, H, generator=g).to(dtype)
    wu, wd = (torch.randn(E, F, H, generator=g) * 0.2).to(dtype), (torch.randn(E, H, F, generator=g) * 0.2).to(dtype)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if top == 1:
        idx[idx == E - 1] = 0                  # an expert may get no row at all
    wt = torch.rand(T, top, generator=g) * 1.5
    res = torch.randn(T, H, generator=g)
    for accumulate in (True, False):
        want = res.clone()
        RefOps().moe_experts(h, idx, wt, None, wu, wd, want, 1.0, None, n_input_weighted=n_in, activation=act, accumulate=accumulate)
        got = res.to(DEV)
        ops.moe_experts(h.to(DEV), idx.to(DEV), wt.to(DEV), None, wu.to(DEV), wd.to(DEV), got, 1.0, Workspace(1024, DEV),
                        n_input_weighted=n_in, activation=act, accumulate=accumulate)
        _close(got, want, dtype, f"experts {act} accumulate={accumulate}")
    if n_in and act == "gelu":
        # the weight is on the INPUT: the same weight on the output gives another result (the expert is not linear)
        other = res.clone()
        RefOps().moe_experts(h, idx, wt, None, wu, wd, other, 1.0, None, n_input_weighted=0, activation=act)
        assert float((other - want).abs().max()) > 1e-2 * float(want.abs().max())


# ---- rotation and cache write ----------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,dk,dv,dims,inter,bs,scaling", [
    (4, 2, 16, 24, 8, True, 16, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}),
    (3, 3, 32, 16, 32, True, 8, None), (6, 1, 16, 16, 0, True, 4, None), (5, 5, 12, 18, 6, False, 4, None),
    (8, 2, 64, 96, 24, True, 16, {"factor": 6.0, "low": 1.0, "high": 8.0, "original": 512})])
def test_rotation_and_cache_write(ops, dtype, nq, nkv, dk, dv, dims, inter, bs, scaling):
    from zllm_b200.cache import CacheManager
    from zllm_b200.parts import KVCacheSpec
    from zllm_b200.parts.rotary import RotaryOnTheFly
    from zllm_b200.models.decoder import Runtime
    g = torch.Generator().manual_seed(nq * dk + dv)
    off_k, off_v = nq * dk, nq * dk + nkv * dk
    ld = -(-(off_v + nkv * dv + nq) // 8) * 8
    cm = CacheManager([(KVCacheSpec(nkv, dk, None, True, dv if dv != dk else None), None)], bs, 64, 3, 160, dtype, DEV)
    freqs = None
    if dims:
        pe = RotaryOnTheFly(dims, 10000.0, scaling, interleaved=inter)
        pe.bind(Runtime(dtype, torch.device(DEV), ops))
        freqs = pe.frequencies()
    slots = [cm.admit() for _ in range(3)]
    cm.ensure(slots[1], 21), cm.advance(slots[1], 21)                # a request that is 21 positions in
    cm.ensure(slots[2], 99), cm.advance(slots[2], 99)
    ctx, after = _ctx(cm, [(slots[0], 37), (slots[1], 1), (slots[2], 2)])
    T = 40
    proj = torch.randn(T, ld, generator=g).to(dtype)
    got = proj.to(DEV)
    ops.rotate_store_kv(got, off_k, off_v, ctx, freqs, cm.view(0), nq, nkv, dk, dv, True)
    want = proj.clone()
    ref_cache = _CpuCache(cm.view(0))
    ref_cache.k_pages.zero_(), ref_cache.v_pages.zero_()
    cpu_freqs = copy.copy(freqs)
    if freqs is not None:
        cpu_freqs.freq = freqs.freq.cpu()
    RefOps().rotate_store_kv(want, off_k, off_v, _cpu(ctx), cpu_freqs, ref_cache, nq, nkv, dk, dv, True)
    _close(got, want, dtype, "rotated projection", scale=4.0)
    # what lies behind the heads (gate logits, padding) is untouched, and so are the value columns
    assert torch.equal(got[:, off_v:].cpu(), proj[:, off_v:])
    _close(cm.view(0).k_pages, ref_cache.k_pages, dtype, "key pages", scale=4.0)
    assert torch.equal(cm.view(0).v_pages.float().cpu(), ref_cache.v_pages)
    if dims and dtype == torch.float32:
        # against the closed form at a far position: row 38 is position 99 of the third request
        x, f = proj[38, off_k:off_k + dk].double(), freqs.freq.cpu().double()
        i = dims // 2 - 1
        a, b = (2 * i, 2 * i + 1) if inter else (i, i + dims // 2)
        ang = torch.tensor(99.0) * f[i]
        assert abs(float(got[38, off_k + a]) - float(x[a] * torch.cos(ang) - x[b] * torch.sin(ang))) < 1e-4
        assert torch.equal(got[38, off_k + dims:off_k + dk].cpu(), proj[38, off_k + dims:off_k + dk])


# ---- the attention kernels --------------------------------------------------------------------------
def _attention_case(ops, dtype, nq, nkv, dk, dv, window, keep, bs, lens, spike=None, gate=True):
    """Requests of ``lens`` = [(cached positions, new rows)]: the cached part is written first (random keys
    and values), then the new rows attend.  ``spike`` = (request, key position): that key and the request's
    last query are made so that their score stands far out, and the key's value is a constant 7."""
    from zllm_b200.cache import CacheManager
    from zllm_b200.parts import KVCacheSpec
    g = torch.Generator().manual_seed(nq * 131 + dk + (window or 0) + sum(a + b for a, b in lens))
    off_k, off_v = nq * dk, nq * dk + nkv * dk
    off_g = off_v + nkv * dv
    ld = -(-(off_g + nq) // 8) * 8
    total = sum(a + b for a, b in lens)
    cm = CacheManager([(KVCacheSpec(nkv, dk, window, True, dv if dv != dk else None, keep), None)], bs,
                      -(-total // bs) + 2 * len(lens) + 4, len(lens), max(a + b for a, b in lens) + bs, dtype, DEV)
    slots = [cm.admit() for _ in lens]
    view = cm.view(0)
    scale = dk ** -0.5
    outs = []
    for phase in (0, 1):
        entries = [(s, n[phase]) for s, n in zip(slots, lens) if n[phase] > 0]
        if not entries:
            continue
        ctx, after = _ctx(cm, entries)
        T = ctx.T
        proj = (torch.randn(T, ld, generator=g) * 0.7).to(dtype)
        if spike is not None:
            r = 0
            for s, n in zip(slots, lens):
                m = n[phase]
                if m == 0:
                    continue
                start = 0 if phase == 0 else n[0]
                if s == slots[spike[0]]:
                    if start <= spike[1] < start + m:                 # the key that stands out
                        row = r + spike[1] - start
                        proj[row, off_k:off_v] = 0
                        proj[row, off_k:off_v].view(nkv, dk)[:, 0] = 6.0
                        proj[row, off_v:off_g] = 7.0
                    if phase == 1 or lens[spike[0]][1] == 0:
                        row = r + m - 1                               # the request's last query looks for it
                        proj[row, :off_k] = 0
                        proj[row, :off_k].view(nq, dk)[:, 0] = 8.0 / scale
                r += m
        dev = proj.to(DEV)
        ops.rotate_store_kv(dev, off_k, off_v, ctx, None, view, nq, nkv, dk, dv, True)
        out = torch.zeros(T, nq * dv, dtype=dtype, device=DEV)
        ops.window_attention(dev, off_g if gate else -1, out, ctx, view, nq, nkv, dk, dv, scale, window, keep)
        want = torch.zeros(T, nq * dv, dtype=dtype)
        RefOps().window_attention(proj, off_g if gate else -1, want, _cpu(ctx), _CpuCache(view), nq, nkv, dk, dv, scale, window, keep)
        _close(out, want, dtype, f"window attention phase {phase}", scale=float(want.float().abs().max().clamp(min=0.05)))
        outs.append((out.float().cpu(), proj, ctx.T))
        for s, n in after:
            cm.advance(s, n)
        cm.check_integrity()
    return outs, (off_g, ld)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,dk,dv,window,keep,bs", [
    (4, 2, 16, 24, 24, 5, 16), (3, 3, 32, 16, 40, 0, 8), (6, 1, 16, 16, None, 0, 4), (3, 3, 24, 40, 7, 9, 8), (5, 5, 12, 18, 13, 3, 4),
    (8, 2, 64, 32, 64, 16, 16), (6, 3, 48, 112, 70, 11, 16), (8, 1, 128, 128, 200, 4, 16), (2, 1, 96, 48, 33, 17, 32),
    # sixteen heads on one key/value head fill the decode tile's rows (its unmasked path); seventeen go to the plain kernel
    (16, 1, 32, 32, 48, 4, 16), (17, 1, 16, 16, 20, 3, 8)])
def test_window_attention_in_prompts_portions_and_decoding(ops, dtype, nq, nkv, dk, dv, window, keep, bs):
    # whole prompts (one longer than several windows), portions with a cached prefix, single decoded tokens
    _attention_case(ops, dtype, nq, nkv, dk, dv, window, keep, bs, [(0, 150), (0, 3), (0, 1)])
    _attention_case(ops, dtype, nq, nkv, dk, dv, window, keep, bs, [(131, 70), (40, 1), (260, 1), (7, 2)])
    _attention_case(ops, dtype, nq, nkv, dk, dv, window, keep, bs, [(300, 1), (17, 1), (1, 1), (64, 1)], gate=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decode", [True, False])
def test_keys_at_every_edge_are_seen_or_not(ops, dtype, decode):
    """One key far out: the last query must find it (its head's output becomes the key's value, 7, times the
    gate) exactly when it is the query's own position, inside the window, or one of the kept first positions --
    at the window's first position and just before it, at the last kept position and just behind it, at page
    borders, far back."""
    nq, nkv, dk, dv, window, keep, bs = 4, 2, 32, 48, 40, 6, 16
    n = 203                                              # the last query sits at position 202
    last = n - 1
    cases = {0: True, keep - 1: True, keep: False, 15: False, 16: False, 100: False, last - window: False,
             last - window + 1: True, last - window + 2: True, 175: True, 176: True, last - 1: True, last: True}
    for key, seen in cases.items():
        lens = [(last, 1)] if decode else [(150, n - 150)]
        outs, (off_g, ld) = _attention_case(ops, dtype, nq, nkv, dk, dv, window, keep, bs, lens + [(30, 1 if decode else 9)], spike=(0, key))
        out, proj, T = outs[-1]
        row = lens[0][1] - 1
        gates = torch.sigmoid(proj[row, off_g:off_g + nq].float())
        heads = out[row].reshape(nq, dv)
        for a in range(nq):
            found = abs(float(heads[a].mean()) - 7.0 * float(gates[a])) < 0.2 * float(gates[a])
            assert found == seen, f"key {key} (query {last}, window {window}, kept {keep}): seen {found}, expected {seen}"


# ---- the whole model ----------------------------------------------------------------------------------
def _runner(d, name, dtype, num_blocks, graphs=False, slots=4, max_rows=512):
    from zllm_b200 import EngineConfig, ModelRunner
    return ModelRunner(d, engine_config=EngineConfig(dtype=dtype, block_size=VASONEX[name][1], num_blocks=num_blocks,
                                                     max_num_seqs=slots, max_num_batched_tokens=max_rows, cuda_graphs=graphs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_way_of_cutting_agrees_with_plain(tmp_path, name, dtype):
    d = make_vasonex_dir(tmp_path, name, dtype)
    cfg, w = read_dir(d)
    V = cfg["vocab"]
    reqs = [(f"r{i}", random_prompt(V, n, 20 + i)) for i, n in enumerate((5, 41, 33, 270, 1, 17, 64, 65))]
    max_tokens = 512
    steps = (TR.family_whole(reqs, "w.") + TR.family_tail(reqs, 40, "t.") + TR.family_portions(reqs, prefix="p.")
             + TR.family_portions(reqs, sizes=(2,), prefix="q.") + TR.family_mixed(reqs, max_tokens, 4, 1, "m.")
             + TR.family_mixed(reqs, max_tokens, 3, 2, "n."))
    bs = VASONEX[name][1]
    runner = _runner(d, name, dtype, max_tokens // bs)
    choices = _Choices(runner, cfg)
    got = TR.replay_inprocess(runner, steps, after_step=choices.after_step)
    runner.ops.check_async_errors()
    for prefix in ("w.", "t.", "p.", "q.", "m.", "n."):
        if dtype == "float32":
            _compare_following_the_choices(got, choices, cfg, w, reqs, prefix, 3e-4, 0.0, f"vasonex {name} {prefix} float32", str(d))
        else:
            _compare_following_the_choices(got, choices, cfg, w, reqs, prefix, 0.0, BF16_OF_SCALE[name], f"vasonex {name} {prefix} bfloat16", str(d),
                                           CLOSE_CALL_BF16)
    if dtype == "float32":
        # the order of every sum is fixed by the position: the ways of cutting agree bit for bit
        for rid, toks in reqs:
            for p in range(len(toks)):
                for prefix in ("t.", "p.", "q.", "m.", "n."):
                    assert torch.equal(got[("w." + rid, p)], got[(prefix + rid, p)]), (prefix, rid, p)
    assert all(f == max_tokens // bs for f in runner.cache.free_pages())
    runner.cache.check_integrity()


def test_a_kept_position_decides_a_logit_far_away(tmp_path):
    """The whole model with one layer's keys edited so that position 2 (kept) and position 9 (not kept) stand out:
    logits hundreds of positions later must agree with the plain implementation, which a lost kept page or a
    window that is one position off would not."""
    def edit(t):
        t["l0.mix.k"] *= 3.0
        t["l0.mix.q"] *= 3.0
    d = make_vasonex_dir(tmp_path, "A", "float32", edit=edit)
    cfg, w = read_dir(d)
    toks = random_prompt(cfg["vocab"], 300, 9)
    ref = {"far": PV.forward(toks, cfg, w).float()}
    runner = _runner(d, "A", "float32", 24)
    for fam in (TR.family_whole, lambda r: TR.family_tail(r, 200), lambda r: TR.family_portions(r, sizes=(23, 2, 16, 1, 5))):
        got = TR.replay_inprocess(runner, fam([("far", toks)]))
        TR.compare(got, ref, [("far", toks)], "", 5e-4, 0.0, "vasonex A sharpened keys")
    # without the kept positions the same logits are far off: the test can see them
    cfg2 = copy.deepcopy(cfg)
    for ly in cfg2["layers"]:
        ly["mixer"] = dict(ly["mixer"], mask={"size": ly["mixer"]["mask"]["size"], "keep_first": 0})
    assert float((PV.forward(toks, cfg2, w).float()[-50:] - ref["far"][-50:]).abs().max()) > 1e-2


def test_long_decoding_in_float32(tmp_path):
    d = make_vasonex_dir(tmp_path, "D", "float32")
    cfg, w = read_dir(d)
    toks = random_prompt(cfg["vocab"], 330, 5)
    ref = {"long": PV.forward(toks, cfg, w).float()}
    runner = _runner(d, "D", "float32", 84)              # 4 positions a page
    got = TR.replay_inprocess(runner, TR.family_tail([("long", toks)], 300))
    TR.compare(got, ref, [("long", toks)], "", 5e-4, 0.0, "vasonex D long decoding")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_through_the_engine(tmp_path, name, dtype, graphs):
    from zllm_b200 import Engine, SamplingParams
    d = make_vasonex_dir(tmp_path, name, dtype, std=0.2)
    cfg, w = read_dir(d)
    prompts = [random_prompt(cfg["vocab"], n, 60 + n) for n in (3, 70, 19, 8, 33, 1)]
    eng = Engine(str(d), dtype=dtype, cuda_graphs=graphs, block_size=VASONEX[name][1], num_blocks=64, max_num_seqs=4,
                 max_num_batched_tokens=48)
    got = eng.generate(prompts, SamplingParams.greedy(max_tokens=24))
    eng.runner.ops.check_async_errors()
    checked = 0
    for p, o in zip(prompts, got):
        assert len(o) == 24
        n = 24
        if dtype == "bfloat16":
            # behind a close call between two experts the bfloat16 stream may be another function's: it is compared up
            # to the first one (the float32 streams are compared to their end)
            _, margins = PV.forward(list(p) + list(o[:-1]), cfg, w, want_margins=True)
            close = (margins < CLOSE_CALL).nonzero().flatten()
            n = 24 if not len(close) else max(0, int(close[0]) - len(p) + 1)
        if n > 0:
            check_greedy_stream(lambda t: PV.forward(t, cfg, w).float(), p, o[:n], dtype, n, gap_of_scale=0.04,
                                what=f"vasonex {name} {dtype} graphs={graphs}")
        checked += n
    assert checked >= 8                        # (the float32 runs compare all 144)
    # and the same streams again through the same engine: slots, pages and graphs used again
    assert eng.generate(prompts, SamplingParams.greedy(max_tokens=24)) == got


def test_the_replay_program_runs_the_model(tmp_path):
    d = make_vasonex_dir(tmp_path, "B", "float32")
    cfg, w = read_dir(d)
    reqs = [(f"r{i}", random_prompt(cfg["vocab"], n, 80 + i)) for i, n in enumerate((9, 50, 3, 21, 40))]
    ref = {rid: PV.forward(toks, cfg, w).float() for rid, toks in reqs}
    steps = TR.family_mixed(reqs, 192, 4, 3)
    got = TR.replay_program(d, "float32", steps, 192, tmp_path / "out", cfg["vocab"], extra_args=("--block-size", "8"))
    TR.compare(got, ref, reqs, "", 3e-4, 0.0, "vasonex B through the replay program")
