"""Sepirax on the GPU: every new kernel alone against its plain torch statement (``ref_ops``),
then the whole model through the engine's step function, cache and scheduler against the plain
whole-sequence implementation (``plain_sepirax``), cut in every way, in both precisions.
"""
import copy

import pytest
import torch

import plain_sepirax as PS
import traces as TR
from configs import random_prompt
from gpu_util import DEV, F32_ATOL, check_greedy_stream, observe
from ref_ops import RefOps
from sepirax_util import SEPIRAX, make_sepirax_dir, read_dir

pytestmark = pytest.mark.gpu

# bounds of the bfloat16 comparisons, as a fraction of the request's largest |logit|, per test model: twice the
# worst observed on a B200 over these tests (A 0.0042, B 0.0076, C 0.0170: C's logits are small, 0.8 at most, so
# the same rounding is a larger fraction; with the tensor-core kernels switched off C reads 0.0164; D 0.0257: it
# chooses 4 of 9 experts, and where two router scores are closer than the rounding of the activations the
# bfloat16 engine may choose the other one -- median 0.0024, 99 % of the positions under 0.011)
BF16_OF_SCALE = {"A": 0.0085, "B": 0.016, "C": 0.034, "D": 0.052}


@pytest.fixture(scope="module")
def ops():
    from zllm_b200.kernels.ops import CudaOps
    o = CudaOps(DEV)
    o.configure(torch.bfloat16)
    return o


def _ctx(cm, entries, planners=(), max_rows=1024, as_decode=False):
    """A step description for entries [(slot, n_tokens)] appended at each slot's cached length."""
    from zllm_b200.engine.batch import StepBuffers, StepEntry, Workspace, fill_step, make_context
    buf = StepBuffers(max_rows, max_rows, DEV)
    ents, starts = [], []
    for slot, n in entries:
        start = cm.length[slot]
        assert cm.ensure(slot, start + n)
        ents.append(StepEntry(slot, [0] * n, ()))
        starts.append(start)
    T, R, nd, plans, mc = fill_step(buf, ents, starts, planners=() if as_decode else planners)
    buf.upload()
    cm.sync_tables()
    ctx = make_context(buf, T, R, nd, plans, mc, Workspace(max_rows, DEV), None if as_decode else ents, starts)
    for (slot, n), s in zip(entries, starts):
        cm.advance(slot, s + n)
    return ctx


def _cpu(ctx):
    c = copy.copy(ctx)
    for k in ("token_ids", "positions", "row_slot", "want_rows", "decode_rows"):
        setattr(c, k, getattr(ctx, k).cpu())
    c.aux = {k: v.cpu() for k, v in ctx.aux.items()}
    return c


class _View:
    """A CPU copy of a cache view (float32) for the plain statements."""

    def __init__(self, view):
        for k, v in vars(view).items():
            setattr(self, k, v.float().cpu() if isinstance(v, torch.Tensor) and v.is_floating_point()
                    else (v.cpu() if isinstance(v, torch.Tensor) else v))


def _close(got, want, dtype, what, f32=2e-5, bf16=0.02):
    got, want = got.float().cpu(), want.float().cpu()
    scale = float(want.abs().max()) or 1.0
    err = float((got - want).abs().max())
    lim = (f32 if dtype == torch.float32 else bf16) * scale
    assert err <= lim, f"{what}: max abs error {err:.3e} > {lim:.3e} (scale {scale:.3e})"


# ---- small kernels --------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh_softcap_and_scaled_embedding(ops, dtype):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(37, 200, generator=g) * 3
    w, b, alpha = torch.randn(200, generator=g), torch.randn(200, generator=g), torch.tensor([0.37])
    out = torch.empty(37, 200, dtype=dtype, device=DEV)
    ops.dynamic_tanh(x.to(DEV), alpha.to(DEV), w.to(DEV), b.to(DEV), out)
    _close(out, torch.tanh(0.37 * x) * w + b, dtype, "dynamic tanh", f32=1e-6, bf16=0.005)
    y = (torch.randn(5, 333, generator=g) * 40).to(DEV)
    want = 30.0 * torch.tanh(y.cpu() / 30.0)
    ops.softcap(y, 30.0)
    _close(y, want, torch.float32, "softcap", f32=1e-6)
    table = torch.randn(50, 64, generator=g).to(dtype)
    tok = torch.tensor([3, 49, 0, 7], dtype=torch.int32)
    e = torch.empty(4, 64, device=DEV)
    ops.embedding(tok.to(DEV), table.to(DEV), e, 16.0)
    assert torch.equal(e.cpu(), table[tok.long()].float() * 16.0)


@pytest.mark.parametrize("E,top,groups,keep", [(12, 3, 3, 2), (6, 1, 1, 1), (64, 6, 8, 4), (5, 5, 1, 1), (8, 2, 4, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router(ops, dtype, E, top, groups, keep):
    g = torch.Generator().manual_seed(E)
    T, H = 50, 96
    h = (torch.randn(T, H, generator=g)).to(dtype)
    wr = (torch.randn(E, H, generator=g) * 0.3).to(dtype)
    idx = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    wt = torch.zeros(T, top, device=DEV)
    ops.moe_route(h.to(DEV), wr.to(DEV), top, groups, keep, idx, wt)
    ri, rw = torch.zeros(T, top, dtype=torch.int32), torch.zeros(T, top)
    RefOps().moe_route(h, wr, top, groups, keep, ri, rw)
    scores = torch.softmax(h.float() @ wr.float().T, dim=-1)
    for t in range(T):
        a = dict(zip(idx[t].tolist(), wt[t].tolist()))
        b = dict(zip(ri[t].tolist(), rw[t].tolist()))
        assert len(a) == top and abs(sum(a.values()) - 1.0) < 1e-5
        if set(a) != set(b):
            # a close call between two experts (the sums run in another order): their scores must be as good as equal
            only_a, only_b = sorted(set(a) - set(b)), sorted(set(b) - set(a))
            assert len(only_a) == len(only_b) == 1 and \
                abs(float(scores[t, only_a[0]] - scores[t, only_b[0]])) < 1e-4 * float(scores[t].max()), (t, a, b, scores[t].tolist())
            continue
        assert all(abs(a[k] - b[k]) < 1e-5 for k in a)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
# widths and expert sizes that are multiples of 32 reach the tensor-core kernel in bfloat16, the others the CUDA-core one
@pytest.mark.parametrize("T,H,F,E,top", [(1, 64, 32, 8, 2), (70, 96, 40, 6, 3), (300, 64, 24, 5, 1), (300, 128, 160, 4, 2), (40, 128, 192, 8, 2),
                                          (9, 256, 96, 16, 4), (700, 96, 72, 3, 1)])
def test_experts(ops, dtype, T, H, F, E, top):
    from zllm_b200.engine.batch import Workspace
    g = torch.Generator().manual_seed(T)
    h = torch.randn(T, H, generator=g).to(dtype)
    wg, wu = (torch.randn(E, F, H, generator=g) * 0.2).to(dtype), (torch.randn(E, F, H, generator=g) * 0.2).to(dtype)
    wd = (torch.randn(E, H, F, generator=g) * 0.2).to(dtype)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if top == 1:
        idx[idx == E - 1] = 0                  # an expert may get no row at all
    wt = torch.rand(T, top, generator=g)
    res = torch.randn(T, H, generator=g)
    want = res.clone()
    RefOps().moe_experts(h, idx, wt, wg, wu, wd, want, 0.7, None)
    got = res.to(DEV)
    ops.moe_experts(h.to(DEV), idx.to(DEV), wt.to(DEV), wg.to(DEV), wu.to(DEV), wd.to(DEV), got, 0.7, Workspace(512, DEV))
    _close(got, want, dtype, "experts")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,G,N,K,stride", [(75, 5, 40, 24, 40), (300, 3, 200, 64, 72), (9, 4, 136, 128, 128)])
def test_products_per_head(ops, dtype, T, G, N, K, stride):
    # K a multiple of 32 with strides of eight reaches the tensor-core kernel in bfloat16
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, G * stride, generator=g).to(dtype)
    w = (torch.randn(G, N, K, generator=g) * 0.3).to(dtype)
    gate = torch.randn(T, 16 + G * N, generator=g).to(dtype)
    for out_dtype, gt in ((torch.float32, None), (dtype, (gate, 16))):
        want = torch.zeros(T, G * N, dtype=out_dtype)
        RefOps().linear_heads(x, stride, w, want, gate=gt, out_scale=0.6)
        got = torch.zeros(T, G * N, dtype=out_dtype, device=DEV)
        ops.linear_heads(x.to(DEV), stride, w.to(DEV), got, gate=(gt[0].to(DEV), gt[1]) if gt else None, out_scale=0.6)
        _close(got, want, out_dtype, "products per head")


# ---- attention through the latent ---------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
# the last three reach the tensor-core kernel in bfloat16 (a latent of 64, 128 or 512 entries, a rotated part of 16 x n)
@pytest.mark.parametrize("H,dn,dr,dims,rank,q_rank,bs", [(4, 16, 8, 8, 48, 40, 16), (3, 24, 16, 8, 72, 56, 8), (9, 8, 0, 0, 200, 32, 16),
                                                         (5, 16, 16, 16, 64, 40, 8), (20, 32, 32, 16, 128, 64, 16),
                                                         (16, 16, 64, 64, 512, 96, 16)])
def test_latent_attention_kernels(ops, dtype, H, dn, dr, dims, rank, q_rank, bs):
    from zllm_b200.cache import CacheManager
    from zllm_b200.parts import KVCacheSpec
    from zllm_b200.parts.rotary import yarn_frequencies
    g = torch.Generator().manual_seed(H)
    cm = CacheManager([(KVCacheSpec(1, rank + dr, None, values=False), None)], bs, 80, 3, 80 * bs, dtype, DEV)
    view = cm.view(0)
    assert view.v_pages is None
    if dims:
        f, mag = yarn_frequencies(dims, 10000.0, 4.0, 32, 8.0, 1.0)
        freqs = (f.to(DEV), mag, dims)
    else:
        freqs = (torch.zeros(0, device=DEV), 1.0, 0)
    cpu_freqs = (freqs[0].cpu(), freqs[1], freqs[2])
    wq, wc = torch.rand(q_rank, generator=g) + 0.5, torch.rand(rank, generator=g) + 0.5
    ld = q_rank + rank + dr + 8
    s0, s1 = cm.admit(), cm.admit()
    ref = RefOps()
    plan = [[(s0, 37)], [(s0, 1), (s1, 2)], [(s1, 60), (s0, 1)], [(s0, 1)], [(s0, 33), (s1, 1)], [(s0, 250)], [(s1, 1), (s0, 1)],
            [(s0, 1)]]
    for entries in plan:
        # steps of single tokens only are given as the engine gives decode steps (no host-side description):
        # long contexts are then taken in splits
        ctx = _ctx(cm, entries, as_decode=all(n == 1 for _, n in entries))
        T = ctx.T
        proj = torch.randn(T, ld, generator=g).to(dtype)
        cq = torch.zeros(T, q_rank, dtype=dtype, device=DEV)
        ops.latent_prepare(proj.to(DEV), 0, q_rank, q_rank, rank, dr, wq.to(DEV), wc.to(DEV), 1e-5, freqs, cq, ctx, view)
        cview = _View(view)
        before = cview.k_pages.clone()
        cq_ref = torch.zeros(T, q_rank, dtype=dtype)
        ref.latent_prepare(proj, 0, q_rank, q_rank, rank, dr, wq, wc, 1e-5, cpu_freqs, cq_ref, _cpu(ctx), cview)
        _close(cq, cq_ref, dtype, "normed query latent", bf16=0.01)
        # the plain statement wrote the same rows into its copy (elsewhere both are what was there before)
        _close(before, cview.k_pages, dtype, "cache rows", f32=1e-5, bf16=0.01)
        cview.k_pages = before                   # attend over what the kernel itself cached
        q = torch.randn(T, H * (dn + dr), generator=g).to(dtype)
        q_lat = torch.randn(T, H * rank, generator=g) * 0.3
        # one key stands out per row: the query's latent side is a multiple of that key's latent
        pos = ctx.positions.cpu().tolist()
        slot = ctx.row_slot.cpu().tolist()
        for t in range(T):
            cands = [p for p in (0, bs - 1, bs, bs + 1, 31, 32, 33, pos[t] - 1, pos[t]) if 0 <= p <= pos[t]]
            p_star = cands[t % len(cands)]
            page = int(cview.block_table[slot[t], p_star // bs])
            c = before[page, 0, p_star % bs, :rank]
            q_lat[t, (t % H) * rank:(t % H + 1) * rank] = c * (20.0 / float(c @ c) / 0.25)
        out = torch.zeros(T, H * rank, dtype=dtype, device=DEV)
        ops.latent_attention(q_lat.to(DEV), q.to(DEV), dn + dr, out, ctx, view, H, rank, dr, freqs, 0.25)
        want = torch.zeros(T, H * rank, dtype=dtype)
        ref.latent_attention(q_lat, q, dn + dr, want, _cpu(ctx), cview, H, rank, dr, cpu_freqs, 0.25)
        _close(out, want, dtype, f"latent attention {entries}", f32=2e-5, bf16=0.02)


# ---- the matrix memory ------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
# sizes that fill the registers exactly (dk 64, 256) take the instantiations made for them, the others the general one
@pytest.mark.parametrize("H,dk,dv", [(2, 16, 24), (3, 40, 16), (1, 100, 200), (2, 160, 40), (2, 64, 32), (1, 256, 48)])
def test_matrix_memory_kernel(ops, dtype, H, dk, dv):
    from zllm_b200.cache import CacheManager
    from zllm_b200.kernels.ops import CudaOps
    from zllm_b200.parts import StateSpec
    g = torch.Generator().manual_seed(dk)
    per = H * (dk * dv + dk + 1)
    cm = CacheManager([(StateSpec((per,), "float32"), None)], 16, 4, 3, 4096, dtype, DEV)
    view = cm.view(0)
    cstate = type("S", (), {})()
    cstate.state = torch.zeros(3, per)
    ref = RefOps()
    s0, s1 = cm.admit(), cm.admit()
    ld = 2 * H * dk + 2 * H * dv + 8
    oq, ok, ov, og = 0, H * dk, 2 * H * dk, 2 * H * dk + H * dv + 8
    bi, bf = torch.randn(H, generator=g), torch.randn(H, generator=g) + 2.0
    wn = torch.rand(H * dv, generator=g) + 0.5
    plan = [([(s0, 19)], False), ([(s0, 1), (s1, 9)], False), ([(s0, 1), (s1, 1)], True), ([(s1, 2), (s0, 8)], False),
            ([(s0, 1)], True), ([(s1, 70)], False)]
    for entries, as_decode in plan:
        ctx = _ctx(cm, entries, planners=(CudaOps.plan_row_segments,), as_decode=as_decode)
        T = ctx.T
        x = (torch.randn(T, ld, generator=g) * 0.7).to(dtype)
        z = torch.randn(T, 2 * H, generator=g) * 3
        out = torch.zeros(T, H * dv, dtype=dtype, device=DEV)
        ops.matrix_memory(x.to(DEV), oq, ok, ov, og, z.to(DEV), bi.to(DEV), bf.to(DEV), 8.0, wn.to(DEV), 1e-5, 0.7, out, ctx,
                          view, H, dk, dv)
        want = torch.zeros(T, H * dv, dtype=dtype)
        ref.matrix_memory(x, oq, ok, ov, og, z, bi, bf, 8.0, wn, 1e-5, 0.7, want, _cpu(ctx), cstate, H, dk, dv)
        _close(out, want, dtype, f"matrix memory {entries}", f32=5e-5, bf16=0.02)
        _close(view.state, cstate.state, torch.float32, "state", f32=5e-5)


# ---- the whole model ------------------------------------------------------------------------------------------
def _runner(d, name, dtype, num_blocks, max_rows=512, slots=4, graphs=False):
    from zllm_b200 import EngineConfig, ModelRunner
    return ModelRunner(d, engine_config=EngineConfig(dtype=dtype, block_size=SEPIRAX[name][1], num_blocks=num_blocks,
                                                     max_num_seqs=slots, max_num_batched_tokens=max_rows, cuda_graphs=graphs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_way_of_cutting_agrees_with_plain(tmp_path, name, dtype):
    d = make_sepirax_dir(tmp_path, name, dtype)
    cfg, w = read_dir(d)
    V = cfg["vocab"]
    reqs = [(f"r{i}", random_prompt(V, n, 20 + i)) for i, n in enumerate((5, 41, 33, 270, 1, 17, 64, 65))]
    ref = {rid: PS.forward(cfg, w, toks).float() for rid, toks in reqs}
    max_tokens = 512
    steps = (TR.family_whole(reqs, "w.") + TR.family_tail(reqs, 40, "t.") + TR.family_portions(reqs, prefix="p.")
             + TR.family_portions(reqs, sizes=(2,), prefix="q.") + TR.family_mixed(reqs, max_tokens, 4, 1, "m.")
             + TR.family_mixed(reqs, max_tokens, 3, 2, "n."))
    bs = SEPIRAX[name][1]
    runner = _runner(d, name, dtype, max_tokens // bs)
    got = TR.replay_inprocess(runner, steps)
    runner.ops.check_async_errors()
    for prefix in ("w.", "t.", "p.", "q.", "m.", "n."):
        if dtype == "float32":
            TR.compare(got, ref, reqs, prefix, 3e-4, 0.0, f"sepirax {name} {prefix} float32")
        else:
            TR.compare(got, ref, reqs, prefix, 0.0, BF16_OF_SCALE[name], f"sepirax {name} {prefix} bfloat16")
    if dtype == "float32":
        # the order of every sum is fixed by the position: the ways of cutting agree bit for bit
        for rid, toks in reqs:
            for p in range(len(toks)):
                for prefix in ("t.", "p.", "q.", "m.", "n."):
                    assert torch.equal(got[("w." + rid, p)], got[(prefix + rid, p)]), (prefix, rid, p)
    assert all(f == max_tokens // bs for f in runner.cache.free_pages())


def test_long_decoding_in_float32(tmp_path):
    d = make_sepirax_dir(tmp_path, "A", "float32")
    cfg, w = read_dir(d)
    toks = random_prompt(cfg["vocab"], 330, 5)
    ref = {"long": PS.forward(cfg, w, toks).float()}
    runner = _runner(d, "A", "float32", 32)
    got = TR.replay_inprocess(runner, TR.family_tail([("long", toks)], 300))
    TR.compare(got, ref, [("long", toks)], "", 5e-4, 0.0, "sepirax A long decoding")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_through_the_engine(tmp_path, name, dtype, graphs):
    from zllm_b200 import Engine, SamplingParams
    d = make_sepirax_dir(tmp_path, name, dtype, std=0.2)
    cfg, w = read_dir(d)
    prompts = [random_prompt(cfg["vocab"], n, 60 + n) for n in (3, 70, 19, 8, 33, 1)]
    eng = Engine(str(d), dtype=dtype, cuda_graphs=graphs, block_size=SEPIRAX[name][1], num_blocks=64, max_num_seqs=4,
                 max_num_batched_tokens=48)
    got = eng.generate(prompts, SamplingParams.greedy(max_tokens=24))
    eng.runner.ops.check_async_errors()
    for p, o in zip(prompts, got):
        check_greedy_stream(lambda t: PS.forward(cfg, w, t).float(), p, o, dtype, 24, gap_of_scale=0.04,
                            what=f"sepirax {name} {dtype} graphs={graphs}")
    # and the same streams again through the same engine: slots, pages and graphs used again
    assert eng.generate(prompts, SamplingParams.greedy(max_tokens=24)) == got


def test_the_replay_program_runs_the_model(tmp_path):
    d = make_sepirax_dir(tmp_path, "B", "float32")
    cfg, w = read_dir(d)
    reqs = [(f"r{i}", random_prompt(cfg["vocab"], n, 80 + i)) for i, n in enumerate((9, 50, 3, 21, 40))]
    ref = {rid: PS.forward(cfg, w, toks).float() for rid, toks in reqs}
    steps = TR.family_mixed(reqs, 192, 4, 3)
    got = TR.replay_program(d, "float32", steps, 192, tmp_path / "out", cfg["vocab"], extra_args=("--block-size", "8"))
    TR.compare(got, ref, reqs, "", 3e-4, 0.0, "sepirax B through the replay program")
