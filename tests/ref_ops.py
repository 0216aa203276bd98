"""Plain torch statements of every kernel the engine calls, one function per kernel.

Two uses: (1) each CUDA kernel is compared alone with the function of the same
name here; (2) given to the engine as its kernel table, they let the host side
(cache, tables, batch description, step, scheduler) run on the CPU in tests.
They are never chosen by the package itself: the product path has CUDA only.

Formulas cite zllm's kernels (src/backend/gpu/shaders.rs) where one exists.
"""
from __future__ import annotations

import math

import torch

GROUP = 8


def deinterleave_gate_up(w):
    """[2I, K] in groups of (8 gate rows, 8 up rows) -> gate [I,K], up [I,K]."""
    two_i, K = w.shape
    w = w.reshape(two_i // (2 * GROUP), 2, GROUP, K)
    return w[:, 0].reshape(-1, K), w[:, 1].reshape(-1, K)


class RefOps:
    decode_split_keys = 256

    def __init__(self, device="cpu"):
        self.device = torch.device(device)
        self.dtype = torch.float32

    def configure(self, dtype):
        self.dtype = dtype

    def decode_splits(self, max_ctx):
        return max(1, -(-max_ctx // self.decode_split_keys))

    # ---- embedding: x[t] = E[token[t]] (fork.rs:935) -------------------------------
    def embedding(self, token_ids, table, out, scale=1.0):
        out.copy_(table[token_ids.long()].float() * scale)

    def linear_plain(self, x, w, out, mode):
        self.linear(x, w, out, mode)

    # ---- Dynamic Tanh and the soft cap ---------------------------------------------------
    def dynamic_tanh(self, x, alpha, weight, bias, out):
        out.copy_((torch.tanh(alpha.float() * x.float()) * weight.float() + bias.float()).to(out.dtype))

    def softcap(self, x, cap):
        x.copy_(cap * torch.tanh(x / cap))

    # ---- attention through a cached latent ------------------------------------------------
    @staticmethod
    def _rotate(v, pos, freqs):
        """v [..., rot]: the first dims entries rotated, entry i with i + dims/2, angle pos * f_i."""
        f, mag, dims = freqs
        if dims == 0:
            return v
        half = dims // 2
        ang = (torch.tensor(float(pos), dtype=torch.float32) * f.float().cpu())
        c, s = torch.cos(ang) * mag, torch.sin(ang) * mag
        a, b = v[..., :half], v[..., half:dims]
        return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], dim=-1)

    def latent_prepare(self, proj, off_q, q_rank, off_kv, rank, rot, wq, wc, eps, freqs, cq, ctx, cache, write_cache=True):
        bs = cache.block_size if write_cache else 1
        for t in range(proj.shape[0]):
            slot = int(ctx.row_slot[t])
            if slot < 0:
                cq[t].zero_()
                continue
            row = proj[t].float()
            a = row[off_q:off_q + q_rank]
            cq[t].copy_((a / torch.sqrt((a * a).mean() + eps) * wq.float()).to(cq.dtype))
            if not write_cache:
                continue
            c = row[off_kv:off_kv + rank]
            c = c / torch.sqrt((c * c).mean() + eps) * wc.float()
            p = int(ctx.positions[t])
            kr = self._rotate(row[off_kv + rank:off_kv + rank + rot], p, freqs)
            page = int(cache.block_table[slot, p // bs])
            assert page >= 0, "write to a position without a page"
            cache.k_pages[page, 0, p % bs, :] = torch.cat([c, kr]).to(cache.k_pages.dtype)

    def latent_attention(self, q_lat, q, q_off, out, ctx, cache, n_heads, rank, rot, freqs, scale):
        bs = cache.block_size
        T = q.shape[0]
        for t in range(T):
            slot = int(ctx.row_slot[t])
            if slot < 0:
                out[t].zero_()
                continue
            p = int(ctx.positions[t])
            idx = torch.arange(0, p + 1)
            pages = cache.block_table[slot, (idx // bs).long()].long()
            assert (pages >= 0).all(), "read of a position whose page was given back"
            rows = cache.k_pages[pages, 0, (idx % bs).long(), :].float()          # [n, rank + rot]
            ql = q_lat[t].float().reshape(n_heads, rank)
            qr = self._rotate(q[t].float().reshape(n_heads, q_off)[:, q_off - rot:], p, freqs)
            sc = (ql @ rows[:, :rank].T + qr @ rows[:, rank:].T) * scale
            out[t].copy_((torch.softmax(sc, dim=-1) @ rows[:, :rank]).reshape(-1).to(out.dtype))

    def linear_heads(self, x, x_head_stride, w, out, gate=None, out_scale=1.0):
        G, N, K = w.shape
        for g in range(G):
            y = x[:, g * x_head_stride:g * x_head_stride + K].float() @ w[g].float().T
            if gate is not None:
                gt, c0 = gate
                y = y * torch.sigmoid(gt[:, c0 + g * N:c0 + (g + 1) * N].float()) * out_scale
            out[:, g * N:(g + 1) * N] = y.to(out.dtype)

    # ---- matrix memory ------------------------------------------------------------------------
    @staticmethod
    def plan_row_segments(entries, starts, aux, bucketed=False):
        from zllm_b200.kernels.ops import CudaOps
        return CudaOps.plan_row_segments(entries, starts, aux, bucketed)

    def matrix_memory(self, qkvg, oq, ok, ov, og, z, bias_i, bias_f, cap, norm_w, eps, mult, out, ctx, cache, H, dk, dv):
        T = qkvg.shape[0]
        x = qkvg.float()
        segs = ctx.aux.get("row_segments") if ctx.aux else None
        runs = [(int(a), int(b), int(c)) for a, b, c, _ in segs.tolist()] if segs is not None else \
            [(t, 1, int(ctx.row_slot[t])) for t in range(T)]
        raw = torch.zeros(T, H, dv)
        for row0, rows, slot in runs:
            if rows <= 0 or slot < 0:
                continue
            st = cache.state[slot].reshape(H, dk * dv + dk + 1)
            for h in range(H):
                S = st[h, :dk * dv].reshape(dk, dv).clone()
                n = st[h, dk * dv:dk * dv + dk].clone()
                m = st[h, dk * dv + dk].clone()
                for t in range(row0, row0 + rows):
                    q = x[t, oq + h * dk:oq + (h + 1) * dk] * dk ** -0.5
                    k = x[t, ok + h * dk:ok + (h + 1) * dk]
                    v = x[t, ov + h * dv:ov + (h + 1) * dv]
                    gi = cap * torch.tanh((z[t, h] + bias_i[h]) / cap)
                    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((z[t, H + h] + bias_f[h]) / cap))
                    m_new = torch.maximum(gf + m, gi)
                    keep, take = torch.exp(gf + m - m_new), torch.exp(gi - m_new)
                    S = keep * S + take * k[:, None] * v[None, :]
                    n = keep * n + take * k
                    m = m_new
                    raw[t, h] = (S.T @ q) / (torch.maximum((n * q).sum().abs(), torch.exp(-m)) + 1e-6)
                st[h, :dk * dv] = S.reshape(-1)
                st[h, dk * dv:dk * dv + dk] = n
                st[h, dk * dv + dk] = m
        y = raw / torch.sqrt((raw * raw).mean(-1, keepdim=True) + eps)
        y = y.reshape(T, H * dv) * norm_w.float() * torch.sigmoid(x[:, og:og + H * dv]) * mult
        live = (ctx.row_slot[:T] >= 0)[:, None]
        out.copy_(torch.where(live, y, torch.zeros_like(y)).to(out.dtype))

    # ---- mixture of experts ----------------------------------------------------------------------
    def moe_route(self, h, w_router, top, groups, keep, idx, weights, score="softmax", normalise=True, n_shared=0,
                  shared_gate=False):
        z = h.float() @ w_router.float().T
        E = z.shape[1] - (1 if shared_gate else 0)
        s = torch.softmax(z[:, :E], dim=-1) if score == "softmax" else torch.sigmoid(z[:, :E])
        T = s.shape[0]
        per = E // groups
        gbest = s.reshape(T, groups, per).max(-1).values
        kept = torch.zeros(T, groups, dtype=torch.bool)
        kept.scatter_(1, torch.topk(gbest, keep, dim=-1).indices, True)
        masked = torch.where(kept[:, :, None].expand(T, groups, per).reshape(T, E), s, torch.full_like(s, -1.0))
        ch = torch.topk(masked, top, dim=-1).indices
        sc = torch.gather(s, 1, ch)
        idx[:, :top] = ch.to(idx.dtype)
        weights[:, :top] = sc / (sc.sum(-1, keepdim=True) + 1e-20) if normalise else sc
        for c in range(n_shared):
            idx[:, top + c] = E + c
            weights[:, top + c] = torch.sigmoid(z[:, E]) if shared_gate else 1.0

    @staticmethod
    def _expert_act(a, activation):
        if activation == "gelu":
            return 0.5 * a * (1.0 + torch.erf(a / math.sqrt(2.0)))
        if activation == "gelu_tanh":
            return 0.5 * a * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (a + 0.044715 * a ** 3)))
        return a / (1.0 + torch.exp(-a))

    def moe_experts(self, h, idx, weights, w_gate, w_up, w_down, residual, scale, ws, n_input_weighted=0, activation="silu",
                    accumulate=True):
        x = h.float()
        for t in range(x.shape[0]):
            acc = torch.zeros(x.shape[1])
            for j in range(idx.shape[1]):
                e = int(idx[t, j])
                on_input = j < n_input_weighted
                c = float(weights[t, j]) if on_input else 1.0
                up = (x[t] @ w_up[e].float().T) * c
                if w_gate is not None:
                    a = (x[t] @ w_gate[e].float().T) * c
                    act = a / (1.0 + torch.exp(-a)) * up
                else:
                    act = self._expert_act(up, activation)
                act = act.to(h.dtype).float()
                acc = acc + (1.0 if on_input else weights[t, j]) * (act @ w_down[e].float().T)
            if accumulate:
                residual[t] += scale * acc
            else:
                residual[t] = scale * acc

    # ---- a branch's output norm, biases ----------------------------------------------------------
    def rmsnorm_add(self, y, bias, weight, eps, residual):
        v = y.float() if bias is None else y.float() + bias.float()
        residual.add_(v * torch.rsqrt((v * v).mean(dim=-1, keepdim=True) + eps) * weight.float())

    def add_bias(self, x, bias):
        x.add_(bias.float())

    def bias_silu_mul(self, gu, bias, out):
        I = out.shape[1]
        g = gu[:, :I].float() + bias[:I].float()
        u = gu[:, I:2 * I].float() + bias[I:].float()
        out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))

    # ---- attention with a window that keeps the first positions ------------------------------------
    def rotate_store_kv(self, proj, off_k, off_v, ctx, freqs, cache, nq, nkv, dk, dv, write_cache=True):
        T = proj.shape[0]
        pos = ctx.positions.long()
        x = proj.float()
        if freqs is not None and freqs.dims:
            half = freqs.dims // 2
            ang = pos.float()[:, None] * freqs.freq.float()[None, :]            # float32 angles
            c, s = (torch.cos(ang) * freqs.magnitude)[:, None, :], (torch.sin(ang) * freqs.magnitude)[:, None, :]
            for start, n in ((0, nq), (off_k, nkv)):
                hd = x[:, start:start + n * dk].reshape(T, n, dk).clone()
                if freqs.interleaved:
                    a, b = hd[..., 0:freqs.dims:2].clone(), hd[..., 1:freqs.dims:2].clone()
                    hd[..., 0:freqs.dims:2] = a * c - b * s
                    hd[..., 1:freqs.dims:2] = b * c + a * s
                else:
                    a, b = hd[..., :half].clone(), hd[..., half:freqs.dims].clone()
                    hd[..., :half] = a * c - b * s
                    hd[..., half:freqs.dims] = b * c + a * s
                x[:, start:start + n * dk] = hd.reshape(T, n * dk)
        live = (ctx.row_slot[:T] >= 0)[:, None]
        proj.copy_(torch.where(live, x, proj.float()).to(proj.dtype))
        if not write_cache:
            return
        bs = cache.block_size
        for t in range(T):
            slot = int(ctx.row_slot[t])
            if slot < 0:
                continue
            p = int(pos[t])
            page = int(cache.block_table[slot, p // bs])
            assert page >= 0, "write to a position without a page"
            cache.k_pages[page, :, p % bs, :] = proj[t, off_k:off_k + nkv * dk].reshape(nkv, dk).to(cache.k_pages.dtype)
            cache.v_pages[page, :, p % bs, :] = proj[t, off_v:off_v + nkv * dv].reshape(nkv, dv).to(cache.v_pages.dtype)

    def window_attention(self, proj, off_g, out, ctx, cache, nq, nkv, dk, dv, scale, window, keep_first):
        T = proj.shape[0]
        bs = cache.block_size
        rep = nq // nkv
        for t in range(T):
            slot = int(ctx.row_slot[t])
            if slot < 0:
                out[t].zero_()
                continue
            p = int(ctx.positions[t])
            q = proj[t, :nq * dk].float().reshape(nq, dk)
            lo = 0 if not window else max(0, p - window + 1)
            idx = torch.tensor([j for j in range(p + 1) if j >= lo or j < (keep_first or 0)])
            pages = cache.block_table[slot, (idx // bs).long()].long()
            assert (pages >= 0).all(), "read of a position whose page was given back"
            K = cache.k_pages[pages, :, (idx % bs).long(), :].float().repeat_interleave(rep, dim=1)    # [n, nq, dk]
            V = cache.v_pages[pages, :, (idx % bs).long(), :].float().repeat_interleave(rep, dim=1)
            pr = torch.softmax(torch.einsum("hd,nhd->hn", q, K) * scale, dim=-1)
            o = torch.einsum("hn,nhd->hd", pr, V)
            if off_g >= 0:
                o = o * torch.sigmoid(proj[t, off_g:off_g + nq].float())[:, None]
            out[t].copy_(o.reshape(-1).to(out.dtype))

    # ---- BNORM (shaders.rs:545-564) --------------------------------------------------
    def rmsnorm(self, x, weight, eps, out, rows=None):
        xf = x.float() if rows is None else x[rows.long()].float()
        inv = torch.rsqrt((xf * xf).mean(dim=-1, keepdim=True) + eps)
        out.copy_((xf * inv * weight.float()).to(out.dtype))

    # ---- products out = x W^T with the three epilogues --------------------------------
    def linear(self, x, w, out, mode):
        xf, wf = x.float(), w.float()
        if mode == "store":
            out.copy_((xf @ wf.T).to(out.dtype))
        elif mode == "add":
            out.add_((xf @ wf.T).to(out.dtype))
        elif mode == "swiglu":
            g, u = deinterleave_gate_up(wf)
            gv = xf @ g.T
            out.copy_((gv / (1.0 + torch.exp(-gv)) * (xf @ u.T)).to(out.dtype))
        else:
            raise ValueError(mode)

    # ---- SILU_MUL (shaders.rs:976-990) -------------------------------------------------
    def silu_mul(self, a, b, out):
        af = a.float()
        out.copy_((af / (1.0 + torch.exp(-af)) * b.float()).to(out.dtype))

    # ---- BROPE + BKV_PACK (shaders.rs:566-587, 727-756) -------------------------------
    def rope_kv_store(self, qkv, ctx, rot, cache, nq, nkv, hd, write_cache=True):
        T = qkv.shape[0]
        pos = ctx.positions.long()
        x = qkv.float().reshape(T, nq + 2 * nkv, hd)
        q, k, v = x[:, :nq], x[:, nq:nq + nkv], x[:, nq + nkv:]
        if rot is not None:
            c = rot.cos[pos][:, None, :]
            s = rot.sin[pos][:, None, :]
            rd = rot.rot_dim

            def rotate(t):
                t = t.clone()
                r = t[..., :rd]
                if rot.interleaved:
                    a, b = r[..., 0::2], r[..., 1::2]
                    o = torch.empty_like(r)
                    o[..., 0::2] = a * c - b * s
                    o[..., 1::2] = a * s + b * c
                else:
                    a, b = r[..., :rd // 2], r[..., rd // 2:]
                    o = torch.cat([a * c - b * s, a * s + b * c], dim=-1)
                t[..., :rd] = o
                return t
            q, k = rotate(q), rotate(k)
        out = torch.cat([q, k, v], dim=1).reshape(T, -1)
        qkv.copy_(out.to(qkv.dtype))
        if not write_cache:
            return
        bs = cache.block_size
        kq = qkv.reshape(T, nq + 2 * nkv, hd)
        for t in range(T):
            slot = int(ctx.row_slot[t])
            if slot < 0:
                continue
            p = int(pos[t])
            page = int(cache.block_table[slot, p // bs])
            assert page >= 0, "write to a position without a page"
            cache.k_pages[page, :, p % bs, :] = kq[t, nq:nq + nkv].to(cache.k_pages.dtype)
            cache.v_pages[page, :, p % bs, :] = kq[t, nq + nkv:].to(cache.v_pages.dtype)

    # ---- BDSDPA_PAGED (shaders.rs:670-725) ----------------------------------------------
    def paged_attention(self, qkv, out, ctx, cache, nq, nkv, hd, scale, window):
        T = qkv.shape[0]
        bs = cache.block_size
        q = qkv.float().reshape(T, nq + 2 * nkv, hd)[:, :nq]
        rep = nq // nkv
        for t in range(T):
            slot = int(ctx.row_slot[t])
            if slot < 0:
                out[t].zero_()
                continue
            p = int(ctx.positions[t])
            lo = 0 if not window else max(0, p - window + 1)
            idx = torch.arange(lo, p + 1)
            pages = cache.block_table[slot, (idx // bs).long()].long()
            assert (pages >= 0).all(), "read of a position whose page was given back"
            K = cache.k_pages[pages, :, (idx % bs).long(), :].float()   # [n, nkv, hd]
            V = cache.v_pages[pages, :, (idx % bs).long(), :].float()
            K = K.repeat_interleave(rep, dim=1)
            V = V.repeat_interleave(rep, dim=1)
            s = torch.einsum("hd,nhd->hn", q[t], K) * scale
            pr = torch.softmax(s, dim=-1)
            o = torch.einsum("hn,nhd->hd", pr, V)
            out[t].copy_(o.reshape(-1).to(out.dtype))

    # ---- fused forms (the compositions they stand for) ----------------------------------------
    def linear_normed(self, x, norm_w, eps, w, out, mode, ws, rows=None):
        h = torch.empty((out.shape[0], x.shape[1]), dtype=w.dtype)
        self.rmsnorm(x, norm_w, eps, h, rows=rows)
        self.linear(h, w, out, mode)

    def qkv_rope_store(self, x, norm, w_qkv, qkv, ctx, rot, cache, nq, nkv, hd, write_cache, ws):
        if norm is not None:
            h = torch.empty(x.shape, dtype=w_qkv.dtype)
            self.rmsnorm(x, norm[0], norm[1], h)
            x = h
        self.linear(x, w_qkv, qkv, "store")
        self.rope_kv_store(qkv, ctx, rot, cache, nq, nkv, hd, write_cache)

    def gather_rows(self, x, rows, out):
        out.copy_(x[rows.long()])

    # ---- BSAMPLE / BARGMAX (shaders.rs:758-850) -----------------------------------------
    def sample(self, logits, temps, seeds, out):
        from plain_llama import gumbel_sample
        for r in range(logits.shape[0]):
            out[r] = gumbel_sample(logits[r].float().cpu(), float(temps[r]), int(seeds[r]) & 0xFFFFFFFF)

    # ---- BTOPK (shaders.rs:852-905) -------------------------------------------------------
    def topk(self, logits, k, vals, idx):
        from plain_llama import topk_desc
        for r in range(logits.shape[0]):
            v, i = topk_desc(logits[r].float().cpu(), k)
            n = len(v)
            vals[r, :n] = torch.tensor(v)
            idx[r, :n] = torch.tensor(i, dtype=idx.dtype)
            if n < k:
                vals[r, n:] = -3.0e38
                idx[r, n:] = -1
