"""The kernel table: every device operation the engine performs, bound to the
hand-written CUDA kernels of ``zllm_b200/csrc``.

Each method checks on the host what the kernel relies on (device, dtype,
contiguity, sizes, capacities), picks the kernel by sizes and precision alone
-- never by trying and falling back -- and raises BackendError when a launch
reports an error.  The reference has one ``record_*`` per operation on its GPU
context (zllm src/backend/gpu/mod.rs:205-376) and can call each alone from a
test; the same holds here.

Precision: with float32 activations every product runs on CUDA cores in float32
(no tensor cores, no reduced-precision mode).  With bfloat16 activations the
products and attention use tensor-core kernels where their sizes allow and the
plain kernels otherwise; softmax, norms, rotations and the residual sum are
float32 in both.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..errors import BackendError
from . import build

MODES = {"store": 0, "add": 1, "swiglu": 2}
ERR_UNSUPPORTED = 10001


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


class CudaOps:
    decode_split_keys = 256

    def __init__(self, device="cuda:0"):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise BackendError(f"CudaOps needs a CUDA device, got {device}")
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device is available; this engine has no CPU path")
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise BackendError(f"the kernels are built for sm_100a (B200); this device is sm_{major}{minor}")
        self.dtype = torch.bfloat16
        self._libs = {}
        self._sample_scratch = None
        self._topk_scratch = None
        self._bound_stream = None
        self._tc_scratch = None
        self._kv_maps = {}
        self._error_words = None
        self.launches = 0
        self.profiling = os.environ.get("ZLLM_PROFILE", "") not in ("", "0")
        if self.profiling:
            self._profile_setup()

    # ---- device time per kind of operation, behind ZLLM_PROFILE=1 ---------------------------
    # The reference has per-section timers behind its ``profile`` feature (zllm
    # src/backend/candle/quantized_llama_fork.rs:1042-1128, printed by src/main.rs:643-658).  Here
    # every outermost operation of the kernel table is bracketed by two CUDA events on the
    # launching stream; ``take_profile()`` waits for them and returns the milliseconds per kind
    # since the last call.  Steps then run without CUDA graphs (events cannot be timed inside a
    # capture), so the shares are those of serialised launches, as a profiler would show them.
    PROFILED = ("embedding", "rmsnorm", "linear", "linear_normed", "qkv_rope_store", "rope_kv_store", "paged_attention",
                "silu_mul", "gather_rows", "sample", "topk", "pool_draw", "advance_decode", "dynamic_tanh", "softcap",
                "latent_prepare", "latent_attention", "linear_heads", "matrix_memory", "moe_route", "moe_experts",
                "rmsnorm_add", "add_bias", "bias_silu_mul", "rotate_store_kv", "window_attention")

    def _profile_setup(self):
        self._prof_depth = 0
        self._prof_events = []
        for name in self.PROFILED:
            inner = getattr(self, name)

            def timed(*a, _inner=inner, _name=name, **kw):
                if self._prof_depth > 0 or torch.cuda.is_current_stream_capturing():
                    return _inner(*a, **kw)
                kind = _name
                if _name in ("linear", "linear_normed"):
                    mode = kw.get("mode", a[3] if _name == "linear" else a[5])
                    kind = f"{_name}[{mode}]"
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                self._prof_depth += 1
                e0.record()
                try:
                    return _inner(*a, **kw)
                finally:
                    e1.record()
                    self._prof_depth -= 1
                    self._prof_events.append((kind, e0, e1))
            setattr(self, name, timed)

    def take_profile(self):
        """{kind of operation: device milliseconds} since the last call; {} unless ZLLM_PROFILE is set."""
        if not self.profiling or not self._prof_events:
            return {}
        torch.cuda.synchronize(self.device)
        out = {}
        for kind, e0, e1 in self._prof_events:
            out[kind] = out.get(kind, 0.0) + e0.elapsed_time(e1)
        self._prof_events = []
        return {k: round(v, 4) for k, v in sorted(out.items(), key=lambda kv: -kv[1])}

    # ------------------------------------------------------------------
    def configure(self, dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise BackendError(f"unsupported activation dtype {dtype}")
        self.dtype = dtype
        # What every model needs is built (in parallel) and loaded now; a part's own kernels (attention of
        # one kind or another, experts, a recurrence) when the part is bound (``prepare``) or, failing
        # that, at their first use (``lib``): a program compiles what its model needs, and no more.
        names = ["elementwise", "gemm_plain", "sampling"]
        if dtype == torch.bfloat16:
            names += ["gemm_decode", "gemm_stream", "gemm_tc"]
        # a word of pinned host memory per kernel family with bounded waits: a wait that gives up
        # writes its code there too, so the engine sees it where it synchronises anyway, without a copy
        if self._error_words is None:
            self._error_words = torch.zeros(len(self.WAIT_FAMILIES), dtype=torch.int32).pin_memory()
        self.prepare(names)
        if dtype == torch.bfloat16 and os.environ.get("ZLLM_GEMM_PAIR", "") == "0":
            # measurement switch: the many-row products on single CTAs (tiles of 128 rows) only
            self._libs["gemm_tc"].zllm_gemm_tc_force_pair(0)

    # the attention kernels of the paged key/value cache, by activation dtype
    PAGED_ATTENTION_KERNELS = {torch.float32: ("attention_plain",),
                               torch.bfloat16: ("attention_plain", "attention_bf16", "attention_decode_tma", "attention_prefill_tc")}

    def lib(self, name):
        lib = self._libs.get(name)
        if lib is None:
            lib = self._libs[name] = build.load(name)
            for i, (family, prefix) in enumerate(self.WAIT_FAMILIES):
                if family == name and self._error_words is not None:
                    code = getattr(lib, prefix + "_set_error_mirror")(c_void_p(self._error_words.data_ptr() + 4 * i))
                    if code != 0:
                        raise BackendError(f"{name}: cannot set the error mirror (CUDA error {code})")
        return lib

    def prepare(self, names):
        """Build (in parallel) and load the kernel groups a part says it will use, so that a model
        compiles what it needs when it is made and not inside its first step."""
        names = [n for n in names if n not in self._libs]
        if names:
            build.build(names)
            for n in names:
                self.lib(n)

    def _stream(self):
        if self._bound_stream is not None:
            return self._bound_stream
        return c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def bind_stream(self):
        """Look the current stream up ONCE for the launches that follow (a step issues more than a
        hundred); ``unbind_stream`` ends it.  Outside such a pair every launch asks torch."""
        self._bound_stream = c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def unbind_stream(self):
        self._bound_stream = None

    def _check(self, code, what):
        self.launches += 1
        if code != 0:
            if code == ERR_UNSUPPORTED:
                raise BackendError(f"{what}: sizes not supported by this kernel")
            raise BackendError(f"{what}: CUDA error {code}")

    def _dev(self, *tensors):
        for t in tensors:
            if t is None:
                continue
            if t.device != self.device:
                raise BackendError(f"tensor on {t.device}, kernels run on {self.device}")
            if not t.is_contiguous():
                raise BackendError("kernel operands must be contiguous")

    def decode_splits(self, max_ctx: int) -> int:
        return max(1, -(-int(max_ctx) // self.decode_split_keys))

    # ---- embedding -----------------------------------------------------
    def embedding(self, token_ids, table, out, scale: float = 1.0):
        """out[t] = table[token_ids[t]] * scale, float32."""
        self._dev(token_ids, table, out)
        T, H = out.shape
        V = table.shape[0]
        if token_ids.dtype != torch.int32 or out.dtype != torch.float32 or table.shape[1] != H \
                or token_ids.numel() != T:
            raise BackendError("embedding: bad operand types or shapes")
        code = self.lib("elementwise").zllm_embedding(_ptr(token_ids), _ptr(table), _ptr(out), c_int(T), c_int(H),
                                                      c_int(V), c_int(table.dtype == torch.bfloat16), c_float(scale),
                                                      self._stream())
        self._check(code, "embedding")

    # ---- rmsnorm -------------------------------------------------------
    def rmsnorm(self, x, weight, eps, out, rows=None):
        """out[t] = rmsnorm(x[t]), or of x[rows[t]] when an int32 index list is given."""
        self._dev(x, weight, out)
        T, H = out.shape
        if x.dtype != torch.float32 or weight.numel() != H or x.shape[1] != H or (rows is None and x.shape[0] != T) \
                or weight.dtype not in (torch.float32, torch.bfloat16) or out.dtype not in (torch.float32, torch.bfloat16):
            raise BackendError("rmsnorm: bad operand types or shapes")
        if rows is not None:
            self._dev(rows)
            if rows.dtype != torch.int32 or rows.numel() != T:
                raise BackendError("rmsnorm: the row list does not match the output")
        code = self.lib("elementwise").zllm_rmsnorm(_ptr(x), _ptr(rows), _ptr(weight), _ptr(out), c_int(T), c_int(H), c_float(eps),
                                                    c_int(weight.dtype == torch.bfloat16),
                                                    c_int(out.dtype == torch.bfloat16), self._stream())
        self._check(code, "rmsnorm")

    # ---- products ------------------------------------------------------
    def linear(self, x, w, out, mode: str):
        """out = x w^T with epilogue ``mode``: "store", "add" (into a float32 out) or "swiglu"
        (w = gate/up rows interleaved in groups of eight, out = silu(gate) * up)."""
        self._dev(x, w, out)
        M, K = x.shape
        N = out.shape[1]
        wn = w.shape[0]
        if mode not in MODES:
            raise BackendError(f"linear: unknown epilogue {mode!r}")
        if w.shape[1] != K or out.shape[0] != M or wn != (2 * N if mode == "swiglu" else N) or x.dtype != w.dtype:
            raise BackendError(f"linear: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} mode {mode}")
        if mode == "add" and out.dtype != torch.float32:
            raise BackendError("linear: the 'add' epilogue accumulates into float32")
        if x.dtype == torch.bfloat16 and self.dtype == torch.bfloat16 and self._linear_bf16(x, w, out, mode, M, N, K):
            return
        code = self.lib("gemm_plain").zllm_gemm_plain(_ptr(x), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K),
                                                      c_int(MODES[mode]), c_int(x.dtype == torch.bfloat16),
                                                      c_int(out.dtype == torch.bfloat16), self._stream())
        self._check(code, "gemm_plain")

    def linear_plain(self, x, w, out, mode: str):
        M, K = x.shape
        N = out.shape[1]
        code = self.lib("gemm_plain").zllm_gemm_plain(_ptr(x), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K),
                                                      c_int(MODES[mode]), c_int(x.dtype == torch.bfloat16),
                                                      c_int(out.dtype == torch.bfloat16), self._stream())
        self._check(code, "gemm_plain")

    # Which kernel takes a bfloat16 product is decided by the sizes alone (never by trial):
    #   rows <= 8: the fused decode product -- except for models whose matrices are large on both
    #   sides (STREAM_FEW_ROWS_MIN_SIDE: from 3B layer sizes on), whose products all go to the TMA-fed
    #   streaming product from 5 rows on, and the largest of them (K of 4096 and more) at any row
    #   count: the fused kernel streams weights through registers and reads the float32 rows again in
    #   every CTA, which costs more the longer K is (8 rows at 8B layer sizes: 5.03 against 6.75 ms a
    #   step, 1 row 3.65 against 3.94; at 3B sizes 2.81 against 3.02 at 5..8 rows and no gain below;
    #   at 1B sizes the fused kernel wins: 0.966 against 1.006 ms with gate/up streamed).  All of a
    #   model's products switch together: kernels with different shared-memory needs side by side
    #   cost more than either kind alone (3B sizes, down alone streamed: 3.12 ms);
    #   9..16: the fused product for small matrices (its fusions save
    #   kernels), the TMA-fed streaming product for matrices of STREAM_MIN_WEIGHTS elements and more;
    #   17..64: the streaming product, but matrices with STREAM_MAX_WEIGHT_ROWS rows and more (the
    #   vocabulary head) go to the many-row kernel, which re-reads x once per 256 rows, not per 128;
    #   more rows: the many-row kernel.
    STREAM_MAX_ROWS = 64
    STREAM_MIN_WEIGHTS = 12 * 1024 * 1024
    STREAM_MAX_WEIGHT_ROWS = 32768
    STREAM_FEW_ROWS_MIN_SIDE = 3072
    STREAM_ANY_ROWS_MIN_WEIGHTS = 50_000_000
    # Rotation and cache write ride in the QKV product's epilogue only when the product has tiles for
    # two waves, so that one tile's (slow, row-by-row) epilogue hides behind the next tile's MMAs:
    # measured per 16-layer step, fused against a pass of its own over qkv: 2,048 rows 4.25 / 4.29 ms,
    # 1,024 rows 3.02 / 2.93 ms, 128 rows 1.37 / 1.29 ms.
    ROPE_IN_PRODUCT_MIN_ROWS = 2048
    UNFUSE_NORM_WEIGHT_ROWS = 32768
    SAMPLE_SCRATCH_ROWS = 1024
    TC_SCRATCH_BYTES = 64 * 1024 * 1024
    DECODE_MAX_ROWS = 16
    LATENT_MMA_RANKS = (64, 128, 256, 512)      # latent sizes the tensor-core latent attention is built for
    LATENT_MAX_SPLITS = 32
    LATENT_SPLIT_KEYS = 64              # the smallest split of a decoding row's keys
    EXPERT_MMA_K = 32                   # the experts' tensor-core product steps through K in pieces of 32

    def _gemm_decode(self, x, norm_w, eps, w, out, mode, M, N, K, rope=None):
        """The fused decode product (csrc/gemm_decode.cu).  rope: (ctx, rot, cache, nq, nkv, hd, store)."""
        if rope is None:
            pos = slot = cos = sin = kp = vp = tb = None
            inter = nq = nkv = hd = mb = bs = store = 0
            code_mode = MODES[mode]
        else:
            ctx, rot, cache, nq, nkv, hd, store = rope
            pos, slot = ctx.positions, ctx.row_slot
            cos, sin = (rot.cos, rot.sin) if rot is not None else (None, None)
            inter = int(rot.interleaved) if rot is not None else 0
            if store:
                kp, vp, tb, mb, bs = cache.k_pages, cache.v_pages, cache.block_table, cache.block_table.shape[1], cache.block_size
            else:
                kp = vp = tb = None
                mb = bs = 1
            code_mode = 3
        code = self.lib("gemm_decode").zllm_gemm_decode(
            _ptr(x), _ptr(norm_w), c_int(norm_w is not None and norm_w.dtype == torch.bfloat16), c_float(eps), _ptr(w),
            _ptr(out), c_int(M), c_int(N), c_int(K), c_int(code_mode), c_int(out.dtype == torch.bfloat16), _ptr(pos),
            _ptr(slot), _ptr(cos), _ptr(sin), c_int(inter), c_int(nq), c_int(nkv), c_int(hd), _ptr(kp), _ptr(vp),
            _ptr(tb), c_int(mb), c_int(bs), c_int(1 if store else 0), self._stream())
        self._check(code, "gemm_decode")

    def _streams(self, M, w) -> bool:
        """True when a product of M rows with matrix w belongs to the streaming kernel."""
        if M <= 8 and min(w.shape[0], w.shape[1]) >= self.STREAM_FEW_ROWS_MIN_SIDE and w.shape[0] < self.STREAM_MAX_WEIGHT_ROWS \
                and (M >= 5 or (w.numel() >= self.STREAM_ANY_ROWS_MIN_WEIGHTS and w.shape[1] >= 4096)):
            return True
        if M <= 8 or M > self.STREAM_MAX_ROWS:
            return False
        if M <= self.DECODE_MAX_ROWS:
            return w.numel() >= self.STREAM_MIN_WEIGHTS
        return w.shape[0] < self.STREAM_MAX_WEIGHT_ROWS

    def _can_fuse_decode(self, x, norm_w, w, M, K) -> bool:
        return (self.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M <= self.DECODE_MAX_ROWS and K % 8 == 0
                and not self._streams(M, w)
                and (x.data_ptr() | w.data_ptr() | (norm_w.data_ptr() if norm_w is not None else 0)) & 15 == 0)

    def linear_normed(self, x, norm_w, eps, w, out, mode, ws, rows=None):
        """out = epilogue(rmsnorm(x; norm_w, eps) w^T), x the float32 residual.  One kernel for decode
        batches; otherwise the norm kernel into a scratch buffer, then the product.  ``rows`` (an
        int32 index list): the product is taken over x[rows] -- the norm kernel reads those rows
        where it stands alone, otherwise they are gathered first."""
        self._dev(x, norm_w, w, out)
        K = x.shape[1]
        M, N = out.shape
        if x.dtype != torch.float32 or norm_w.numel() != K or w.shape[1] != K or w.shape[0] != (2 * N if mode == "swiglu" else N) \
                or (rows is None and x.shape[0] != M) or (rows is not None and rows.numel() != M):
            raise BackendError("linear_normed: bad operand types or shapes")
        # The fused form has every CTA read the float32 rows of x again (4 M K bytes beside its own
        # 32 K bytes of weights per 16 rows): from a few rows on and for matrices of many rows the
        # norm as a kernel of its own and bfloat16 rows are faster (8 rows: the head 90 against 130 us,
        # gate/up 16.7 against 18.9 us; one row: 88 against 100 and 16.3 against 15.1)
        unfuse = w.shape[0] >= self.UNFUSE_NORM_WEIGHT_ROWS and M >= (1 if w.shape[0] >= self.STREAM_MAX_WEIGHT_ROWS else 4)
        fused = self._can_fuse_decode(x, norm_w, w, M, K) and not unfuse and not (mode == "swiglu" and N % 8) \
            and not (mode == "add" and out.dtype != torch.float32)
        if fused:
            if rows is not None:
                g = ws.get("normed_rows", (M, K), torch.float32)
                self.gather_rows(x, rows, g)
                x = g
            self._gemm_decode(x, norm_w, eps, w, out, mode, M, N, K)
            return
        h = ws.get("normed", (M, K), self.dtype)
        self.rmsnorm(x, norm_w, eps, h, rows=rows)
        self.linear(h, w, out, mode)

    def qkv_rope_store(self, x, norm, w_qkv, qkv, ctx, rot, cache, nq, nkv, hd, write_cache, ws):
        """qkv = [rmsnorm](x) w_qkv^T, q and k rotated, k and v written to their cache pages.
        ``norm`` is (weight, eps) when x is the float32 residual, None when x is already normed."""
        self._dev(x, w_qkv, qkv)
        M, K = x.shape
        N = (nq + 2 * nkv) * hd
        if tuple(qkv.shape) != (M, N) or tuple(w_qkv.shape) != (N, K):
            raise BackendError("qkv_rope_store: shapes do not match the head counts")
        norm_w, eps = norm if norm is not None else (None, 0.0)
        fused = (self._can_fuse_decode(x, norm_w, w_qkv, M, K) and qkv.dtype == torch.bfloat16 and hd % 16 == 0
                 and (rot is None or rot.rot_dim == hd) and (norm is None or x.dtype == torch.float32)
                 and (norm is not None or x.dtype == torch.bfloat16))
        if fused:
            if write_cache:
                self._check_cache(cache, nkv, hd, qkv.dtype, "qkv_rope_store")
            self._gemm_decode(x, norm_w, eps, w_qkv, qkv, "store", M, N, K,
                              rope=(ctx, rot, cache, nq, nkv, hd, bool(write_cache)))
            return
        if norm is not None:
            h = ws.get("normed", (M, K), self.dtype)
            self.rmsnorm(x, norm_w, eps, h)
            x = h
        # many rows: rotation and cache write in the epilogue of the tensor-core product (head sizes
        # 64 and 128, half-split pairs over the whole head); otherwise a pass of their own over qkv
        if M >= self.ROPE_IN_PRODUCT_MIN_ROWS and self.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and qkv.dtype == torch.bfloat16 \
                and w_qkv.dtype == torch.bfloat16 and hd in (64, 128) and K % 8 == 0 \
                and (rot is None or (rot.rot_dim == hd and not rot.interleaved)) \
                and (x.data_ptr() | w_qkv.data_ptr() | qkv.data_ptr()) & 15 == 0:
            self._dev(ctx.positions, ctx.row_slot)
            if ctx.positions.numel() != M or ctx.row_slot.numel() != M:
                raise BackendError("qkv_rope_store: the step's rows do not match qkv")
            if write_cache:
                self._check_cache(cache, nkv, hd, qkv.dtype, "qkv_rope_store")
                kp, vp, tb, mb, bs = cache.k_pages, cache.v_pages, cache.block_table, cache.block_table.shape[1], cache.block_size
            else:
                kp = vp = tb = None
                mb = bs = 1
            code = self.lib("gemm_tc").zllm_gemm_tc_qkv_rope(
                _ptr(x), _ptr(w_qkv), _ptr(qkv), c_int(M), c_int(K), _ptr(ctx.positions), _ptr(ctx.row_slot),
                _ptr(rot.cos if rot is not None else None), _ptr(rot.sin if rot is not None else None), c_int(nq), c_int(nkv),
                c_int(hd), _ptr(kp), _ptr(vp), _ptr(tb), c_int(mb), c_int(bs), c_int(1 if write_cache else 0), self._stream())
            self._check(code, "gemm_tc_qkv_rope")
            return
        self.linear(x, w_qkv, qkv, "store")
        self.rope_kv_store(qkv, ctx, rot, cache, nq, nkv, hd, write_cache)

    def _linear_bf16(self, x, w, out, mode, M, N, K) -> bool:
        """Tensor-core products for bfloat16 operands; False: these sizes go to the plain kernel.
        The choice depends on the sizes only."""
        if K % 8 or (mode == "swiglu" and N % 8) or (x.data_ptr() | w.data_ptr()) & 15:
            return False
        tc_ok = N % 8 == 0 and out.data_ptr() % 16 == 0
        if self._streams(M, w) or (M <= self.STREAM_MAX_ROWS and M > self.DECODE_MAX_ROWS and not tc_ok):
            code = self.lib("gemm_stream").zllm_gemm_stream_bf16(_ptr(x), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K),
                                                                 c_int(MODES[mode]), c_int(out.dtype == torch.bfloat16),
                                                                 self._stream())
            self._check(code, "gemm_stream_bf16")
            return True
        if M <= self.DECODE_MAX_ROWS:
            self._gemm_decode(x, None, 0.0, w, out, mode, M, N, K)
            return True
        if tc_ok:
            if self._tc_scratch is None:     # float32 partial tiles of products whose K is split (few tiles)
                self._tc_scratch = torch.empty(self.TC_SCRATCH_BYTES // 4, dtype=torch.float32, device=self.device)
            code = self.lib("gemm_tc").zllm_gemm_tc_bf16(_ptr(x), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K),
                                                         c_int(MODES[mode]), c_int(out.dtype == torch.bfloat16),
                                                         _ptr(self._tc_scratch), c_longlong(self.TC_SCRATCH_BYTES),
                                                         self._stream())
            self._check(code, "gemm_tc_bf16")
            return True
        return False

    WAIT_FAMILIES = (("gemm_tc", "zllm_gemm_tc"), ("gemm_stream", "zllm_gemm_stream"),
                     ("attention_decode_tma", "zllm_attention_decode_tma"),
                     ("attention_prefill_tc", "zllm_attention_prefill_tc"))

    def check_async_errors(self):
        """Raise if a kernel's bounded wait gave up since the last call (synchronises the device)."""
        found = None
        for i, (name, prefix) in enumerate(self.WAIT_FAMILIES):
            lib = self._libs.get(name)
            if lib is not None:
                v = getattr(lib, prefix + "_error")()
                if v != 0 and found is None:
                    found = (name, v)
        if self._error_words is not None:
            self._error_words.zero_()
        if found is not None:
            raise BackendError(f"{found[0]}: a bounded wait ran out (code {found[1]}); results of that launch are invalid")

    def raise_if_a_wait_gave_up(self):
        """The same check without touching the device: reads the pinned words the kernels mirror
        their error codes into.  For the places where the engine has just synchronised."""
        w = self._error_words
        if w is not None and bool(w.any()):
            self.check_async_errors()                    # names the kernel, clears the flags, raises
            raise BackendError("a bounded wait ran out; results of that launch are invalid")

    def set_wait_test_hook(self, family: str, limit: int = 0, skip_loads: bool = False):
        """Tests: lower a kernel family's wait limit to ``limit`` polls (0: the default) and, with
        ``skip_loads``, make its producer issue no copy, so that its waits for data run out with
        nothing in flight and the kernel's give-up path runs."""
        prefix = dict(self.WAIT_FAMILIES)[family]
        code = getattr(self.lib(family), prefix + "_test_hook")(ctypes.c_uint(limit), c_int(1 if skip_loads else 0))
        if code != 0:
            raise BackendError(f"{family}: test hook failed (CUDA error {code})")

    # ---- dynamic tanh, soft cap ------------------------------------------
    def dynamic_tanh(self, x, alpha, weight, bias, out):
        """out = tanh(alpha x) * weight + bias; x float32, alpha a one-element float32 tensor."""
        self._dev(x, alpha, weight, bias, out)
        T, H = out.shape
        if x.dtype != torch.float32 or tuple(x.shape) != (T, H) or weight.numel() != H or bias.numel() != H \
                or alpha.numel() != 1 or any(t.dtype != torch.float32 for t in (alpha, weight, bias)) \
                or out.dtype not in (torch.float32, torch.bfloat16):
            raise BackendError("dynamic_tanh: bad operand types or shapes")
        code = self.lib("elementwise").zllm_dynamic_tanh(_ptr(x), _ptr(alpha), _ptr(weight), _ptr(bias), _ptr(out), c_int(T),
                                                         c_int(H), c_int(out.dtype == torch.bfloat16), self._stream())
        self._check(code, "dynamic_tanh")

    def softcap(self, x, cap: float):
        """x <- cap tanh(x / cap) in place (float32)."""
        self._dev(x)
        if x.dtype != torch.float32 or not cap > 0:
            raise BackendError("softcap: float32 values and a positive cap")
        code = self.lib("elementwise").zllm_softcap(_ptr(x), c_longlong(x.numel()), c_float(cap), self._stream())
        self._check(code, "softcap")

    # ---- attention through a latent ----------------------------------------
    def _check_latent_cache(self, cache, width, dtype, what):
        self._dev(cache.k_pages, cache.block_table)
        if cache.k_pages.dtype != dtype or tuple(cache.k_pages.shape[1:]) != (1, cache.block_size, width) \
                or cache.block_table.dtype != torch.int32:
            raise BackendError(f"{what}: cache pages {tuple(cache.k_pages.shape)} {cache.k_pages.dtype} do not match "
                               f"rows of {width} entries, block {cache.block_size}, {dtype}")

    def latent_prepare(self, proj, off_q, q_rank, off_kv, rank, rot, wq, wc, eps, freqs, cq, ctx, cache, write_cache=True):
        """From the stacked down-projections ``proj``: cq = rmsnorm(query latent) * wq; the row's
        cache entry [rmsnorm(latent) * wc | rotated key part] written to its page.
        freqs = (frequencies [dims/2] float32 on the device, magnitude, dims)."""
        self._dev(proj, wq, wc, freqs[0], cq, ctx.positions, ctx.row_slot)
        T = proj.shape[0]
        if cq.dtype != proj.dtype or tuple(cq.shape) != (T, q_rank) or wq.numel() != q_rank or wc.numel() != rank \
                or max(off_q + q_rank, off_kv + rank + rot) > proj.shape[1] or freqs[0].numel() * 2 != freqs[2] \
                or ctx.positions.numel() != T:
            raise BackendError("latent_prepare: bad operand types or shapes")
        if write_cache:
            self._check_latent_cache(cache, rank + rot, proj.dtype, "latent_prepare")
        code = self.lib("latent_attention").zllm_latent_prepare(
            _ptr(proj), c_int(proj.shape[1]), c_int(off_q), c_int(q_rank), c_int(off_kv), c_int(rank), c_int(rot), _ptr(wq),
            _ptr(wc), c_float(eps), _ptr(freqs[0]), c_float(freqs[1]), c_int(freqs[2]), _ptr(ctx.positions),
            _ptr(ctx.row_slot), _ptr(cq), _ptr(cache.k_pages if write_cache else None),
            _ptr(cache.block_table if write_cache else None), c_int(cache.block_table.shape[1] if write_cache else 1),
            c_int(cache.block_size if write_cache else 1), c_int(1 if write_cache else 0), c_int(T),
            c_int(proj.dtype == torch.bfloat16), self._stream())
        self._check(code, "latent_prepare")

    def latent_attention(self, q_lat, q, q_off, out, ctx, cache, n_heads, rank, rot, freqs, scale):
        """out[t, h] = sum_j softmax_j(scale (q_lat[t, h] . c_j + rotated(q[t, h, -rot:]) . kr_j)) c_j over
        the cached positions j <= the row's own, [c_j | kr_j] being the cache rows."""
        self._dev(q_lat, q, out, ctx.positions, ctx.row_slot)
        T = q.shape[0]
        if q_lat.dtype != torch.float32 or tuple(q_lat.shape) != (T, n_heads * rank) or tuple(out.shape) != (T, n_heads * rank) \
                or out.dtype != q.dtype or q.shape[1] != n_heads * q_off:
            raise BackendError("latent_attention: bad operand types or shapes")
        self._check_latent_cache(cache, rank + rot, q.dtype, "latent_attention")
        if q.dtype == torch.bfloat16 and rank in self.LATENT_MMA_RANKS and rot % 16 == 0:
            # tensor cores: the heads are the rows of the tile.  A step of single tokens only (decoding) has
            # few rows: their keys are divided into splits of a multiple of 256 that a second kernel merges
            n_splits, split_keys = 1, 0
            if ctx.n_decode == T:
                # the framework's split count (in pieces of decode_split_keys, a power of two inside graphs) bounds
                # the context; the latent kernel cuts it finer, into at most LATENT_MAX_SPLITS splits of whole key blocks
                reach = (ctx.fixed_splits or self.decode_splits(ctx.max_context)) * self.decode_split_keys
                n_splits = max(1, min(self.LATENT_MAX_SPLITS, reach // self.LATENT_SPLIT_KEYS))
                split_keys = -(-(-(-reach // n_splits)) // 32) * 32
            part_o = part_ml = None
            if n_splits > 1:
                part_o = ctx.ws.get("latent_part_o", (T, n_heads * self.LATENT_MAX_SPLITS * rank), torch.float32, cap=T)
                part_ml = ctx.ws.get("latent_part_ml", (T, n_heads * self.LATENT_MAX_SPLITS * 2), torch.float32, cap=T)
            code = self.lib("latent_attention_mma").zllm_latent_attention_mma(
                _ptr(q_lat), _ptr(q), c_int(q.shape[1]), c_int(q_off), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(ctx.positions),
                _ptr(ctx.row_slot), _ptr(cache.k_pages), _ptr(cache.block_table), c_int(cache.block_table.shape[1]),
                c_int(cache.block_size), c_int(T), c_int(n_heads), c_int(rank), c_int(rot), _ptr(freqs[0]), c_float(freqs[1]),
                c_int(freqs[2]), c_float(scale), c_int(n_splits), c_int(split_keys), self._stream())
            self._check(code, "latent_attention_mma")
            return
        code = self.lib("latent_attention").zllm_latent_attention(
            _ptr(q_lat), _ptr(q), c_int(q.shape[1]), c_int(q_off), _ptr(out), _ptr(ctx.positions), _ptr(ctx.row_slot),
            _ptr(cache.k_pages), _ptr(cache.block_table), c_int(cache.block_table.shape[1]), c_int(cache.block_size), c_int(T),
            c_int(n_heads), c_int(rank), c_int(rot), _ptr(freqs[0]), c_float(freqs[1]), c_int(freqs[2]), c_float(scale),
            c_int(q.dtype == torch.bfloat16), self._stream())
        self._check(code, "latent_attention")

    def linear_heads(self, x, x_head_stride, w, out, gate=None, out_scale: float = 1.0):
        """Per head g: out[:, g*N:(g+1)*N] = x[:, g*stride : g*stride + K] w[g]^T with w [G, N, K];
        with ``gate`` = (tensor [T, >= c + G*N], first column c) the result is multiplied by
        sigmoid(gate) * out_scale."""
        self._dev(x, w, out, gate[0] if gate is not None else None)
        G, N, K = w.shape
        T = x.shape[0]
        gptr, ldg = c_void_p(0), 0
        if gate is not None:
            gt, c0 = gate
            if gt.dtype != x.dtype or gt.shape[0] != T or c0 < 0 or c0 + G * N > gt.shape[1]:
                raise BackendError("linear_heads: the gate does not match the output")
            gptr, ldg = c_void_p(gt.data_ptr() + c0 * gt.element_size()), gt.shape[1]
        if tuple(out.shape) != (T, G * N) or (G - 1) * x_head_stride + K > x.shape[1] \
                or x.dtype not in (w.dtype, torch.float32) or out.dtype not in (w.dtype, torch.float32):
            raise BackendError("linear_heads: bad operand types or shapes")
        if w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and K % self.EXPERT_MMA_K == 0 and x.shape[1] % 8 == 0 \
                and x_head_stride % 8 == 0 and (x.data_ptr() | w.data_ptr()) & 15 == 0:
            code = self.lib("gemm_grouped_mma").zllm_gemm_heads_mma(
                _ptr(x), c_int(x.shape[1]), c_int(x_head_stride), _ptr(w), _ptr(out), gptr, c_int(ldg), c_float(out_scale), c_int(T),
                c_int(N), c_int(K), c_int(G), c_int(out.dtype == torch.float32), self._stream())
            self._check(code, "gemm_heads_mma")
            return
        code = self.lib("gemm_grouped").zllm_gemm_heads(
            _ptr(x), c_int(x.shape[1]), c_int(x_head_stride), _ptr(w), _ptr(out), gptr, c_int(ldg), c_float(out_scale), c_int(T),
            c_int(N), c_int(K), c_int(G), c_int(w.dtype == torch.bfloat16), c_int(x.dtype == torch.float32),
            c_int(out.dtype == torch.float32), self._stream())
        self._check(code, "gemm_heads")

    # ---- matrix memory (mLSTM) -----------------------------------------------
    @staticmethod
    def plan_row_segments(entries, starts, aux, bucketed=False):
        """A step planner for mixers with per-request state: every entry's run of rows as
        [first row, rows, slot, position of the first row].  ``bucketed``: the list is rounded up
        to a power of two with empty segments, which the kernels skip."""
        n_real = len(entries)
        n = n_real
        if bucketed:
            n = 1
            while n < n_real:
                n *= 2
        host, off = aux.take(4 * n)
        host[4 * n_real:4 * n] = (0, 0, -1, 0) * (n - n_real)
        r = 0
        for i, (e, start) in enumerate(zip(entries, starts)):
            m = len(e.tokens)
            host[4 * i:4 * i + 4] = (r, m, e.slot, start)
            r += m
        return {"row_segments": (off, (n, 4))}

    def matrix_memory(self, qkvg, oq, ok, ov, og, z, bias_i, bias_f, cap, norm_w, eps, mult, out, ctx, cache, H, dk, dv):
        """The mLSTM recurrence over the step's rows, request by request, from and into the state
        slots; out [T, H*dv] = unit-RMS(per head) * norm_w * sigmoid(gate) * mult."""
        self._dev(qkvg, z, bias_i, bias_f, norm_w, out, ctx.row_slot, cache.state)
        T = qkvg.shape[0]
        st = cache.state
        per_slot = H * (dk * dv + dk + 1)
        if z.dtype != torch.float32 or tuple(z.shape) != (T, 2 * H) or st.dtype != torch.float32 \
                or st.shape[1] != per_slot or tuple(out.shape) != (T, H * dv) or out.dtype != qkvg.dtype \
                or norm_w.numel() != H * dv or any(t.dtype != torch.float32 for t in (bias_i, bias_f, norm_w)):
            raise BackendError("matrix_memory: bad operand types or shapes")
        segs = ctx.aux.get("row_segments") if ctx.aux else None
        fac = ctx.ws.get("mlstm_factors", (T, H * 4), torch.float32)
        raw = ctx.ws.get("mlstm_raw", (T, H * dv), torch.float32)
        code = self.lib("mlstm").zllm_mlstm(
            _ptr(qkvg), c_int(qkvg.shape[1]), c_int(oq), c_int(ok), c_int(ov), c_int(og), _ptr(z), _ptr(bias_i), _ptr(bias_f),
            c_float(cap), _ptr(norm_w), c_float(eps), c_float(mult), _ptr(segs), c_int(segs.shape[0] if segs is not None else 0),
            _ptr(ctx.row_slot), _ptr(st), c_longlong(per_slot), _ptr(fac), _ptr(raw), _ptr(out), c_int(T), c_int(H),
            c_int(dk), c_int(dv), c_int(qkvg.dtype == torch.bfloat16), self._stream())
        self._check(code, "mlstm")
        self.launches += 2

    # ---- mixture of experts ------------------------------------------------------
    EXPERT_ACTIVATIONS = {"silu": 0, "gelu": 1, "gelu_tanh": 2}

    def moe_route(self, h, w_router, top, groups, keep, idx, weights, score: str = "softmax", normalise: bool = True,
                  n_shared: int = 0, shared_gate: bool = False):
        """Per row: router scores (softmax over the experts, or a sigmoid each), the ``top`` experts among
        the ``keep`` best of ``groups`` groups, their weights (divided by their sum if ``normalise``).
        Behind them ``n_shared`` choices that every row has, the experts E, E+1, ..., with the weight 1 or,
        with ``shared_gate`` (the router matrix then has a row E for it), sigmoid of that row's logit."""
        self._dev(h, w_router, idx, weights)
        T, H = h.shape
        E = w_router.shape[0] - (1 if shared_gate else 0)
        cols = top + n_shared
        if w_router.shape[1] != H or w_router.dtype != h.dtype or idx.dtype != torch.int32 or weights.dtype != torch.float32 \
                or tuple(idx.shape) != (T, cols) or tuple(weights.shape) != (T, cols) or score not in ("softmax", "sigmoid"):
            raise BackendError("moe_route: bad operand types or shapes")
        code = self.lib("moe").zllm_moe_route(_ptr(h), _ptr(w_router), _ptr(idx), _ptr(weights), c_int(T), c_int(H), c_int(E),
                                              c_int(top), c_int(groups), c_int(keep), c_int(score == "sigmoid"),
                                              c_int(1 if normalise else 0), c_int(n_shared), c_int(1 if shared_gate else 0),
                                              c_int(h.dtype == torch.bfloat16), self._stream())
        self._check(code, "moe_route")

    def moe_experts(self, h, idx, weights, w_gate, w_up, w_down, residual, scale, ws, n_input_weighted: int = 0,
                    activation: str = "silu", accumulate: bool = True):
        """residual[t] (+)= scale * sum_j a_j * expert_{idx[t, j]}(b_j h[t]).  An expert is
        down(silu(gate x) * (up x)), or down(f(up x)) when ``w_gate`` is None (f = ``activation``).
        The first ``n_input_weighted`` choices of a row carry their weight on the expert's input
        (b_j = weights[t, j], a_j = 1), the others on its output (a_j = weights[t, j], b_j = 1).
        w_gate, w_up [E, F, H], w_down [E, H, F]."""
        self._dev(h, idx, weights, w_gate, w_up, w_down, residual)
        T, H = h.shape
        top = idx.shape[1]
        E, F, _ = w_up.shape
        if (w_gate is not None and tuple(w_gate.shape) != (E, F, H)) or tuple(w_up.shape) != (E, F, H) \
                or tuple(w_down.shape) != (E, H, F) or residual.dtype != torch.float32 or tuple(residual.shape) != (T, H) \
                or any(t is not None and t.dtype != h.dtype for t in (w_gate, w_up, w_down)) \
                or activation not in self.EXPERT_ACTIVATIONS or not 0 <= n_input_weighted <= top \
                or tuple(weights.shape) != (T, top) or weights.dtype != torch.float32:
            raise BackendError("moe_experts: bad operand types or shapes")
        n = T * top
        off = ws.get("moe_offsets", (1, E + 1), torch.int32, cap=1)
        perm = ws.get("moe_perm", (T, top), torch.int32)
        act = ws.get("moe_act", (n, F), h.dtype, cap=ws.max_rows * top)
        y = ws.get("moe_out", (n, H), torch.float32, cap=ws.max_rows * top)
        moe = self.lib("moe")
        is_bf16 = h.dtype == torch.bfloat16
        self._check(moe.zllm_moe_sort(_ptr(idx), _ptr(off), _ptr(perm), c_int(n), c_int(E), self._stream()), "moe_sort")
        first_mode = 1 if w_gate is not None else 2
        first = (w_gate, w_up) if w_gate is not None else (w_up, None)
        rs = weights if n_input_weighted > 0 else None
        act_code = self.EXPERT_ACTIVATIONS[activation]
        # each product goes to the tensor-core kernel when its K allows (bfloat16, K a multiple of 32),
        # else to the CUDA-core kernel: decided by the sizes alone
        for x_in, w_a, w_b, dst, N, K, mode, scale_rows in ((h, first[0], first[1], act, F, H, first_mode, rs),
                                                            (act, w_down, None, y, H, F, 0, None)):
            if is_bf16 and K % self.EXPERT_MMA_K == 0 and (x_in.data_ptr() | w_a.data_ptr() | (w_b.data_ptr() if w_b is not None else 0)) & 15 == 0:
                code = self.lib("gemm_grouped_mma").zllm_gemm_experts_mma(
                    _ptr(x_in), _ptr(w_a), _ptr(w_b), _ptr(dst), _ptr(off), _ptr(perm), c_int(top), c_int(n), c_int(E), c_int(N),
                    c_int(K), c_int(mode), _ptr(scale_rows), c_int(n_input_weighted), c_int(act_code), self._stream())
                self._check(code, "gemm_experts_mma")
            else:
                code = self.lib("gemm_grouped").zllm_gemm_experts(
                    _ptr(x_in), _ptr(w_a), _ptr(w_b), _ptr(dst), _ptr(off), _ptr(perm), c_int(top), c_int(n), c_int(E), c_int(N),
                    c_int(K), c_int(mode), _ptr(scale_rows), c_int(n_input_weighted), c_int(act_code), c_int(is_bf16),
                    self._stream())
                self._check(code, "gemm_experts")
        self._check(moe.zllm_moe_combine(_ptr(y), _ptr(weights), _ptr(residual), c_int(T), c_int(H), c_int(top),
                                         c_float(scale), c_int(n_input_weighted), c_int(0 if accumulate else 1), self._stream()),
                    "moe_combine")

    # ---- silu * up -----------------------------------------------------
    def silu_mul(self, a, b, out):
        self._dev(a, b, out)
        if a.shape != b.shape or a.shape != out.shape or a.dtype != b.dtype or a.dtype != out.dtype:
            raise BackendError("silu_mul: operands differ in shape or dtype")
        code = self.lib("elementwise").zllm_silu_mul(_ptr(a), _ptr(b), _ptr(out), c_longlong(a.numel()),
                                                     c_int(a.dtype == torch.bfloat16), self._stream())
        self._check(code, "silu_mul")

    # ---- rows of the float32 residual ----------------------------------
    def gather_rows(self, x, rows, out):
        self._dev(x, rows, out)
        R, H = out.shape
        if x.dtype != torch.float32 or out.dtype != torch.float32 or rows.dtype != torch.int32 or rows.numel() != R \
                or x.shape[1] != H:
            raise BackendError("gather_rows: bad operand types or shapes")
        code = self.lib("elementwise").zllm_gather_rows(_ptr(x), _ptr(rows), _ptr(out), c_int(R), c_int(H),
                                                        self._stream())
        self._check(code, "gather_rows")

    # ---- a branch's output norm, biases ------------------------------------------------
    def rmsnorm_add(self, y, bias, weight, eps, residual):
        """residual += rmsnorm(y + bias) * weight, float32; ``bias`` may be None."""
        self._dev(y, bias, weight, residual)
        T, H = residual.shape
        if y.dtype != torch.float32 or residual.dtype != torch.float32 or tuple(y.shape) != (T, H) or weight.numel() != H \
                or weight.dtype not in (torch.float32, torch.bfloat16) \
                or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != H)):
            raise BackendError("rmsnorm_add: bad operand types or shapes")
        code = self.lib("elementwise").zllm_rmsnorm_add(_ptr(y), _ptr(bias), _ptr(weight), _ptr(residual), c_int(T), c_int(H),
                                                        c_float(eps), c_int(weight.dtype == torch.bfloat16), self._stream())
        self._check(code, "rmsnorm_add")

    def add_bias(self, x, bias):
        """x[t] += bias, float32."""
        self._dev(x, bias)
        if x.dtype != torch.float32 or bias.dtype != torch.float32 or bias.numel() != x.shape[1]:
            raise BackendError("add_bias: bad operand types or shapes")
        code = self.lib("elementwise").zllm_add_bias(_ptr(x), _ptr(bias), c_int(x.shape[0]), c_int(x.shape[1]), self._stream())
        self._check(code, "add_bias")

    def bias_silu_mul(self, gu, bias, out):
        """out = silu(gu[:, :I] + bias[:I]) * (gu[:, I:2I] + bias[I:]); gu [T, >= 2I], bias float32 [2I]."""
        self._dev(gu, bias, out)
        T, I = out.shape
        if gu.dtype != out.dtype or gu.shape[0] != T or gu.shape[1] < 2 * I or bias.dtype != torch.float32 or bias.numel() != 2 * I:
            raise BackendError("bias_silu_mul: bad operand types or shapes")
        code = self.lib("elementwise").zllm_bias_silu_mul(_ptr(gu), c_int(gu.shape[1]), _ptr(bias), _ptr(out), c_int(T), c_int(I),
                                                          c_int(gu.dtype == torch.bfloat16), self._stream())
        self._check(code, "bias_silu_mul")

    # ---- attention with a window that keeps the first positions ----------------------------
    def _check_window_cache(self, cache, nkv, dk, dv, dtype, what):
        kp, vp = cache.k_pages, cache.v_pages
        self._dev(kp, vp, cache.block_table)
        if kp.dtype != dtype or vp.dtype != dtype or tuple(kp.shape[1:]) != (nkv, cache.block_size, dk) \
                or tuple(vp.shape[1:]) != (nkv, cache.block_size, dv) or vp.shape[0] != kp.shape[0] \
                or cache.block_table.dtype != torch.int32:
            raise BackendError(f"{what}: cache pages {tuple(kp.shape)} / {tuple(vp.shape)} {kp.dtype} do not match "
                               f"(kv heads {nkv}, block {cache.block_size}, key size {dk}, value size {dv}, {dtype})")

    def rotate_store_kv(self, proj, off_k, off_v, ctx, freqs, cache, nq, nkv, dk, dv, write_cache=True):
        """The queries (columns 0..) and keys (from ``off_k``) of ``proj`` rotated in place over their first
        ``freqs.dims`` entries by position * frequency; keys and values (from ``off_v``) written to their pages.
        ``freqs``: a ``RotaryFrequencies`` (frequencies on the device, magnitude, dims, pairing) or None."""
        self._dev(proj, ctx.positions, ctx.row_slot)
        T, ld = proj.shape
        if ctx.positions.numel() != T or ctx.row_slot.numel() != T or off_v + nkv * dv > ld:
            raise BackendError("rotate_store_kv: the projection does not match the head counts or the step's rows")
        if freqs is not None:
            self._dev(freqs.freq)
            if freqs.freq.dtype != torch.float32 or freqs.freq.numel() * 2 != freqs.dims or freqs.dims > dk:
                raise BackendError("rotate_store_kv: the frequencies do not match the rotated entries")
        if write_cache:
            self._check_window_cache(cache, nkv, dk, dv, proj.dtype, "rotate_store_kv")
            kp, vp, tb, mb, bs = cache.k_pages, cache.v_pages, cache.block_table, cache.block_table.shape[1], cache.block_size
        else:
            kp = vp = tb = None
            mb, bs = 1, 1
        code = self.lib("attention_window").zllm_rotate_store_kv(
            _ptr(proj), c_int(ld), c_int(off_k), c_int(off_v), _ptr(ctx.positions), _ptr(ctx.row_slot),
            _ptr(freqs.freq if freqs is not None else None), c_float(freqs.magnitude if freqs is not None else 1.0),
            c_int(freqs.dims if freqs is not None else 0), c_int(int(freqs.interleaved) if freqs is not None else 0),
            _ptr(kp), _ptr(vp), _ptr(tb), c_int(mb), c_int(bs), c_int(T), c_int(nq), c_int(nkv), c_int(dk), c_int(dv),
            c_int(1 if write_cache else 0), c_int(proj.dtype == torch.bfloat16), self._stream())
        self._check(code, "rotate_store_kv")

    def window_attention(self, proj, off_g, out, ctx, cache, nq, nkv, dk, dv, scale, window, keep_first):
        """out[t, a] = sigmoid(gate)(t, a) * sum_j softmax_j(scale q(t, a) . k_j) v_j over the keys j <= the row's
        position with (position - j < window or j < keep_first); ``window`` None: all of them; ``off_g`` < 0:
        no gates.  Queries at the front of ``proj``, gate logits at column ``off_g``."""
        self._dev(proj, out, ctx.positions, ctx.row_slot)
        T, ld = proj.shape
        self._check_window_cache(cache, nkv, dk, dv, proj.dtype, "window_attention")
        if tuple(out.shape) != (T, nq * dv) or out.dtype != proj.dtype or nq * dk > ld:
            raise BackendError("window_attention: output does not match")
        G = nq // nkv
        if proj.dtype == torch.bfloat16 and self.dtype == torch.bfloat16 and dk % 16 == 0 and dv % 16 == 0 and max(dk, dv) <= 128 \
                and G <= 16 and scale > 0 and ld % 8 == 0 and (proj.data_ptr() | out.data_ptr()) & 15 == 0 \
                and os.environ.get("ZLLM_WINDOW_ATTENTION_PLAIN", "") in ("", "0"):
            # tensor cores: decoded rows with the group's heads as the tile's rows, portions by query tiles
            tiles = ctx.aux.get("query_tiles") if ctx.aux else None
            n_tiles = tiles.shape[0] if tiles is not None else 0
            code = self.lib("attention_window").zllm_window_attention_bf16(
                _ptr(proj), c_int(ld), c_int(off_g), _ptr(out), _ptr(ctx.decode_rows), c_int(ctx.n_decode), _ptr(tiles),
                c_int(n_tiles), _ptr(ctx.positions), _ptr(ctx.row_slot), _ptr(cache.k_pages), _ptr(cache.v_pages),
                _ptr(cache.block_table), c_int(cache.block_table.shape[1]), c_int(cache.block_size), c_int(nq), c_int(nkv),
                c_int(dk), c_int(dv), c_float(scale), c_int(window or 0), c_int(keep_first or 0), self._stream())
            self._check(code, "window_attention_bf16")
            if ctx.n_decode > 0 and n_tiles > 0:
                self.launches += 1
            return
        code = self.lib("attention_window").zllm_window_attention_plain(
            _ptr(proj), c_int(ld), c_int(off_g), _ptr(out), _ptr(ctx.positions), _ptr(ctx.row_slot), _ptr(cache.k_pages),
            _ptr(cache.v_pages), _ptr(cache.block_table), c_int(cache.block_table.shape[1]), c_int(cache.block_size), c_int(T),
            c_int(nq), c_int(nkv), c_int(dk), c_int(dv), c_float(scale), c_int(window or 0), c_int(keep_first or 0),
            c_int(proj.dtype == torch.bfloat16), self._stream())
        self._check(code, "window_attention_plain")

    # ---- rotary + cache write ------------------------------------------
    def _check_cache(self, cache, nkv, hd, dtype, what):
        kp, vp = cache.k_pages, cache.v_pages
        self._dev(kp, vp, cache.block_table)
        if kp.dtype != dtype or tuple(kp.shape[1:]) != (nkv, cache.block_size, hd) or kp.shape != vp.shape \
                or cache.block_table.dtype != torch.int32:
            raise BackendError(f"{what}: cache pages {tuple(kp.shape)} {kp.dtype} do not match "
                               f"(kv heads {nkv}, block {cache.block_size}, head_dim {hd}, {dtype})")

    def rope_kv_store(self, qkv, ctx, rot, cache, nq, nkv, hd, write_cache=True):
        self._dev(qkv, ctx.positions, ctx.row_slot)
        T = qkv.shape[0]
        if qkv.shape[1] != (nq + 2 * nkv) * hd or ctx.positions.numel() != T or ctx.row_slot.numel() != T:
            raise BackendError("rope_kv_store: qkv does not match the head counts or the step's rows")
        if rot is not None:
            self._dev(rot.cos, rot.sin)
            if rot.cos.dtype != torch.float32 or rot.cos.shape[1] * 2 != rot.rot_dim or rot.rot_dim > hd:
                raise BackendError("rope_kv_store: rotary tables do not match rot_dim")
        if write_cache:
            self._check_cache(cache, nkv, hd, qkv.dtype, "rope_kv_store")
            kp, vp, tb, mb, bs = cache.k_pages, cache.v_pages, cache.block_table, cache.block_table.shape[1], cache.block_size
        else:
            kp = vp = tb = None
            mb, bs = 1, 1
        code = self.lib("elementwise").zllm_rope_kv_store(
            _ptr(qkv), _ptr(ctx.positions), _ptr(ctx.row_slot), _ptr(rot.cos if rot is not None else None),
            _ptr(rot.sin if rot is not None else None), c_int(rot.rot_dim if rot is not None else 0),
            c_int(int(rot.interleaved) if rot is not None else 0), _ptr(kp), _ptr(vp), _ptr(tb), c_int(mb), c_int(bs),
            c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_int(1 if write_cache else 0),
            c_int(qkv.dtype == torch.bfloat16), self._stream())
        self._check(code, "rope_kv_store")

    # ---- attention over the cache ----------------------------------------
    def paged_attention(self, qkv, out, ctx, cache, nq, nkv, hd, scale, window):
        self._dev(qkv, out, ctx.positions, ctx.row_slot)
        T = qkv.shape[0]
        self._check_cache(cache, nkv, hd, qkv.dtype, "paged_attention")
        if tuple(out.shape) != (T, nq * hd) or out.dtype != qkv.dtype:
            raise BackendError("paged_attention: output does not match")
        if qkv.dtype == torch.bfloat16 and self.dtype == torch.bfloat16 and \
                self._attention_bf16(qkv, out, ctx, cache, nq, nkv, hd, scale, window):
            return
        self.attention_plain(qkv, out, ctx.positions, ctx.row_slot, cache, nq, nkv, hd, scale, window)

    def attention_plain(self, qkv, out, positions, row_slot, cache, nq, nkv, hd, scale, window):
        T = qkv.shape[0]
        code = self.lib("attention_plain").zllm_attention_plain(
            _ptr(qkv), _ptr(out), _ptr(positions), _ptr(row_slot), _ptr(cache.k_pages), _ptr(cache.v_pages),
            _ptr(cache.block_table), c_int(cache.block_table.shape[1]), c_int(cache.block_size), c_int(T), c_int(nq),
            c_int(nkv), c_int(hd), c_float(scale), c_int(window or 0), c_int(qkv.dtype == torch.bfloat16),
            self._stream())
        self._check(code, "attention_plain")

    def _kv_tensor_maps(self, cache, nkv, hd):
        """The TMA descriptors (host buffers of 128 bytes) of a layer's key and value pools, made
        once per pool; None when the TMA kernel does not take this head or page size."""
        bs = cache.block_size
        if hd not in (64, 128) or bs < 8 or bs > 256 or bs & (bs - 1):
            return None
        key = (cache.k_pages.data_ptr(), cache.v_pages.data_ptr(), tuple(cache.k_pages.shape))
        maps = self._kv_maps.get(key)
        if maps is None:
            lib = self.lib("attention_decode_tma")
            bufs = []
            for pages in (cache.k_pages, cache.v_pages):
                buf = ctypes.create_string_buffer(128)
                code = lib.zllm_attention_kv_map(buf, _ptr(pages), c_longlong(pages.shape[0]), c_int(nkv), c_int(bs), c_int(hd))
                if code != 0:
                    raise BackendError(f"attention_kv_map: the driver refused the tensor map (code {code})")
                bufs.append(buf)
            maps = self._kv_maps[key] = tuple(bufs)
        return maps

    QUERY_TILE = 128        # query rows of one tile of the prefill attention kernels (PF_QROWS in csrc)

    @classmethod
    def plan_query_tiles(cls, entries, starts, aux, bucketed=False):
        """The step planner of the attention path: every portion (an entry of two tokens or more)
        cut into tiles of QUERY_TILE rows, as [first row, rows, slot, position of the first row].
        ``bucketed``: the list is rounded up to a power of two with empty tiles (0 rows, slot -1),
        which the kernels skip, so that steps of like shape can replay one captured graph."""
        q = cls.QUERY_TILE
        n_real = sum(-(-len(e.tokens) // q) for e in entries if len(e.tokens) > 1)
        n = n_real
        if bucketed and n_real:
            n = 1
            while n < n_real:
                n *= 2
        host, off = aux.take(4 * n)
        if n > n_real:
            host[4 * n_real:4 * n] = (0, 0, -1, 0) * (n - n_real)
        r = i = 0
        for e, start in zip(entries, starts):
            m = len(e.tokens)
            if m > 1:
                for q0 in range(0, m, q):
                    host[i:i + 4] = (r + q0, min(q, m - q0), e.slot, start + q0)
                    i += 4
            r += m
        return {"query_tiles": (off, (n, 4))}

    def _attention_bf16(self, qkv, out, ctx, cache, nq, nkv, hd, scale, window) -> bool:
        """Tensor-core attention: decoded rows by the split kernel, portions by the tiled kernel.
        False: head size or group not taken, every row goes to the plain kernel."""
        if hd % 16 or hd > 128 or nq // nkv > 16 or not scale > 0:
            return False
        lib = self.lib("attention_bf16")
        tb = cache.block_table
        if ctx.n_decode > 0:
            max_splits = max(1, -(-tb.shape[1] * cache.block_size // self.decode_split_keys))
            n_splits = min(max_splits, ctx.fixed_splits or self.decode_splits(ctx.max_context))
            # slots per (row, head): the splits, and behind them room for the partials of a merge in
            # two passes (one per 32 splits)
            max_splits += -(-max_splits // 32)
            nd = ctx.n_decode
            part_o = ctx.ws.get("attn_part_o", (nd, nq * max_splits * hd), torch.float32, cap=nd)
            part_ml = ctx.ws.get("attn_part_ml", (nd, nq * max_splits * 2), torch.float32, cap=nd)
            maps = self._kv_tensor_maps(cache, nkv, hd) if not window and nq // nkv <= 8 else None
            if maps:
                # pages by TMA: head sizes 64 and 128, page sizes 8..256 that are powers of two, no window
                code = self.lib("attention_decode_tma").zllm_attention_decode_tma(
                    _ptr(qkv), _ptr(out), _ptr(ctx.decode_rows), c_int(nd), _ptr(ctx.positions), _ptr(ctx.row_slot),
                    maps[0], maps[1], _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(tb), c_int(tb.shape[1]),
                    c_int(cache.block_size), c_int(nq), c_int(nkv),
                    c_int(hd), c_float(scale), _ptr(part_o), _ptr(part_ml), c_int(n_splits), c_int(max_splits),
                    self._stream())
                self._check(code, "attention_decode_tma")
                if n_splits == 1:
                    self.launches -= 1          # one split per row: the kernel writes the output itself
            else:
                code = lib.zllm_attention_decode_bf16(
                    _ptr(qkv), _ptr(out), _ptr(ctx.decode_rows), c_int(nd), _ptr(ctx.positions), _ptr(ctx.row_slot),
                    _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(tb), c_int(tb.shape[1]), c_int(cache.block_size),
                    c_int(nq), c_int(nkv), c_int(hd), c_float(scale), c_int(window or 0), _ptr(part_o), _ptr(part_ml),
                    c_int(n_splits), c_int(max_splits), self._stream())
                self._check(code, "attention_decode_bf16")
            self.launches += 2 if 256 <= n_splits <= 1024 else 1               # split kernel + merge (in two passes
                                                                                # from 256 to 1,024 splits)
        bs = cache.block_size
        tiles = ctx.aux.get("query_tiles")
        n_tiles = tiles.shape[0] if tiles is not None else 0
        if n_tiles > 0 and not window and hd in (64, 128) and (16 if hd == 128 else 8) <= bs <= 128 \
                and bs & (bs - 1) == 0:
            # the tcgen05 kernel: Q and pages by TMA, S and O in tensor memory
            code = self.lib("attention_prefill_tc").zllm_attention_prefill_tc(
                _ptr(qkv), c_int(qkv.shape[0]), _ptr(out), _ptr(tiles), c_int(n_tiles), _ptr(cache.k_pages),
                _ptr(cache.v_pages), c_longlong(cache.k_pages.shape[0]), _ptr(tb), c_int(tb.shape[1]), c_int(bs),
                c_int(nq), c_int(nkv), c_int(hd), c_float(scale), self._stream())
            self._check(code, "attention_prefill_tc")
        elif n_tiles > 0:
            code = lib.zllm_attention_prefill_bf16(
                _ptr(qkv), _ptr(out), _ptr(tiles), c_int(n_tiles), _ptr(cache.k_pages), _ptr(cache.v_pages),
                _ptr(tb), c_int(tb.shape[1]), c_int(cache.block_size), c_int(nq), c_int(nkv), c_int(hd),
                c_float(scale), c_int(window or 0), self._stream())
            self._check(code, "attention_prefill_bf16")
        return True

    # ---- sampling --------------------------------------------------------
    def sample(self, logits, temps, seeds, out):
        """out[r] = argmax_i(logits[r,i]/temp_r + Gumbel(seed_r, i)); temp <= 0: plain argmax,
        lowest index on ties."""
        self._dev(logits, temps, seeds, out)
        R, V = logits.shape
        if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() < R:
            raise BackendError("sample: bad operand types or shapes")
        if temps is not None and (temps.dtype != torch.float32 or temps.numel() < R):
            raise BackendError("sample: temps must be float32 [rows]")
        if seeds is not None and (seeds.dtype not in (torch.int32, torch.uint32) or seeds.numel() < R):
            raise BackendError("sample: seeds must be 32-bit [rows]")
        # scratch of the many-blocks-per-row kernel: made once (captured graphs keep its address);
        # more rows than it holds use the one-block-per-row kernel
        if self._sample_scratch is None:
            n = self.SAMPLE_SCRATCH_ROWS
            self._sample_scratch = (torch.zeros((n, 64), dtype=torch.float32, device=self.device),
                                    torch.zeros((n, 64), dtype=torch.int32, device=self.device),
                                    torch.zeros(n, dtype=torch.int32, device=self.device))
        sc = self._sample_scratch if R <= self.SAMPLE_SCRATCH_ROWS else (None, None, None)
        code = self.lib("sampling").zllm_sample(_ptr(logits), _ptr(temps), _ptr(seeds), _ptr(out), c_int(R), c_int(V),
                                                _ptr(sc[0]), _ptr(sc[1]), _ptr(sc[2]), self._stream())
        self._check(code, "sample")

    def advance_decode(self, tok, pos, row_slot, seeds, out, hist, counter):
        """tok <- out, pos += 1, seed += 0x9E3779B1 for live rows; out appended to the history ring."""
        self._dev(tok, pos, row_slot, seeds, out, hist, counter)
        B = tok.numel()
        if hist.shape[1] != B or pos.numel() != B or out.numel() < B:
            raise BackendError("advance_decode: shapes do not match the bucket")
        code = self.lib("sampling").zllm_advance_decode(_ptr(tok), _ptr(pos), _ptr(row_slot), _ptr(seeds), _ptr(out),
                                                        _ptr(hist), _ptr(counter), c_int(hist.shape[0]), c_int(B),
                                                        self._stream())
        self._check(code, "advance_decode")

    TOPK_SCRATCH_ROWS = 128
    TOPK_STRETCHES = 256                # csrc/sampling.cu

    def topk(self, logits, k, vals, idx):
        """The k best entries of every row, value descending, index ascending."""
        self._dev(logits, vals, idx)
        R, V = logits.shape
        if logits.dtype != torch.float32 or vals.dtype != torch.float32 or idx.dtype != torch.int32 \
                or tuple(vals.shape) != (R, k) or tuple(idx.shape) != (R, k):
            raise BackendError("topk: bad operand types or shapes")
        cv = ci = None
        if R <= self.TOPK_SCRATCH_ROWS and k <= 64:        # candidates of the two-stage kernels; fixed for graphs
            if self._topk_scratch is None:
                n = self.TOPK_SCRATCH_ROWS * ((self.TOPK_STRETCHES + 32) * 64 + 64)
                self._topk_scratch = (torch.empty(n, dtype=torch.float32, device=self.device),
                                      torch.empty(n, dtype=torch.int32, device=self.device))
            cv, ci = self._topk_scratch
        code = self.lib("sampling").zllm_topk(_ptr(logits), _ptr(vals), _ptr(idx), c_int(R), c_int(V), c_int(k),
                                              _ptr(cv), _ptr(ci), self._stream())
        self._check(code, "topk")
        if cv is not None and 16384 <= V <= self.TOPK_STRETCHES * 512:
            self.launches += 3               # group maxima, stretches, two merges

    def pool_draw(self, vals, idx, ptemp, topk, topp, seeds, out):
        """out[r] = a draw among row r's descending candidates (temperature ptemp[r], the first
        topk[r] of them (0: all), cut at cumulative mass topp[r]); rows with ptemp <= 0 keep out[r].
        ptemp, topp float64; the arithmetic is the host path's (sampling/sampler.py), in double."""
        self._dev(vals, idx, ptemp, topk, topp, seeds, out)
        R, k = vals.shape
        if vals.dtype != torch.float32 or idx.dtype != torch.int32 or ptemp.dtype != torch.float64 or topp.dtype != torch.float64 \
                or topk.dtype != torch.int32 or seeds.dtype != torch.int32 or out.dtype != torch.int32 or tuple(idx.shape) != (R, k) \
                or min(ptemp.numel(), topk.numel(), topp.numel(), seeds.numel(), out.numel()) < R:
            raise BackendError("pool_draw: bad operand types or shapes")
        code = self.lib("sampling").zllm_pool_draw(_ptr(vals), _ptr(idx), _ptr(ptemp), _ptr(topk), _ptr(topp), _ptr(seeds),
                                                   _ptr(out), c_int(R), c_int(k), self._stream())
        self._check(code, "pool_draw")
