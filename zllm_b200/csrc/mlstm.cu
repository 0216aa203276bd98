// A matrix memory with exponential gates (mLSTM): per request and head a matrix S [dk, dv], a
// vector n [dk] and a running maximum m of the accumulated log gates, all float32, carried
// from token to token in the request's state slot.
//
//   gi = cap tanh((zi + bi) / cap)                     log input gate
//   gf = logsigmoid(cap tanh((zf + bf) / cap))         log forget gate
//   m' = max(gf + m, gi);  keep = exp(gf + m - m');  take = exp(gi - m')
//   S' = keep S + take k v^T;   n' = keep n + take k
//   out = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6),   q already times dk^(-1/2)
//
// Three kernels per step of the engine:
//   mlstm_gates:  one block per (segment, head): eight tokens at a time are staged in shared memory
//                 (q, k, and the two gates with their tanh and logsigmoid) by three warps while
//                 the first warp walks the eight before them in order: m, n and n.q; leaves
//                 (keep, take, denominator) per (row, head) and the new n, m.
//   mlstm_scan:   blocks per (segment, head, slice of dv): a group of lanes owns one column of S
//                 in registers (16 rows per thread) and walks the tokens in order; q, k, v and
//                 the per-token factors come through shared memory eight tokens at a time.
//   mlstm_finish: per row and head: out / rms(out), times the norm weight, the output gate
//                 sigmoid(g) and a constant.
// A segment is the run of a request's rows in the step, (first row, rows, slot, ...), from a
// table the host wrote; without a table every row is a segment of its own (decode steps) and
// its slot is row_slot[row].  Segments with no rows or a negative slot are skipped.
// State of a slot: per head [S (dk*dv) | n (dk) | m].
#include "common.cuh"
#include <math.h>

#define ML_NL 16          // n entries per lane: dk <= 512
#define ML_CHUNK 8        // tokens staged at a time
#define ML_COLT 256       // threads of a scan block that walk columns of S
#define ML_RPT 16         // rows of S per thread
#define ML_PROD 64        // threads of a scan block that only bring in the next chunk

__device__ __forceinline__ bool segment_of(const int* segs, const int* row_slot, int s, int& row0, int& rows, int& slot) {
    if (segs != nullptr) {
        row0 = segs[4 * s]; rows = segs[4 * s + 1]; slot = segs[4 * s + 2];
    } else {
        row0 = s; rows = 1; slot = row_slot[s];
    }
    return rows > 0 && slot >= 0;
}

#define ML_GTHREADS 128   // threads of a gates block: all stage a chunk, the first warp walks it

// eight consecutive operand values as float32 (the address is 16-byte aligned for bfloat16, 32 for float32)
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// Stage q (scaled) and k of tokens t0 .. t0+nc-1 of head h into dst[j * per + (0..dk-1 | dk..2dk-1)].
// vec: pieces of eight values by 16-byte loads, several in flight per thread; else value by value.
template <typename AT>
__device__ __forceinline__ void stage_qk(float* dst, int per, const AT* qkv, int ld, int oq, int ok, int h, int dk,
                                         size_t t0, int nc, float qscale, int vec, int tid, int NTHR) {
    if (vec) {
        const int pieces = 2 * dk / 8;                         // per token
        for (int i0 = tid; i0 < nc * pieces; i0 += NTHR * 4) {
            float v[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * NTHR;
                if (i < nc * pieces) {
                    const int j = i / pieces, e = (i - j * pieces) * 8;
                    const AT* src = qkv + (t0 + j) * ld + (e < dk ? oq + (size_t)h * dk + e : ok + (size_t)h * dk + (e - dk));
                    load8(src, v[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * NTHR;
                if (i < nc * pieces) {
                    const int j = i / pieces, e = (i - j * pieces) * 8;
                    const float sc = e < dk ? qscale : 1.f;
                    float* d = dst + j * per + e;
#pragma unroll
                    for (int x = 0; x < 8; ++x) d[x] = v[u][x] * sc;
                }
            }
        }
        return;
    }
    for (int i = tid; i < nc * 2 * dk; i += NTHR) {
        const int j = i / (2 * dk), e = i - j * 2 * dk;
        dst[j * per + e] = e < dk ? to_f32(qkv[(t0 + j) * ld + oq + (size_t)h * dk + e]) * qscale
                                  : to_f32(qkv[(t0 + j) * ld + ok + (size_t)h * dk + (e - dk)]);
    }
}

// NLT > 0: dk is exactly 32 * NLT (no bounds checks, no idle registers); NLT == 0: any dk up to 32 * ML_NL.
template <typename AT, int NLT>
__global__ void __launch_bounds__(ML_GTHREADS) mlstm_gates_kernel(
    const AT* qkv, int ld, int oq, int ok, const float* z, const float* __restrict__ bi, const float* __restrict__ bf,
    float cap, float qscale, const int* __restrict__ segs, const int* row_slot, float* state, size_t state_stride,
    float* fac, int H, int dk, int dv, int vec) {
    // A chunk of eight tokens at a time: three warps stage q, k and the two log gates of the NEXT chunk while
    // the first warp walks this one: the running maximum as a short chain (a few operations per token), the
    // exponentials of the chunk by eight lanes at once, n and the partial n.q token by token, and the
    // eight sums over the lanes together at the end, so that few long latencies follow one another.
    extern __shared__ float qk_stage[];                      // [2][ML_CHUNK][2 * dk]: the chunk walked and the next one
    __shared__ float gate2[2][ML_CHUNK][2];
    __shared__ float coef[ML_CHUNK][3];                      // keep, take, exp(-m) per token
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int row0, rows, slot;
    if (!segment_of(segs, row_slot, blockIdx.x, row0, rows, slot)) return;
    const int per = 2 * dk;
    float* st = state + (size_t)slot * state_stride + (size_t)h * ((size_t)dk * dv + dk + 1);
    float* np = st + (size_t)dk * dv;
    constexpr int NLV = NLT > 0 ? NLT : ML_NL;
    float n[NLV];
    float m = 0.f;
    if (warp == 0) {
#pragma unroll
        for (int i = 0; i < NLV; ++i) { const int r = lane + 32 * i; n[i] = (NLT > 0 || r < dk) ? np[r] : 0.f; }
        m = np[dk];
    }
    const float b_i = bi[h], b_f = bf[h];
    // threads tid of nthr bring the chunk at c0 into buffer b: q, k, and the two log gates
    auto produce = [&](int b, int c0, int tid, int nthr) {
        const int nc = min(ML_CHUNK, rows - c0);
        stage_qk<AT>(qk_stage + (size_t)b * ML_CHUNK * per, per, qkv, ld, oq, ok, h, dk, (size_t)(row0 + c0), nc, qscale, vec,
                     tid, nthr);
        if (tid < nc) {
            const size_t t = (size_t)(row0 + c0 + tid);
            const float zi = z[t * 2 * H + h], zf = z[t * 2 * H + H + h];
            const float a = cap * tanhf((zf + b_f) / cap);
            gate2[b][tid][0] = cap * tanhf((zi + b_i) / cap);
            gate2[b][tid][1] = fminf(a, 0.f) - log1pf(expf(-fabsf(a)));
        }
    };
    produce(0, 0, threadIdx.x, ML_GTHREADS);
    __syncthreads();
    int buf = 0;
    for (int c0 = 0; c0 < rows; c0 += ML_CHUNK, buf ^= 1) {
        const int nc = min(ML_CHUNK, rows - c0);
        if (warp != 0) {
            // three warps bring in the next chunk while the first walks this one
            if (c0 + ML_CHUNK < rows) produce(buf ^ 1, c0 + ML_CHUNK, threadIdx.x - 32, ML_GTHREADS - 32);
            __syncthreads();
            continue;
        }
        const float (*gate)[2] = gate2[buf];
        const float* qk_now = qk_stage + (size_t)buf * ML_CHUNK * per;
        // the running maximum of the chunk, token by token; every lane computes it (no exchange needed)
        float m_at[ML_CHUNK + 1];
        m_at[0] = m;
#pragma unroll
        for (int j = 0; j < ML_CHUNK; ++j) m_at[j + 1] = j < nc ? fmaxf(gate[j][1] + m_at[j], gate[j][0]) : m_at[j];
#pragma unroll
        for (int j = 0; j < ML_CHUNK; ++j)
            if (lane == j && j < nc) {
                coef[j][0] = expf(gate[j][1] + m_at[j] - m_at[j + 1]);
                coef[j][1] = expf(gate[j][0] - m_at[j + 1]);
                coef[j][2] = expf(-m_at[j + 1]);
            }
        m = m_at[ML_CHUNK];
        __syncwarp();
        float dot[ML_CHUNK];
#pragma unroll
        for (int j = 0; j < ML_CHUNK; ++j) {
            dot[j] = 0.f;
            if (j < nc) {
                const float keep = coef[j][0], take = coef[j][1];
                const float* q = qk_now + j * per;
                const float* k = q + dk;
#pragma unroll
                for (int i = 0; i < NLV; ++i) {
                    const int r = lane + 32 * i;
                    if (NLT > 0 || r < dk) {
                        n[i] = keep * n[i] + take * k[r];
                        dot[j] = fmaf(n[i], q[r], dot[j]);
                    }
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int j = 0; j < ML_CHUNK; ++j) dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], o);
#pragma unroll
        for (int j = 0; j < ML_CHUNK; ++j)
            if (lane == j && j < nc) {
                float* f = fac + ((size_t)(row0 + c0 + j) * H + h) * 4;
                f[0] = coef[j][0]; f[1] = coef[j][1]; f[2] = fmaxf(fabsf(dot[j]), coef[j][2]) + 1e-6f;
            }
        __syncthreads();                                  // the next chunk is in place, this one may be overwritten
    }
    if (warp != 0) return;
#pragma unroll
    for (int i = 0; i < NLV; ++i) { const int r = lane + 32 * i; if (NLT > 0 || r < dk) np[r] = n[i]; }
    if (lane == 0) np[dk] = m;
}


// KPT > 0: kp is KPT and dk exactly KPT * ML_RPT (offsets known to the compiler, no bounds checks); 0: any.
template <typename AT, int KPT>
__global__ void __launch_bounds__(ML_COLT + ML_PROD) mlstm_scan_kernel(
    const AT* qkv, int ld, int oq, int ok, int ov, const float* fac, float qscale, const int* __restrict__ segs,
    const int* row_slot, float* state, size_t state_stride, float* out, int H, int dk, int dv, int kp, int vec) {
    // kp lanes share a column of S (rows sub, sub + kp, ...: ML_RPT of them per thread), so that a step is
    // short and an SM holds many warps; the lanes' partial sums are added with shuffles.  Two more warps
    // bring the next eight tokens into the other half of shared memory while these are walked.
    extern __shared__ float sm[];                     // [2][ML_CHUNK][per]
    pdl_trigger();
    pdl_wait();
    if (KPT > 0) { kp = KPT; dk = KPT * ML_RPT; }
    const int h = blockIdx.y;
    int row0, rows, slot;
    if (!segment_of(segs, row_slot, blockIdx.x, row0, rows, slot)) return;
    const int tidx = threadIdx.x;
    const bool producer = tidx >= ML_COLT;
    const int vs = ML_COLT / kp;                      // columns of this block
    const int sub = tidx % kp;
    const int lcol = producer ? 0 : tidx / kp;
    const int col = blockIdx.z * vs + lcol;
    const bool has = !producer && col < dv;
    float* S = state + (size_t)slot * state_stride + (size_t)h * ((size_t)dk * dv + dk + 1);
    float s[ML_RPT];
#pragma unroll
    for (int i = 0; i < ML_RPT; ++i) { const int r = sub + i * kp; s[i] = (has && (KPT > 0 || r < dk)) ? S[(size_t)r * dv + col] : 0.f; }
    const int per = 2 * dk + vs + 4;                  // floats staged per token: q, k, v slice, factors
    auto produce = [&](int b, int c0, int tid, int nthr) {
        const int nc = min(ML_CHUNK, rows - c0);
        float* dst = sm + (size_t)b * ML_CHUNK * per;
        stage_qk<AT>(dst, per, qkv, ld, oq, ok, h, dk, (size_t)(row0 + c0), nc, qscale, vec, tid, nthr);
        for (int i = tid; i < nc * (vs + 4); i += nthr) {
            const int j = i / (vs + 4), e = i - j * (vs + 4);
            const size_t t = (size_t)(row0 + c0 + j);
            float v;
            if (e < vs) {
                const int cc = blockIdx.z * vs + e;
                v = cc < dv ? to_f32(qkv[t * ld + ov + (size_t)h * dv + cc]) : 0.f;
            } else v = fac[(t * H + h) * 4 + (e - vs)];
            dst[j * per + 2 * dk + e] = v;
        }
    };
    produce(0, 0, tidx, ML_COLT + ML_PROD);
    __syncthreads();
    int buf = 0;
    for (int c0 = 0; c0 < rows; c0 += ML_CHUNK, buf ^= 1) {
        const int nc = min(ML_CHUNK, rows - c0);
        if (producer) {
            if (c0 + ML_CHUNK < rows) produce(buf ^ 1, c0 + ML_CHUNK, tidx - ML_COLT, ML_PROD);
        } else {
            const float* now = sm + (size_t)buf * ML_CHUNK * per;
            for (int j = 0; j < nc; ++j) {
                const float* q = now + j * per;
                const float* k = q + dk;
                const float vv = q[2 * dk + lcol];
                const float keep = q[2 * dk + vs], take = q[2 * dk + vs + 1], den = q[2 * dk + vs + 2];
                const float tv = take * vv;
                float part[4] = {0.f, 0.f, 0.f, 0.f};     // four chains instead of one of dependent additions
#pragma unroll
                for (int i = 0; i < ML_RPT; ++i) {
                    const int r = sub + i * kp;
                    if (KPT > 0 || r < dk) {
                        s[i] = fmaf(tv, k[r], keep * s[i]);
                        part[i & 3] = fmaf(s[i], q[r], part[i & 3]);
                    }
                }
                float num = (part[0] + part[1]) + (part[2] + part[3]);
                for (int o = 1; o < kp; o <<= 1) num += __shfl_xor_sync(0xffffffffu, num, o);
                if (has && sub == 0) out[(size_t)(row0 + c0 + j) * H * dv + (size_t)h * dv + col] = num / den;
            }
        }
        __syncthreads();                              // the next chunk is in place, this one may be overwritten
    }
    if (has) {
#pragma unroll
        for (int i = 0; i < ML_RPT; ++i) { const int r = sub + i * kp; if (KPT > 0 || r < dk) S[(size_t)r * dv + col] = s[i]; }
    }
}

template <typename AT>
__global__ void __launch_bounds__(256) mlstm_finish_kernel(const float* raw, const AT* gate, int ldg, int og,
                                                           const float* __restrict__ w, AT* out, const int* row_slot, int H,
                                                           int dv, float eps, float mult) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const bool pad = row_slot[t] < 0;
    for (int h = warp; h < H; h += nw) {
        const float* r = raw + ((size_t)t * H + h) * dv;
        AT* o = out + ((size_t)t * H + h) * dv;
        if (pad) {
            for (int c = lane; c < dv; c += 32) o[c] = from_f32<AT>(0.f);
            continue;
        }
        float ss = 0.f;
        for (int c = lane; c < dv; c += 32) ss += r[c] * r[c];
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss / (float)dv + eps);
        for (int c = lane; c < dv; c += 32) {
            const float g = to_f32(gate[(size_t)t * ldg + og + (size_t)h * dv + c]);
            o[c] = from_f32<AT>(r[c] * inv * w[h * dv + c] * (1.f / (1.f + expf(-g))) * mult);
        }
    }
}

// qkv [T, ld]: head h's queries at column oq + h*dk, keys at ok + h*dk, values at ov + h*dv,
// output-gate inputs at og + h*dv.  z [T, 2H] float32: the input gates' then the forget gates'
// projections.  fac [T, H, 4] and raw [T, H*dv] float32 are scratch; out [T, H*dv] receives
// the gated, normed result.  segs: null or [n_seg, 4].
ZLLM_API int zllm_mlstm(const void* qkv, int ld, int oq, int ok, int ov, int og, const float* z, const float* bi,
                        const float* bf, float cap, const float* wnorm, float eps, float mult, const int* segs, int n_seg,
                        const int* row_slot, float* state, long long state_stride, float* fac, float* raw, void* out, int T,
                        int H, int dk, int dv, int is_bf16, void* stream) {
    if (T <= 0) return 0;
    if (dk <= 0 || dk > 32 * ML_NL || dv <= 0 || H <= 0 || !(cap > 0.f)) return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int ns = segs != nullptr ? n_seg : T;
    const float qscale = 1.f / sqrtf((float)dk);
    int kp = 1;
    while (kp * ML_RPT < dk) kp *= 2;                 // lanes per column of S: ML_RPT rows per thread, at most 32 lanes
    const int vs = ML_COLT / kp;
    const size_t smem = (size_t)2 * ML_CHUNK * (2 * dk + vs + 4) * sizeof(float);     // two chunks: walked, and brought in
    const size_t gsmem = (size_t)2 * ML_CHUNK * 2 * dk * sizeof(float);
    dim3 grid(ns, H, (dv + vs - 1) / vs);
    // pieces of eight values by 16-byte loads when every run of q and k starts on such a boundary
    const int el = is_bf16 ? 2 : 4;
    const int vec = (dk % 8 == 0 && ld % 8 == 0 && oq % 8 == 0 && ok % 8 == 0 && ((uintptr_t)qkv % (8 * el)) == 0) ? 1 : 0;
    // the kernels are instantiated for the sizes that fill their registers exactly (dk = 32 * 2^a for the
    // gates, dk = 16 * kp for the scan) and once for any size
#define ML_LAUNCH(AT)                                                                                                         \
    do {                                                                                                                      \
        auto gk = mlstm_gates_kernel<AT, 0>;                                                                                  \
        if (dk == 32) gk = mlstm_gates_kernel<AT, 1>;                                                                         \
        else if (dk == 64) gk = mlstm_gates_kernel<AT, 2>;                                                                    \
        else if (dk == 128) gk = mlstm_gates_kernel<AT, 4>;                                                                   \
        else if (dk == 256) gk = mlstm_gates_kernel<AT, 8>;                                                                   \
        else if (dk == 512) gk = mlstm_gates_kernel<AT, 16>;                                                                  \
        auto sk = mlstm_scan_kernel<AT, 0>;                                                                                   \
        if (dk == kp * ML_RPT) {                                                                                              \
            if (kp == 1) sk = mlstm_scan_kernel<AT, 1>;                                                                       \
            else if (kp == 2) sk = mlstm_scan_kernel<AT, 2>;                                                                  \
            else if (kp == 4) sk = mlstm_scan_kernel<AT, 4>;                                                                  \
            else if (kp == 8) sk = mlstm_scan_kernel<AT, 8>;                                                                  \
            else if (kp == 16) sk = mlstm_scan_kernel<AT, 16>;                                                                \
            else if (kp == 32) sk = mlstm_scan_kernel<AT, 32>;                                                                \
        }                                                                                                                     \
        if (smem > 48 * 1024 || gsmem > 48 * 1024) {        /* dk = 512 needs 66 KB of dynamic shared memory */              \
            cudaError_t e = cudaFuncSetAttribute(gk, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);                 \
            if (e == cudaSuccess) e = cudaFuncSetAttribute(sk, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);       \
            if (e != cudaSuccess) return (int)e;                                                                              \
        }                                                                                                                     \
        code = launch_pdl(gk, dim3(ns, H), dim3(ML_GTHREADS), gsmem, s, (const AT*)qkv, ld, oq, ok, z, bi, bf, cap, qscale, segs, \
                          row_slot, state, (size_t)state_stride, fac, H, dk, dv, vec);                                        \
        if (code) return code;                                                                                                \
        code = launch_pdl(sk, grid, dim3(ML_COLT + ML_PROD), smem, s, (const AT*)qkv, ld, oq, ok, ov, (const float*)fac, qscale, \
                          segs, row_slot, state, (size_t)state_stride, raw, H, dk, dv, kp, vec);                               \
        if (code) return code;                                                                                                \
    } while (0)
    int code;
    if (ns > 0) {
        if (is_bf16) ML_LAUNCH(bf16);
        else ML_LAUNCH(float);
    }
#undef ML_LAUNCH
    if (is_bf16)
        return launch_pdl(mlstm_finish_kernel<bf16>, dim3(T), dim3(256), 0, s, raw, (const bf16*)qkv, ld, og, wnorm, (bf16*)out,
                          row_slot, H, dv, eps, mult);
    return launch_pdl(mlstm_finish_kernel<float>, dim3(T), dim3(256), 0, s, raw, (const float*)qkv, ld, og, wnorm, (float*)out,
                      row_slot, H, dv, eps, mult);
}
