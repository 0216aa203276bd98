// The experts' products, and the per-head products, on tensor cores (bfloat16 operands, float32 accumulation).
//
// Same interface as the per-expert kernel of gemm_grouped.cu: rows are (token, choice) pairs sorted
// by expert, expert e owns the sorted range off[e]..off[e+1]-1, sorted entry i stands for pair
// perm[i].  A CTA takes a tile of 128 sorted rows of ONE expert and 128 weight rows:
//   first product  (gated):  64 gate rows and the 64 up rows of the same outputs; the rows of x are
//                  gathered (x[perm[i] / top]); act[i][n] = silu(gate) * up in bfloat16;
//   first product  (no gate): 128 rows of the one matrix, rows of x gathered; act[i][n] = f(sum), f one of silu,
//                  gelu (erf), gelu (tanh); in both forms the float32 sums of the first n_scaled choices of a
//                  token are multiplied by the pair's router weight first (a weight on the expert's input);
//   second product:          128 rows of the down matrix; y[perm[i]][n] in float32 (scattered).
// K runs in pieces of 64 or 32 through a three-stage cp.async ring; fragments come from shared memory with
// ldmatrix and go to mma.sync m16n8k16; eight warps as 4 x 2, each 32 rows x 64 columns.  Every
// output is the sum over k in a fixed order that depends on K alone, so a row's result does not
// depend on which other rows share its tile.  Needs K % 32 == 0 and 16-byte aligned operands;
// other sizes go to the CUDA-core kernel.
#include "attention_common.cuh"

#define TM 128
#define TN 128
// K is walked in pieces of TK = 64 through 3 stages (110 KB of shared memory, two CTAs per SM, 72 KB of weights
// in flight per SM) when K is a multiple of 64, else in pieces of 32 (61 KB, three CTAs per SM).  A shared-memory row holds TK + 8 bfloat16, so that
// the eight rows of an ldmatrix fall on distinct banks.

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// The product of one tile: A rows and B rows arrive through the cp.async ring, PER_THREAD 16-byte pieces of
// each per thread and stage (a_src / b_src: where the thread's pieces start in global memory, dst: where
// they go in a stage, a_live: whether the A row exists); acc[mt][nt] are the warp's 2 x 8 tiles of 16 x 8.
template <bool SWIGLU, int TK, int STAGES, int PER_THREAD>
__device__ __forceinline__ void tile_mainloop(bf16* As, bf16* Bs, const bf16* (&a_src)[PER_THREAD], const bf16* (&b_src)[PER_THREAD],
                                              const bool (&a_live)[PER_THREAD], const int (&dst)[PER_THREAD], int K, bool warp_live,
                                              int wm, int wn, int lane, float (&acc)[2][8][4]) {
    constexpr int LDS = TK + 8;
    auto load_stage = [&](int st, int kt) {
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            if (a_live[i]) cp_async16(As + st * TM * LDS + dst[i], a_src[i] + (size_t)kt * TK);
            cp_async16(Bs + st * TN * LDS + dst[i], b_src[i] + (size_t)kt * TK);
        }
    };
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;

    const int KT = K / TK;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < KT) load_stage(s, s);
        cp_async_commit();
    }
    for (int kt = 0; kt < KT; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (kt + STAGES - 1 < KT) load_stage((kt + STAGES - 1) % STAGES, kt + STAGES - 1);
        cp_async_commit();
        const bf16* Ast = As + (kt % STAGES) * TM * LDS;
        const bf16* Bst = Bs + (kt % STAGES) * TN * LDS;
        if (!warp_live) continue;                            // this warp's 32 rows lie beyond the expert's range (few rows)
#pragma unroll
        for (int ks = 0; ks < TK / 16; ++ks) {
            unsigned af[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
                ldmatrix_x4(af[mt], Ast + (wm * 32 + mt * 16 + (lane & 15)) * LDS + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                // 16 weight rows per ldmatrix: with SWIGLU the warp's first 32 are gate rows, the last 32 their up rows
                const int brow = SWIGLU ? (p < 2 ? wn * 32 + p * 16 : 64 + wn * 32 + (p - 2) * 16) : wn * 64 + p * 16;
                unsigned bfr[4];
                ldmatrix_x4(bfr, Bst + (brow + (lane & 7) + (lane >> 4) * 8) * LDS + ks * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    mma16816(acc[mt][2 * p], af[mt], bfr[0], bfr[1]);
                    mma16816(acc[mt][2 * p + 1], af[mt], bfr[2], bfr[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
}

#define ACT_SILU 0
#define ACT_GELU 1
#define ACT_GELU_TANH 2
__device__ __forceinline__ float expert_act(float z, int act) {
    if (act == ACT_GELU) return 0.5f * z * (1.f + erff(z * 0.70710678118654752440f));
    if (act == ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
    return z / (1.f + expf(-z));
}

// MODE 0: second product (rows in sorted order, float32 rows scattered); 1: gated first product; 2: first product
// with one matrix and an activation (both gather their rows)
template <int MODE, int TK, int STAGES>
__global__ void __launch_bounds__(256) gemm_experts_mma_kernel(const bf16* x, const bf16* __restrict__ w,
                                                               const bf16* __restrict__ wu, void* out, const int* off,
                                                               const int* perm, int top, int E, int N, int K,
                                                               const float* row_scale, int n_scaled, int act) {
    constexpr bool SWIGLU = MODE == 1;
    constexpr bool GATHER = MODE != 0;
    constexpr int LDS = TK + 8, PIECES = TK / 8, PER_THREAD = TM * PIECES / 256;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* As = reinterpret_cast<bf16*>(smem_raw);            // [STAGES][TM][LDS]
    bf16* Bs = As + STAGES * TM * LDS;                       // [STAGES][TN][LDS]
    __shared__ int s_e, s_row0;
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x < 32) {
        // which (expert, tile of its rows) is tile blockIdx.y: the experts' tile counts 32 at a time, a prefix
        // sum over the lanes, the first expert whose running total passes the tile
        const int lane_ = threadIdx.x;
        int before = 0, found_e = E, found_row0 = 0;
        for (int e0 = 0; e0 < E && found_e == E; e0 += 32) {
            const int ee = e0 + lane_;
            const int lo = ee < E ? off[ee] : 0;
            const int tiles = ee < E ? (off[ee + 1] - lo + TM - 1) / TM : 0;
            int incl = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane_ >= o) incl += v;
            }
            const int start = before + incl - tiles;                      // tiles before this lane's expert
            const bool mine = tiles > 0 && (int)blockIdx.y >= start && (int)blockIdx.y < start + tiles;
            const unsigned who = __ballot_sync(0xffffffffu, mine);
            if (who) {
                const int src = __ffs(who) - 1;
                found_e = e0 + src;
                found_row0 = __shfl_sync(0xffffffffu, lo + ((int)blockIdx.y - start) * TM, src);
            }
            before += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane_ == 0) { s_e = found_e; s_row0 = found_row0; }
    }
    __syncthreads();
    const int e = s_e;
    if (e >= E) return;
    const int row0 = s_row0, row_end = off[e + 1];
    const int n0 = blockIdx.x * (SWIGLU ? TN / 2 : TN);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 1, wn = warp & 1;

    // what this thread copies per stage: PER_THREAD 16-byte pieces of A rows and as many of B rows
    const bf16* a_src[PER_THREAD];
    const bf16* b_src[PER_THREAD];
    int dst[PER_THREAD];
    bool a_live[PER_THREAD];
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
        const int c = tid + i * 256, r = c / PIECES, kc = c % PIECES;
        int ri = row0 + r;
        a_live[i] = ri < row_end;                            // rows beyond the expert's range are neither loaded nor stored:
        if (ri >= row_end) ri = row0;                        // what a product makes of them stays in rows nobody reads
        const size_t src = GATHER ? (size_t)(perm[ri] / top) : (size_t)ri;
        a_src[i] = x + src * K + kc * 8;
        int n;
        const bf16* base;
        if (SWIGLU) { n = n0 + (r & 63); base = (r < 64 ? w : wu) + (size_t)e * N * K; }
        else { n = n0 + r; base = w + (size_t)e * N * K; }
        if (n >= N) n = N - 1;
        b_src[i] = base + (size_t)n * K + kc * 8;
        dst[i] = r * LDS + kc * 8;
    }
    float acc[2][8][4];
    const bool warp_live = row0 + wm * 32 < row_end;
    tile_mainloop<SWIGLU, TK, STAGES, PER_THREAD>(As, Bs, a_src, b_src, a_live, dst, K, warp_live, wm, wn, lane, acc);
    // epilogue: thread holds rows lane/4 (+8) and columns 2*(lane%4), +1 of every 16x8 tile
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = row0 + wm * 32 + mt * 16 + (lane >> 2) + half * 8;
            if (r >= row_end) continue;
            float cs = 1.f;
            if (GATHER && row_scale != nullptr) {
                const int pr = perm[r];
                if (pr % top < n_scaled) cs = row_scale[pr];
            }
            if (SWIGLU) {
                bf16* orow = reinterpret_cast<bf16*>(out) + (size_t)r * N;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int n = n0 + wn * 32 + nt * 8 + 2 * (lane & 3) + c;
                        if (n >= N) continue;
                        const float g = acc[mt][nt][half * 2 + c] * cs, u = acc[mt][nt + 4][half * 2 + c] * cs;
                        orow[n] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
                    }
            } else if (GATHER) {
                bf16* orow = reinterpret_cast<bf16*>(out) + (size_t)r * N;
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int n = n0 + wn * 64 + nt * 8 + 2 * (lane & 3) + c;
                        if (n < N) orow[n] = __float2bfloat16_rn(expert_act(acc[mt][nt][half * 2 + c] * cs, act));
                    }
            } else {
                float* orow = reinterpret_cast<float*>(out) + (size_t)perm[r] * N;
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int n = n0 + wn * 64 + nt * 8 + 2 * (lane & 3) + c;
                        if (n < N) orow[n] = acc[mt][nt][half * 2 + c];
                    }
            }
        }
}

// As zllm_gemm_experts (gemm_grouped.cu) for bfloat16: modes 1 and 2: out = act [n_pairs, N] bfloat16
// in sorted order from gathered rows of x; mode 0: out = y [n_pairs, N] float32 scattered.
ZLLM_API int zllm_gemm_experts_mma(const void* x, const void* w, const void* wu, void* out, const int* off, const int* perm,
                                   int top, int n_pairs, int E, int N, int K, int mode, const float* row_scale, int n_scaled,
                                   int act, void* stream) {
    if (n_pairs <= 0 || N <= 0) return 0;
    if (K <= 0 || (K % 32) || E <= 0 || top <= 0 || mode < 0 || mode > 2 || act < 0 || act > 2 ||
        (((uintptr_t)x | (uintptr_t)w | (uintptr_t)wu) & 15))
        return ZLLM_ERR_UNSUPPORTED;
    const int swiglu = mode == 1;
    cudaStream_t s = (cudaStream_t)stream;
    // pieces of 64 wherever K allows: measured at 2,048 rows of 32 experts 0.44 against 0.50 ms per layer, and at few
    // rows the wider pieces keep more weights in flight
    const bool few = K % 64 == 0;
    const size_t smem = few ? (size_t)3 * (TM + TN) * 72 * sizeof(bf16) : (size_t)3 * (TM + TN) * 40 * sizeof(bf16);
    static bool raised = false;
    if (!raised) {
        const int big = 3 * (TM + TN) * 72 * (int)sizeof(bf16), small = 3 * (TM + TN) * 40 * (int)sizeof(bf16);
        cudaError_t e = cudaSuccess;
#define GE_ATTR(MD) \
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_experts_mma_kernel<MD, 32, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, small); \
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_experts_mma_kernel<MD, 64, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
        GE_ATTR(0) GE_ATTR(1) GE_ATTR(2)
#undef GE_ATTR
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    const int n_cols = swiglu ? TN / 2 : TN;
    dim3 grid((N + n_cols - 1) / n_cols, (n_pairs + TM - 1) / TM + E);
#define GE_GO(MD, TKV, STV) return launch_pdl(gemm_experts_mma_kernel<MD, TKV, STV>, grid, dim3(256), smem, s, (const bf16*)x, \
                                              (const bf16*)w, (const bf16*)wu, out, off, perm, top, E, N, K, row_scale, n_scaled, act)
    if (mode == 1 && few) GE_GO(1, 64, 3);
    if (mode == 1) GE_GO(1, 32, 3);
    if (mode == 2 && few) GE_GO(2, 64, 3);
    if (mode == 2) GE_GO(2, 32, 3);
    if (few) GE_GO(0, 64, 3);
    GE_GO(0, 32, 3);
#undef GE_GO
}

// ---------------------------------------------------------------- per head
// out[t][g*N + n] = x[t][g*xg : g*xg + K] . w[g][n], optionally times sigmoid(gate[t][g*N + n]) * out_scale:
// the per-head products of gemm_grouped.cu on tensor cores.  Tile (n tile, 128 rows of the step, head).
template <bool OUT_F32, int TK, int STAGES>
__global__ void __launch_bounds__(256) gemm_heads_mma_kernel(const bf16* x, int ldx, int xg, const bf16* __restrict__ w, void* out,
                                                             const bf16* gate, int ldg, float out_scale, int T, int N, int K,
                                                             int G) {
    constexpr int LDS = TK + 8, PIECES = TK / 8, PER_THREAD = TM * PIECES / 256;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* As = reinterpret_cast<bf16*>(smem_raw);
    bf16* Bs = As + STAGES * TM * LDS;
    pdl_trigger();
    pdl_wait();
    const int g = blockIdx.z, row0 = blockIdx.y * TM, row_end = T, n0 = blockIdx.x * TN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 1, wn = warp & 1;
    const bf16* a_src[PER_THREAD];
    const bf16* b_src[PER_THREAD];
    int dst[PER_THREAD];
    bool a_live[PER_THREAD];
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
        const int c = tid + i * 256, r = c / PIECES, kc = c % PIECES;
        int ri = row0 + r;
        a_live[i] = ri < row_end;
        if (ri >= row_end) ri = row0;
        a_src[i] = x + (size_t)ri * ldx + (size_t)g * xg + kc * 8;
        int n = n0 + r;
        if (n >= N) n = N - 1;
        b_src[i] = w + ((size_t)g * N + n) * K + kc * 8;
        dst[i] = r * LDS + kc * 8;
    }
    float acc[2][8][4];
    const bool warp_live = row0 + wm * 32 < row_end;
    tile_mainloop<false, TK, STAGES, PER_THREAD>(As, Bs, a_src, b_src, a_live, dst, K, warp_live, wm, wn, lane, acc);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = row0 + wm * 32 + mt * 16 + (lane >> 2) + half * 8;
            if (r >= row_end) continue;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int n = n0 + wn * 64 + nt * 8 + 2 * (lane & 3) + c;
                    if (n >= N) continue;
                    float v = acc[mt][nt][half * 2 + c];
                    if (gate != nullptr) v = v * (1.f / (1.f + expf(-to_f32(gate[(size_t)r * ldg + (size_t)g * N + n])))) * out_scale;
                    const size_t o = ((size_t)r * G + g) * N + n;
                    if (OUT_F32) reinterpret_cast<float*>(out)[o] = v;
                    else reinterpret_cast<bf16*>(out)[o] = __float2bfloat16_rn(v);
                }
        }
}

// As zllm_gemm_heads (gemm_grouped.cu) for bfloat16 x, w and gate; out float32 or bfloat16.
ZLLM_API int zllm_gemm_heads_mma(const void* x, int ldx, int xg, const void* w, void* out, const void* gate, int ldg,
                                 float out_scale, int T, int N, int K, int G, int out_f32, void* stream) {
    if (T <= 0 || N <= 0 || G <= 0) return 0;
    if (K <= 0 || (K % 32) || (ldx % 8) || (xg % 8) || (((uintptr_t)x | (uintptr_t)w) & 15)) return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const bool few = K % 64 == 0;
    const size_t smem = few ? (size_t)3 * (TM + TN) * 72 * sizeof(bf16) : (size_t)3 * (TM + TN) * 40 * sizeof(bf16);
    static bool raised = false;
    if (!raised) {
        const int big = 3 * (TM + TN) * 72 * (int)sizeof(bf16), small = 3 * (TM + TN) * 40 * (int)sizeof(bf16);
        cudaError_t e = cudaFuncSetAttribute(gemm_heads_mma_kernel<true, 32, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, small);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_heads_mma_kernel<false, 32, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, small);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_heads_mma_kernel<true, 64, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_heads_mma_kernel<false, 64, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    dim3 grid((N + TN - 1) / TN, (T + TM - 1) / TM, G);
#define GH_GO(F32, TKV) return launch_pdl(gemm_heads_mma_kernel<F32, TKV, 3>, grid, dim3(256), smem, s, (const bf16*)x, ldx, xg, \
                                          (const bf16*)w, out, (const bf16*)gate, ldg, out_scale, T, N, K, G)
    if (out_f32 && few) GH_GO(true, 64);
    if (out_f32) GH_GO(true, 32);
    if (few) GH_GO(false, 64);
    GH_GO(false, 32);
#undef GH_GO
}
