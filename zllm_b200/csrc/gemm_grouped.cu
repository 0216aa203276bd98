// Many small products in one launch, on CUDA cores with float32 accumulation.
//
//   per head:   out[t][g*N + n] = sum_k x[t][g*xg + k] * W[g][n][k]          (g = head)
//               optionally times sigmoid(gate[t][g*N + n]) * out_scale: an output gate.
//   per expert: rows are (token, choice) pairs sorted by their expert; expert e owns the sorted
//               range off[e]..off[e+1]-1; sorted entry i stands for pair perm[i].
//               first product:   act[i][n]      = silu(c x[perm[i]/top] . Wg[e][n]) * (c x[perm[i]/top] . Wu[e][n])   (gated)
//                           or   act[i][n]      = f(c x[perm[i]/top] . Wu[e][n]),  f = silu, gelu (erf) or gelu (tanh)
//                                c = row_scale[perm[i]] for the first n_scaled choices of a token, else 1: a router
//                                weight that multiplies what the expert READS (applied to the float32 sums)
//               second product:  y[perm[i]][n]  = act[i] . Wd[e][n]
//
// Every output element is accumulated by one thread over k = 0..K-1 in that order, so its
// value depends on its own operand rows only, never on the batch around it (as gemm_plain.cu).
#include "common.cuh"

#define GB 64        // tile rows and columns
#define GK 16

// activations of an expert without a gate matrix
#define ACT_SILU 0
#define ACT_GELU 1
#define ACT_GELU_TANH 2
__device__ __forceinline__ float expert_act(float z, int act) {
    if (act == ACT_GELU) return 0.5f * z * (1.f + erff(z * 0.70710678118654752440f));
    if (act == ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
    return z / (1.f + expf(-z));
}

// The inner tile: 256 threads, 4x4 outputs each; a(r, k) and b(c, k) fetch operand elements.
template <bool DUAL, typename FA, typename FB, typename FU>
__device__ __forceinline__ void tile_product(int K, FA a, FB b, FU u, float (&acc)[4][4], float (&accu)[4][4]) {
    __shared__ float xs[GK][GB + 1];
    __shared__ float ws[GK][GB + 1];
    __shared__ float us[DUAL ? GK : 1][GB + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    for (int k0 = 0; k0 < K; k0 += GK) {
        for (int i = threadIdx.x; i < GB * GK; i += 256) {
            const int r = i / GK, c = i - r * GK;
            xs[c][r] = (k0 + c < K) ? a(r, k0 + c) : 0.f;
            ws[c][r] = (k0 + c < K) ? b(r, k0 + c) : 0.f;
            if (DUAL) us[c][r] = (k0 + c < K) ? u(r, k0 + c) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            float av[4], bv[4], uv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = ws[kk][tx * 4 + j];
            if (DUAL) {
#pragma unroll
                for (int j = 0; j < 4; ++j) uv[j] = us[kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
                    if (DUAL) accu[i][j] = fmaf(av[i], uv[j], accu[i][j]);
                }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------- per head
template <typename AT, typename WT, typename OT>
__global__ void __launch_bounds__(256) gemm_heads_kernel(const AT* x, int ldx, int xg, const WT* __restrict__ w, OT* out,
                                                         const AT* gate, int ldg, float out_scale, int T, int N, int K, int G) {
    pdl_trigger();
    pdl_wait();
    const int g = blockIdx.z;
    const int m0 = blockIdx.y * GB, n0 = blockIdx.x * GB;
    const AT* xb = x + (size_t)g * xg;
    const WT* wb = w + (size_t)g * N * K;
    float acc[4][4] = {}, accu[4][4];
    auto a = [&](int r, int k) { const int m = m0 + r; return m < T ? to_f32(xb[(size_t)m * ldx + k]) : 0.f; };
    auto b = [&](int c, int k) { const int n = n0 + c; return n < N ? to_f32(wb[(size_t)n * K + k]) : 0.f; };
    tile_product<false>(K, a, b, b, acc, accu);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            const size_t o = ((size_t)m * G + g) * N + n;
            float v = acc[i][j];
            if (gate != nullptr) v = v * (1.f / (1.f + expf(-to_f32(gate[(size_t)m * ldg + (size_t)g * N + n])))) * out_scale;
            out[o] = from_f32<OT>(v);
        }
    }
}

// x [T, ldx] with head g's K inputs at column g*xg; w [G, N, K]; out [T, G*N]; gate (may be null)
// of x's dtype, row t at gate + t*ldg, G*N entries.  x_f32 / out_f32: those operands are float32 whatever ``is_bf16`` says
// about the weights (and the gate).
ZLLM_API int zllm_gemm_heads(const void* x, int ldx, int xg, const void* w, void* out, const void* gate, int ldg, float out_scale,
                             int T, int N, int K, int G, int is_bf16, int x_f32, int out_f32, void* stream) {
    if (T <= 0 || N <= 0 || G <= 0) return 0;
    if (K <= 0 || (gate != nullptr && x_f32 && is_bf16)) return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((N + GB - 1) / GB, (T + GB - 1) / GB, G);
#define GH_GO(AT, WT, OT) return launch_pdl(gemm_heads_kernel<AT, WT, OT>, grid, dim3(256), 0, s, (const AT*)x, ldx, xg, \
                                            (const WT*)w, (OT*)out, (const AT*)gate, ldg, out_scale, T, N, K, G)
    if (!is_bf16) GH_GO(float, float, float);
    if (x_f32 && out_f32) GH_GO(float, bf16, float);
    if (x_f32) GH_GO(float, bf16, bf16);
    if (out_f32) GH_GO(bf16, bf16, float);
    GH_GO(bf16, bf16, bf16);
#undef GH_GO
}

// ---------------------------------------------------------------- per expert
// Tile ``blockIdx.y`` of the launch is tile (e, mt) of the experts' row ranges taken in order;
// tiles beyond the last one return at once (the launch is sized for the worst case).
template <typename AT, typename OT, bool SWIGLU>
__global__ void __launch_bounds__(256) gemm_experts_kernel(const AT* x, const AT* __restrict__ w, const AT* __restrict__ wu, OT* out,
                                                           const int* off, const int* perm, int top, int gather,
                                                           int scatter, int E, int N, int K, const float* row_scale,
                                                           int n_scaled, int act) {
    __shared__ int s_e, s_row0;
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x == 0) {
        int tile = blockIdx.y, e = 0;
        for (; e < E; ++e) {
            const int tiles = (off[e + 1] - off[e] + GB - 1) / GB;
            if (tile < tiles) break;
            tile -= tiles;
        }
        s_e = e;
        s_row0 = e < E ? off[e] + tile * GB : 0;
    }
    __syncthreads();
    const int e = s_e;
    if (e >= E) return;
    const int row0 = s_row0, row_end = off[e + 1];
    const int n0 = blockIdx.x * GB;
    const AT* wb = w + (size_t)e * N * K;
    const AT* ub = SWIGLU ? wu + (size_t)e * N * K : nullptr;
    float acc[4][4] = {}, accu[4][4] = {};
    auto a = [&](int r, int k) {
        const int i = row0 + r;
        if (i >= row_end) return 0.f;
        const size_t src = gather ? (size_t)(perm[i] / top) : (size_t)i;
        return to_f32(x[src * K + k]);
    };
    auto b = [&](int c, int k) { const int n = n0 + c; return n < N ? to_f32(wb[(size_t)n * K + k]) : 0.f; };
    auto u = [&](int c, int k) { const int n = n0 + c; return n < N ? to_f32(ub[(size_t)n * K + k]) : 0.f; };
    tile_product<SWIGLU>(K, a, b, u, acc, accu);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        if (r >= row_end) continue;
        const size_t orow = scatter ? (size_t)perm[r] : (size_t)r;
        float c = 1.f;
        if (gather && row_scale != nullptr && perm[r] % top < n_scaled) c = row_scale[perm[r]];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j] * c;
            if (SWIGLU) v = v / (1.f + expf(-v)) * (accu[i][j] * c);
            else if (gather) v = expert_act(v, act);
            out[orow * N + n] = from_f32<OT>(v);
        }
    }
}

// n_pairs = tokens * top sorted entries.
// mode 1 (gated first product): w and wu are the experts' gate and up matrices [E, N, K], rows of x are
//   gathered (x[perm[i] / top]), out [n_pairs, N] in sorted order, of x's dtype.
// mode 2 (first product without a gate): the same with w alone and the activation ``act``.
// mode 0 (second product): x [n_pairs, K] in sorted order, out [n_pairs, N] float32 scattered to perm[i].
// row_scale (may be null) [n_pairs] by pair: multiplies the input of the first n_scaled choices of every token.
ZLLM_API int zllm_gemm_experts(const void* x, const void* w, const void* wu, void* out, const int* off, const int* perm,
                               int top, int n_pairs, int E, int N, int K, int mode, const float* row_scale, int n_scaled,
                               int act, int is_bf16, void* stream) {
    if (n_pairs <= 0 || N <= 0) return 0;
    if (K <= 0 || E <= 0 || top <= 0 || mode < 0 || mode > 2 || act < 0 || act > 2) return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((N + GB - 1) / GB, (n_pairs + GB - 1) / GB + E);
    if (mode == 1) {
        if (is_bf16)
            return launch_pdl(gemm_experts_kernel<bf16, bf16, true>, grid, dim3(256), 0, s, (const bf16*)x, (const bf16*)w,
                              (const bf16*)wu, (bf16*)out, off, perm, top, 1, 0, E, N, K, row_scale, n_scaled, act);
        return launch_pdl(gemm_experts_kernel<float, float, true>, grid, dim3(256), 0, s, (const float*)x, (const float*)w,
                          (const float*)wu, (float*)out, off, perm, top, 1, 0, E, N, K, row_scale, n_scaled, act);
    }
    if (mode == 2) {
        if (is_bf16)
            return launch_pdl(gemm_experts_kernel<bf16, bf16, false>, grid, dim3(256), 0, s, (const bf16*)x, (const bf16*)w,
                              (const bf16*)nullptr, (bf16*)out, off, perm, top, 1, 0, E, N, K, row_scale, n_scaled, act);
        return launch_pdl(gemm_experts_kernel<float, float, false>, grid, dim3(256), 0, s, (const float*)x, (const float*)w,
                          (const float*)nullptr, (float*)out, off, perm, top, 1, 0, E, N, K, row_scale, n_scaled, act);
    }
    if (is_bf16)
        return launch_pdl(gemm_experts_kernel<bf16, float, false>, grid, dim3(256), 0, s, (const bf16*)x, (const bf16*)w,
                          (const bf16*)nullptr, (float*)out, off, perm, top, 0, 1, E, N, K, (const float*)nullptr, 0, 0);
    return launch_pdl(gemm_experts_kernel<float, float, false>, grid, dim3(256), 0, s, (const float*)x, (const float*)w,
                      (const float*)nullptr, (float*)out, off, perm, top, 0, 1, E, N, K, (const float*)nullptr, 0, 0);
}
