// Routing of a mixture of experts: router scores, the choice of experts, the sorting of
// (token, choice) pairs by expert, and the weighted sum of the experts' outputs.
//
//   moe_route:    z = Wr h in float32, s = softmax(z) over all E experts, or s = sigmoid(z) one by
//                 one.  Experts form ``groups`` equal groups of neighbours; a group counts by its
//                 largest score; only experts of the ``keep`` best groups can be chosen (groups =
//                 keep = 1: no restriction).  The ``top`` largest scores among those are chosen,
//                 lowest index first on ties; their weights are the scores, divided by their sum
//                 (+ 1e-20) if asked.  Behind them every row gets ``n_shared`` more choices, the
//                 experts E, E+1, ... that every token visits, with the weight 1 or, when the
//                 router matrix has a row E for it, sigmoid(z_E): the gate of the shared expert.
//   moe_sort:     a counting sort of the T*top pairs by expert: off[E+1], perm[T*top].
//   moe_combine:  out[t] (+)= scale * sum_j weight[t][j] * y[t*top + j], j in order; the first
//                 ``n_unit`` choices count with weight 1 (their weight went into the expert's input).
#include "common.cuh"
#include <math.h>

#define MOE_MAX_E 1024

// eight consecutive values as float32 (16-byte aligned for bfloat16, 32 for float32)
__device__ __forceinline__ void moe_load8(const bf16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void moe_load8(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

template <typename AT>
__global__ void __launch_bounds__(256) moe_route_kernel(const AT* h, const AT* __restrict__ wr, int* idx, float* wt, int H,
                                                        int E, int top, int groups, int keep, int vec, int sigmoid_scores,
                                                        int normalise, int n_shared, int shared_gate) {
    __shared__ float sc[MOE_MAX_E + 1];
    __shared__ float gs[MOE_MAX_E];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const AT* hr = h + (size_t)t * H;
    const int n_cols = top + n_shared;                // choices per row
    for (int e = warp; e < E + (shared_gate ? 1 : 0); e += nw) {
        const AT* w = wr + (size_t)e * H;
        float dot = 0.f;
        if (vec) {                                   // pieces of eight values, a lane's pieces 256 apart
#pragma unroll 4
            for (int i = lane * 8; i < H; i += 256) {       // unrolled: several pairs of loads in flight
                float a[8], b[8];
                moe_load8(hr + i, a);
                moe_load8(w + i, b);
#pragma unroll
                for (int x = 0; x < 8; ++x) dot = fmaf(a[x], b[x], dot);
            }
        } else {
            for (int i = lane; i < H; i += 32) dot = fmaf(to_f32(hr[i]), to_f32(w[i]), dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) sc[e] = dot;
    }
    __syncthreads();
    if (warp != 0) return;
    // the choices every row has: the shared expert's pieces, behind its own gate if it has one
    const float shared_w = shared_gate ? 1.f / (1.f + expf(-sc[E])) : 1.f;
    for (int c = lane; c < n_shared; c += 32) {
        idx[(size_t)t * n_cols + top + c] = E + c;
        wt[(size_t)t * n_cols + top + c] = shared_w;
    }
    if (sigmoid_scores) {
        for (int e = lane; e < E; e += 32) sc[e] = 1.f / (1.f + expf(-sc[e]));
        __syncwarp();
    } else {
        // softmax over the experts
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, sc[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float p = expf(sc[e] - mx); sc[e] = p; sum += p; }
        sum = warp_sum(sum);
        __syncwarp();
        for (int e = lane; e < E; e += 32) sc[e] = sc[e] / sum;
        __syncwarp();
    }
    // groups: the best ``keep`` by their largest score; the others' experts are struck out
    const int per = E / groups;
    if (groups > 1 && keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            float b = -1.f;
            for (int i = 0; i < per; ++i) b = fmaxf(b, sc[g * per + i]);
            gs[g] = b;
        }
        __syncwarp();
        // a group stays if fewer than ``keep`` groups beat it (lower index wins a tie)
        for (int g = lane; g < groups; g += 32) {
            const float mine = gs[g];
            int better = 0;
            for (int o = 0; o < groups; ++o) better += (gs[o] > mine) || (gs[o] == mine && o < g);
            if (better >= keep)
                for (int i = 0; i < per; ++i) sc[g * per + i] = -2.f - sc[g * per + i];   // struck out, value kept
        }
        __syncwarp();
    }
    // the ``top`` largest allowed scores, one at a time (a NaN score is never chosen; if nothing
    // is left the lowest free index is taken so that the list always names valid experts)
    float total = 0.f;
    for (int j = 0; j < top; ++j) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = sc[e];
            if (v >= 0.f && (v > bv || (v == bv && e < bi))) { bv = v; bi = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) { bi = j < E ? j : 0; bv = 0.f; }
        if (lane == 0) {
            idx[(size_t)t * n_cols + j] = bi;
            wt[(size_t)t * n_cols + j] = bv;
            sc[bi] = -1.f;
        }
        total += bv;
        __syncwarp();
    }
    if (normalise) {
        const float inv = 1.f / (total + 1e-20f);
        for (int j = lane; j < top; j += 32) wt[(size_t)t * n_cols + j] *= inv;
    }
}

// idx, wt: [T, top + n_shared].  wr: [E (+ 1 with shared_gate), H].
ZLLM_API int zllm_moe_route(const void* h, const void* wr, int* idx, float* wt, int T, int H, int E, int top, int groups,
                            int keep, int sigmoid_scores, int normalise, int n_shared, int shared_gate, int is_bf16,
                            void* stream) {
    if (T <= 0) return 0;
    if (E <= 0 || E + n_shared > MOE_MAX_E || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||
        top > keep * (E / groups) || n_shared < 0 || (shared_gate && n_shared == 0))
        return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = (H % 8 == 0 && (((uintptr_t)h | (uintptr_t)wr) % (is_bf16 ? 16 : 32)) == 0) ? 1 : 0;
    if (is_bf16)
        return launch_pdl(moe_route_kernel<bf16>, dim3(T), dim3(256), 0, s, (const bf16*)h, (const bf16*)wr, idx, wt, H, E, top,
                          groups, keep, vec, sigmoid_scores, normalise, n_shared, shared_gate);
    return launch_pdl(moe_route_kernel<float>, dim3(T), dim3(256), 0, s, (const float*)h, (const float*)wr, idx, wt, H, E, top,
                      groups, keep, vec, sigmoid_scores, normalise, n_shared, shared_gate);
}

// One block.  The order of pairs inside an expert's range depends on the atomics; no result
// does, since every pair's outputs are computed from its own row alone.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* idx, int* off, int* perm, int n, int E) {
    __shared__ int cnt[MOE_MAX_E + 1];
    __shared__ int cur[MOE_MAX_E];
    pdl_trigger();
    pdl_wait();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[min(max(idx[i], 0), E - 1)], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) { const int c = cnt[e]; cnt[e] = run; cur[e] = run; run += c; }
        cnt[E] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) off[e] = cnt[e];
    for (int i = threadIdx.x; i < n; i += blockDim.x) perm[atomicAdd(&cur[min(max(idx[i], 0), E - 1)], 1)] = i;
}

ZLLM_API int zllm_moe_sort(const int* idx, int* off, int* perm, int n_pairs, int E, void* stream) {
    if (n_pairs <= 0) return 0;
    if (E <= 0 || E > MOE_MAX_E) return ZLLM_ERR_UNSUPPORTED;
    return launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, idx, off, perm, n_pairs, E);
}

__global__ void __launch_bounds__(256) moe_combine_kernel(const float* y, const float* wt, float* residual, int H, int top,
                                                          float scale, int n_unit, int overwrite) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float s = 0.f;
        for (int j = 0; j < top; ++j)
            s = fmaf(j < n_unit ? 1.f : wt[(size_t)t * top + j], y[((size_t)t * top + j) * H + c], s);
        if (overwrite) residual[(size_t)t * H + c] = scale * s;
        else residual[(size_t)t * H + c] += scale * s;
    }
}

// top: choices per row (shared ones included); the first n_unit of them are summed with weight 1
ZLLM_API int zllm_moe_combine(const float* y, const float* wt, float* residual, int T, int H, int top, float scale,
                              int n_unit, int overwrite, void* stream) {
    if (T <= 0) return 0;
    return launch_pdl(moe_combine_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, y, wt, residual, H, top, scale, n_unit,
                      overwrite);
}
