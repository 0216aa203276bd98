// Attention through a low-rank latent, over the paged cache.
//
// A position's cache row is [c (rank entries) | kr (rot entries)]: the normed latent from which
// every head's keys and values are linear maps (k_h = Uk_h c, v_h = Uv_h c), and one rotated key
// part shared by all heads.  The maps are moved to the query side and behind the weighted sum:
//     score_h(i, j) = scale * ( (Uk_h^T q_h(i)) . c(j) + qr_h(i) . kr(j) )
//     out_h(i)      = Uv_h * sum_j softmax_j(score_h(i, .)) c(j)
// so the attention itself is one shared "kv head" with keys of rank + rot entries whose first
// rank entries are also the values; nothing but c and kr is ever cached or expanded.
//
//   latent_prepare:    per row, from the stacked down-projections: RMS-norm of the query latent,
//                      RMS-norm of c, rotation of kr, write of [c | kr] into the row's page.
//   latent_attention:  per (row, group of heads): the queries' latent side comes in float32, the
//                      rotated side is rotated here; keys in blocks of 32 through shared memory,
//                      online softmax, all in float32 and in an order fixed by the position alone.
//
// Rotation: the first ``dims`` of the rot entries, entry i with entry i + dims/2, by the angle
// position * freq[i] computed in float32 here (no table, so no largest position); cos and sin
// are multiplied by ``mag``.
#include "common.cuh"
#include <math.h>

template <typename AT>
__global__ void __launch_bounds__(256) latent_prepare_kernel(
    const AT* proj, int ldp, int off_q, int q_rank, int off_kv, int rank, int rot,
    const float* __restrict__ wq, const float* __restrict__ wc, float eps,
    const float* __restrict__ freq, float mag, int dims,
    const int* positions, const int* row_slot, AT* cq, AT* pages, const int* __restrict__ table, int max_blocks, int bs,
    int store) {
    __shared__ float red[33];
    pdl_trigger();
    const int t = blockIdx.x;
    const int slot = row_slot[t];
    const int pos = positions[t];
    pdl_wait();
    AT* cqr = cq + (size_t)t * q_rank;
    if (slot < 0) {                                   // padding row: defined values, nothing cached
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cqr[i] = from_f32<AT>(0.f);
        return;
    }
    const AT* row = proj + (size_t)t * ldp;
    float sq = 0.f, sc = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) { const float v = to_f32(row[off_q + i]); sq += v * v; }
    for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_f32(row[off_kv + i]); sc += v * v; }
    sq = block_sum(sq, red);
    sc = block_sum(sc, red);
    const float iq = 1.f / sqrtf(sq / (float)q_rank + eps);
    const float ic = 1.f / sqrtf(sc / (float)rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cqr[i] = from_f32<AT>(to_f32(row[off_q + i]) * iq * wq[i]);
    if (!store) return;
    const int page = table[(size_t)slot * max_blocks + pos / bs];
    if (page < 0) return;
    AT* dst = pages + ((size_t)page * bs + (pos % bs)) * (rank + rot);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<AT>(to_f32(row[off_kv + i]) * ic * wc[i]);
    const AT* kr = row + off_kv + rank;
    const int half = dims >> 1;
    for (int i = threadIdx.x; i < rot; i += blockDim.x) {
        float v;
        if (i < dims) {
            const int j = i < half ? i : i - half;
            const float ang = __fmul_rn((float)pos, freq[j]);
            const float c = cosf(ang) * mag, s = sinf(ang) * mag;
            const float a = to_f32(kr[j]), b = to_f32(kr[j + half]);
            v = i < half ? a * c - b * s : b * c + a * s;
        } else {
            v = to_f32(kr[i]);
        }
        dst[rank + i] = from_f32<AT>(v);
    }
}

// proj [T, ldp]: columns off_q.. (q_rank of them) are the query latent before its norm, columns
// off_kv.. are rank latent entries then rot key entries.  cq [T, q_rank] receives the normed
// query latent; pages [n_pages, bs, rank + rot] the cache rows.
ZLLM_API int zllm_latent_prepare(const void* proj, int ldp, int off_q, int q_rank, int off_kv, int rank, int rot,
                                 const float* wq, const float* wc, float eps, const float* freq, float mag, int dims,
                                 const int* positions, const int* row_slot, void* cq, void* pages, const int* table,
                                 int max_blocks, int bs, int store, int T, int is_bf16, void* stream) {
    if (T <= 0) return 0;
    if (dims > rot || (dims & 1) || q_rank <= 0 || rank <= 0) return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (is_bf16)
        return launch_pdl(latent_prepare_kernel<bf16>, dim3(T), dim3(256), 0, s, (const bf16*)proj, ldp, off_q, q_rank, off_kv,
                          rank, rot, wq, wc, eps, freq, mag, dims, positions, row_slot, (bf16*)cq, (bf16*)pages, table,
                          max_blocks, bs, store);
    return launch_pdl(latent_prepare_kernel<float>, dim3(T), dim3(256), 0, s, (const float*)proj, ldp, off_q, q_rank, off_kv,
                      rank, rot, wq, wc, eps, freq, mag, dims, positions, row_slot, (float*)cq, (float*)pages, table,
                      max_blocks, bs, store);
}

// ---------------------------------------------------------------- attention, CUDA cores
#define LA_KEYS 32

template <typename AT, int NR>      // NR: latent entries per lane (rank <= 32 * NR)
__global__ void __launch_bounds__(256) latent_attention_kernel(
    const float* q_lat, const AT* q, int ldq, int q_off, AT* out, const int* positions, const int* row_slot,
    const AT* pages, const int* __restrict__ table, int max_blocks, int bs, int n_heads, int rank, int rot,
    const float* __restrict__ freq, float mag, int dims, float scale) {
    extern __shared__ float sm[];
    const int D = rank + rot, DP = D + 1;
    const int hpb = blockDim.x >> 5;
    float* qs = sm;                                  // [hpb][DP]
    float* ks = sm + (size_t)hpb * DP;               // [LA_KEYS][DP]
    pdl_trigger();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * hpb + warp;
    const int slot = row_slot[t];
    const int pos = positions[t];
    pdl_wait();
    const bool live = h < n_heads;
    AT* o = out + ((size_t)t * n_heads + (live ? h : 0)) * rank;
    if (slot < 0) {
        if (live) for (int d = lane; d < rank; d += 32) o[d] = from_f32<AT>(0.f);
        return;
    }
    if (live) {
        const float* ql = q_lat + ((size_t)t * n_heads + h) * rank;
        for (int d = lane; d < rank; d += 32) qs[warp * DP + d] = ql[d];
        const AT* qr = q + (size_t)t * ldq + (size_t)h * q_off + (q_off - rot);      // the head's last rot entries
        const int half = dims >> 1;
        for (int i = lane; i < rot; i += 32) {
            float v;
            if (i < dims) {
                const int j = i < half ? i : i - half;
                const float ang = __fmul_rn((float)pos, freq[j]);
                const float c = cosf(ang) * mag, s = sinf(ang) * mag;
                const float a = to_f32(qr[j]), b = to_f32(qr[j + half]);
                v = i < half ? a * c - b * s : b * c + a * s;
            } else {
                v = to_f32(qr[i]);
            }
            qs[warp * DP + rank + i] = v;
        }
    }
    const int* trow = table + (size_t)slot * max_blocks;
    float m = -INFINITY, l = 0.f;
    float acc[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) acc[i] = 0.f;
    for (int base = 0; base <= pos; base += LA_KEYS) {
        const int n = min(LA_KEYS, pos - base + 1);
        __syncthreads();                              // the block before is consumed (and qs is written)
        for (int i = threadIdx.x; i < n * D; i += blockDim.x) {
            const int j = i / D, d = i - j * D;
            const int key = base + j;
            const int page = trow[key / bs];
            ks[j * DP + d] = page >= 0 ? to_f32(pages[((size_t)page * bs + (key % bs)) * D + d]) : 0.f;
        }
        __syncthreads();
        if (!live) continue;
        float s = -INFINITY;
        if (lane < n) {
            const float* kj = ks + lane * DP;
            const float* qh = qs + warp * DP;
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot = fmaf(qh[d], kj[d], dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = lane < n ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < NR; ++i) acc[i] *= corr;
        for (int j = 0; j < n; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const float* kj = ks + j * DP;
#pragma unroll
            for (int i = 0; i < NR; ++i) {
                const int d = lane + 32 * i;
                if (d < rank) acc[i] = fmaf(pj, kj[d], acc[i]);
            }
        }
        m = m_new;
    }
    if (!live) return;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) o[d] = from_f32<AT>(acc[i] * inv);
    }
}

template <typename AT, int NR>
static int launch_latent_attention(const float* q_lat, const void* q, int ldq, int q_off, void* out, const int* positions,
                                   const int* row_slot, const void* pages, const int* table, int max_blocks, int bs, int T,
                                   int n_heads, int rank, int rot, const float* freq, float mag, int dims, float scale,
                                   cudaStream_t s) {
    const int hpb = n_heads < 8 ? n_heads : 8;
    const size_t smem = (size_t)(hpb + LA_KEYS) * (rank + rot + 1) * sizeof(float);
    if (smem > 200 * 1024) return ZLLM_ERR_UNSUPPORTED;
    auto kern = latent_attention_kernel<AT, NR>;
    static size_t raised = 0;
    if (smem > 48 * 1024 && smem > raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        raised = 200 * 1024;
    }
    return launch_pdl(kern, dim3(T, (n_heads + hpb - 1) / hpb), dim3(32 * hpb), smem, s, q_lat, (const AT*)q, ldq, q_off,
                      (AT*)out, positions, row_slot, (const AT*)pages, table, max_blocks, bs, n_heads, rank, rot, freq, mag,
                      dims, scale);
}

// q_lat [T, heads, rank] float32: the queries moved to the latent side.  q [T, ldq]: the
// up-projected queries, head h at column h * q_off, its last ``rot`` entries still unrotated.
// out [T, heads, rank]: the softmax-weighted sums of the latents.
ZLLM_API int zllm_latent_attention(const float* q_lat, const void* q, int ldq, int q_off, void* out, const int* positions,
                                   const int* row_slot, const void* pages, const int* table, int max_blocks, int bs, int T,
                                   int n_heads, int rank, int rot, const float* freq, float mag, int dims, float scale,
                                   int is_bf16, void* stream) {
    if (T <= 0) return 0;
    if (dims > rot || (dims & 1) || rank <= 0 || rank > 1024 || n_heads <= 0 || rot > q_off) return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
#define LA_GO(AT, NR) return launch_latent_attention<AT, NR>(q_lat, q, ldq, q_off, out, positions, row_slot, pages, table, \
                                                             max_blocks, bs, T, n_heads, rank, rot, freq, mag, dims, scale, s)
    if (is_bf16) {
        if (rank <= 128) LA_GO(bf16, 4);
        if (rank <= 512) LA_GO(bf16, 16);
        LA_GO(bf16, 32);
    }
    if (rank <= 128) LA_GO(float, 4);
    if (rank <= 512) LA_GO(float, 16);
    LA_GO(float, 32);
#undef LA_GO
}
