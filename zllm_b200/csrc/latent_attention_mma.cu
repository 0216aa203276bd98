// Attention through a cached latent on tensor cores (bfloat16 operands, float32 scores, softmax
// and accumulation).  The math is that of latent_attention.cu: one shared "kv head" whose cache
// row is [c (RANK) | kr (rot)]; the queries arrive on the latent side (q_lat, float32) with their
// rotated part still to rotate; out[t, h] = sum_j softmax_j(scale q_abs[t, h] . row_j) c_j.
//
// Since every head reads the same keys, the HEADS are the rows of the tensor-core tile: a CTA takes
// one row of the step and a group of 16 heads (M = 16, the native height of mma.sync m16n8k16),
// walks the row's keys in blocks of 32 through a two-stage cp.async ring, and
//   S = Q K^T:  warp w takes 16 of the block's keys and one half of the rank + rot inner steps; the
//               two halves are added in a fixed order when the scores are read back;
//   softmax:    every warp reads all 16 x 32 scores from shared memory (the same values in every
//               warp), keeps the running maximum and sum of its rows, and packs P as its A operand;
//   O += P V:   warp w owns RANK / 4 columns of the latent; V is the key tile itself, read with
//               ldmatrix.trans.
// With few rows in a step (decoding) the keys of a row are divided into splits (whole key blocks) over
// gridDim.z; the partial (maximum, sum, O) of the splits are merged by a second kernel.
// Sizes: RANK in {64, 128, 256, 512}, rot a multiple of 16; others go to the CUDA-core kernel.
#include "attention_common.cuh"

#define LM_KEYS 32
#define LM_HEADS 16
#define LM_MAXHALF 128          // rotated pairs per head at most

__device__ __forceinline__ void lm_cp_async16(void* dst, const void* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void lm_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void lm_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

template <int RANK>
__global__ void __launch_bounds__(128) latent_attention_mma_kernel(
    const float* q_lat, const bf16* q, int ldq, int q_off, bf16* out, float* part_o, float* part_ml, const int* positions,
    const int* row_slot, const bf16* pages, const int* __restrict__ table, int max_blocks, int bs, int n_heads, int rot,
    const float* __restrict__ freq, float mag, int dims, float scale, int n_splits, int split_keys, int bs_shift) {
    extern __shared__ __align__(16) unsigned char lm_smem[];
    const int D = RANK + rot, LDK = D + 8;
    bf16* Qs = reinterpret_cast<bf16*>(lm_smem);                       // [16][LDK]
    bf16* Ks = Qs + LM_HEADS * LDK;                                    // [2][LM_KEYS][LDK]
    float* Ss = reinterpret_cast<float*>(Ks + 2 * LM_KEYS * LDK);      // [2][16][LM_KEYS + 1]
    constexpr int SP = LM_KEYS + 1;
    pdl_trigger();
    const int t = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int slot = row_slot[t];
    const int pos = positions[t];
    pdl_wait();
    const int r0 = lane >> 2, qd = lane & 3;                           // the thread's rows r0, r0 + 8; its column pair
    constexpr int NT = RANK / 32;                                      // 8-column tiles of O per warp
    const int colbase = warp * (RANK / 4);
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    const int k_begin = split * split_keys;
    const int k_end = slot < 0 ? 0 : min(pos + 1, n_splits > 1 ? k_begin + split_keys : pos + 1);
    if (k_begin < k_end) {
        // ---- the queries of the 16 heads: latent side as given, rotated side rotated here (the row's
        //      cosines and sines once, for all heads)
        __shared__ float rc[LM_MAXHALF], rs[LM_MAXHALF];
        const int half = dims >> 1;
        for (int j = tid; j < half; j += 128) {
            const float ang = __fmul_rn((float)pos, freq[j]);
            rc[j] = cosf(ang) * mag;
            rs[j] = sinf(ang) * mag;
        }
        __syncthreads();
        for (int i = tid; i < LM_HEADS * D; i += 128) {
            const int row = i / D, d = i - row * D;
            const int h = g * LM_HEADS + row;
            float v = 0.f;
            if (h < n_heads) {
                if (d < RANK) v = q_lat[((size_t)t * n_heads + h) * RANK + d];
                else {
                    const bf16* qr = q + (size_t)t * ldq + (size_t)h * q_off + (q_off - rot);
                    const int e = d - RANK;
                    if (e < dims) {
                        const int j = e < half ? e : e - half;
                        const float a = to_f32(qr[j]), b = to_f32(qr[j + half]);
                        v = e < half ? a * rc[j] - b * rs[j] : b * rc[j] + a * rs[j];
                    } else v = to_f32(qr[e]);
                }
            }
            Qs[row * LDK + d] = __float2bfloat16_rn(v);
        }
        const int* trow = table + (size_t)slot * max_blocks;
        const int chunks = D / 8;                                      // 16-byte pieces of a cache row
        // a warp brings in every fourth key of the block: one page lookup per key, the lanes over its pieces
        auto load_block = [&](int st, int base) {
            bf16* dst = Ks + st * LM_KEYS * LDK;
            for (int j = warp; j < LM_KEYS; j += 4) {
                const int key = base + j;
                // page and place in the page: shifts when the page size is a power of two (bs_shift >= 0)
                const int blk_i = bs_shift >= 0 ? key >> bs_shift : key / bs;
                const int in_page = bs_shift >= 0 ? key & (bs - 1) : key - blk_i * bs;
                int page = -1;
                if (key < k_end) page = trow[blk_i];
                const bf16* src = pages + ((size_t)(page >= 0 ? page : 0) * bs + in_page) * D;
                for (int c = lane; c < chunks; c += 32) {
                    if (page >= 0) lm_cp_async16(dst + j * LDK + c * 8, src + c * 8);
                    else *reinterpret_cast<uint4*>(dst + j * LDK + c * 8) = make_uint4(0u, 0u, 0u, 0u);   // no key: zeros, never garbage
                }
            }
        };
        const int n_blocks = (k_end - k_begin + LM_KEYS - 1) / LM_KEYS;
        load_block(0, k_begin);
        lm_commit();
        // scores are kept in units of log2 (scale * log2 e), so that the exponentials are one ex2 each, as in the
        // framework's other tensor-core attention kernels; the maxima of the splits are in the same units
        const float scale2 = scale * 1.4426950408889634f;
        const int ksteps = D / 16, ks_half = (ksteps + 1) / 2;
        const int kh = warp & 1, part = warp >> 1;
        const int ks0 = part * ks_half, ks1 = min(ksteps, ks0 + ks_half);
        for (int blk = 0; blk < n_blocks; ++blk) {
            const int base = k_begin + blk * LM_KEYS;
            if (blk + 1 < n_blocks) load_block((blk + 1) & 1, base + LM_KEYS);
            lm_commit();
            lm_wait<1>();
            __syncthreads();                                           // the block's keys (and, first time, Qs) are visible
            const bf16* Kst = Ks + (blk & 1) * LM_KEYS * LDK;
            // ---- scores of 16 keys over this warp's half of the inner steps
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            for (int ks = ks0; ks < ks1; ++ks) {
                unsigned a[4], b[4];
                ldmatrix_x4(a, Qs + (lane & 15) * LDK + ks * 16 + (lane >> 4) * 8);
                ldmatrix_x4(b, Kst + (kh * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + ks * 16 + ((lane >> 3) & 1) * 8);
                mma16816(s[0], a, b[0], b[1]);
                mma16816(s[1], a, b[2], b[3]);
            }
            float* sp = Ss + part * LM_HEADS * SP;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int key = kh * 16 + nt * 8 + 2 * qd + c;
                    sp[r0 * SP + key] = s[nt][c];
                    sp[(r0 + 8) * SP + key] = s[nt][2 + c];
                }
            __syncthreads();
            // ---- softmax of the thread's two rows over the block's 32 keys; P as the A operand
            const int n_valid = min(LM_KEYS, k_end - base);
            float p[2][8];
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int rr = 0; rr < 2; ++rr)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int key = (e >> 2) * 16 + ((e >> 1) & 1) * 8 + 2 * qd + (e & 1);
                    const int row = r0 + rr * 8;
                    const float v = (Ss[row * SP + key] + Ss[LM_HEADS * SP + row * SP + key]) * scale2;
                    p[rr][e] = key < n_valid ? v : -INFINITY;
                    mx[rr] = fmaxf(mx[rr], p[rr][e]);
                }
            unsigned pa[2][4];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
                const float m_new = fmaxf(m_run[rr], mx[rr]);
                const float corr = ex2_approx(m_run[rr] - m_new);          // 2^(-inf) = 0 at the first block
                float sum = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    p[rr][e] = ex2_approx(p[rr][e] - m_new);               // a masked key: 2^(-inf) = 0
                    sum += p[rr][e];
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                l_run[rr] = l_run[rr] * corr + sum;
                m_run[rr] = m_new;
#pragma unroll
                for (int i = 0; i < NT; ++i) { o[i][2 * rr] *= corr; o[i][2 * rr + 1] *= corr; }
            }
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2) {
                pa[j2][0] = pack_bf16(p[0][j2 * 4 + 0], p[0][j2 * 4 + 1]);
                pa[j2][1] = pack_bf16(p[1][j2 * 4 + 0], p[1][j2 * 4 + 1]);
                pa[j2][2] = pack_bf16(p[0][j2 * 4 + 2], p[0][j2 * 4 + 3]);
                pa[j2][3] = pack_bf16(p[1][j2 * 4 + 2], p[1][j2 * 4 + 3]);
            }
            // ---- O += P V over this warp's columns of the latent
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2)
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    unsigned b[4];
                    ldmatrix_x4_trans(b, Kst + (j2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + colbase + np * 16 + (lane >> 4) * 8);
                    mma16816(o[2 * np], pa[j2], b[0], b[1]);
                    mma16816(o[2 * np + 1], pa[j2], b[2], b[3]);
                }
            __syncthreads();                                           // the stage and the scores may be written again
        }
        lm_wait<0>();
    }
    // ---- results: the output itself with one split, else the split's partial
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int h = g * LM_HEADS + r0 + rr * 8;
        if (h >= n_heads) continue;
        if (n_splits == 1) {
            const float inv = l_run[rr] > 0.f ? 1.f / l_run[rr] : 0.f;
            bf16* orow = out + ((size_t)t * n_heads + h) * RANK + colbase;
#pragma unroll
            for (int i = 0; i < NT; ++i)
                *reinterpret_cast<__nv_bfloat162*>(orow + i * 8 + 2 * qd) =
                    __floats2bfloat162_rn(o[i][2 * rr] * inv, o[i][2 * rr + 1] * inv);
        } else {
            const size_t idx = ((size_t)t * n_heads + h) * n_splits + split;
            float* prow = part_o + idx * RANK + colbase;
#pragma unroll
            for (int i = 0; i < NT; ++i) *reinterpret_cast<float2*>(prow + i * 8 + 2 * qd) = make_float2(o[i][2 * rr], o[i][2 * rr + 1]);
            if (warp == 0 && qd == 0) { part_ml[idx * 2] = m_run[rr]; part_ml[idx * 2 + 1] = l_run[rr]; }
        }
    }
}

// out[t, h] = sum_s w_s O_s / sum_s w_s l_s with w_s = 2^(m_s - max m) (the maxima are in units of log2), splits in order.
template <int RANK>
__global__ void __launch_bounds__(128) latent_merge_kernel(const float* part_o, const float* part_ml, bf16* out, int n_splits) {
    __shared__ float wgt[64];                            // a split's weight, once for all columns (n_splits <= 64)
    __shared__ float inv_s;
    pdl_trigger();
    pdl_wait();
    const size_t th = blockIdx.x;                        // (row, head)
    const float* ml = part_ml + th * n_splits * 2;
    if (threadIdx.x < 32) {
        float M = -INFINITY;
        for (int s = threadIdx.x; s < n_splits; s += 32) M = fmaxf(M, ml[2 * s]);
        M = warp_max(M);
        float den = 0.f;
        for (int s = threadIdx.x; s < n_splits; s += 32) {
            const float w = ml[2 * s] == -INFINITY ? 0.f : exp2f(ml[2 * s] - M);
            wgt[s] = w;
            den += w * ml[2 * s + 1];
        }
        den = warp_sum(den);
        if (threadIdx.x == 0) inv_s = den > 0.f ? 1.f / den : 0.f;
    }
    __syncthreads();
    const float inv = inv_s;
    for (int d = threadIdx.x; d < RANK; d += 128) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) acc = fmaf(wgt[s], part_o[(th * n_splits + s) * RANK + d], acc);
        out[th * RANK + d] = __float2bfloat16_rn(acc * inv);
    }
}

template <int RANK>
static int launch_latent_mma(const float* q_lat, const void* q, int ldq, int q_off, void* out, float* part_o, float* part_ml,
                             const int* positions, const int* row_slot, const void* pages, const int* table, int max_blocks,
                             int bs, int T, int n_heads, int rot, const float* freq, float mag, int dims, float scale,
                             int n_splits, int split_keys, cudaStream_t s) {
    const int D = RANK + rot;
    const size_t smem = (size_t)(LM_HEADS + 2 * LM_KEYS) * (D + 8) * sizeof(bf16) + 2 * LM_HEADS * (LM_KEYS + 1) * sizeof(float);
    if (smem > 200 * 1024) return ZLLM_ERR_UNSUPPORTED;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel<RANK>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    int bs_shift = -1;
    if (bs > 0 && (bs & (bs - 1)) == 0) { bs_shift = 0; while ((1 << bs_shift) < bs) ++bs_shift; }
    int code = launch_pdl(latent_attention_mma_kernel<RANK>, dim3(T, (n_heads + LM_HEADS - 1) / LM_HEADS, n_splits), dim3(128), smem, s,
                          q_lat, (const bf16*)q, ldq, q_off, (bf16*)out, part_o, part_ml, positions, row_slot, (const bf16*)pages,
                          table, max_blocks, bs, n_heads, rot, freq, mag, dims, scale, n_splits, split_keys, bs_shift);
    if (code || n_splits == 1) return code;
    return launch_pdl(latent_merge_kernel<RANK>, dim3(T * n_heads), dim3(128), 0, s, (const float*)part_o, (const float*)part_ml,
                      (bf16*)out, n_splits);
}

// As zllm_latent_attention (latent_attention.cu), bfloat16 only.  n_splits > 1: the keys of a row
// are taken in splits of split_keys; part_o [T, heads, n_splits, rank] and part_ml [T, heads,
// n_splits, 2] float32 are scratch.
ZLLM_API int zllm_latent_attention_mma(const float* q_lat, const void* q, int ldq, int q_off, void* out, float* part_o,
                                       float* part_ml, const int* positions, const int* row_slot, const void* pages,
                                       const int* table, int max_blocks, int bs, int T, int n_heads, int rank, int rot,
                                       const float* freq, float mag, int dims, float scale, int n_splits, int split_keys,
                                       void* stream) {
    if (T <= 0) return 0;
    if (dims > rot || (dims & 1) || dims > 2 * LM_MAXHALF || (rot % 16) || n_heads <= 0 || rot > q_off || n_splits < 1 || n_splits > 64 || (n_splits > 1 && split_keys % LM_KEYS) ||
        (((uintptr_t)pages | (uintptr_t)out | (uintptr_t)part_o) & 15))
        return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
#define LM_GO(R) return launch_latent_mma<R>(q_lat, q, ldq, q_off, out, part_o, part_ml, positions, row_slot, pages, table, \
                                             max_blocks, bs, T, n_heads, rot, freq, mag, dims, scale, n_splits, split_keys, s)
    if (rank == 64) LM_GO(64);
    if (rank == 128) LM_GO(128);
    if (rank == 256) LM_GO(256);
    if (rank == 512) LM_GO(512);
#undef LM_GO
    return ZLLM_ERR_UNSUPPORTED;
}
