// Attention over the paged cache with a sliding window that keeps the first positions, value
// heads of a size of their own and an output gate per head.
//
// The step's rows come as ONE projection array ``proj`` [T, ld]: per row the query heads
// [nq * dk], the key heads at column off_k [nkv * dk], the value heads at off_v [nkv * dv] and,
// if the mixer has them, the gate logits at off_g [nq].  Two kernels:
//
//   rotate_store_kv   rotates the first ``dims`` entries of every query and key head in place by the
//                     angle position * f_i (formed in float32; pairs (2i, 2i+1) or (i, i + dims/2)),
//                     then writes the row's keys and values into the page of its position:
//                     keys  [page][kv head][position in page][dk],
//                     values [page][kv head][position in page][dv].
//   window_attention  query at position p of a request sees key j iff j <= p and
//                     (p - j < window or j < keep_first); window <= 0: every j <= p.  Scores
//                     q.k * scale, softmax and the weighted sum in float32 with a running maximum;
//                     the head's result times sigmoid(gate logit) when there are gates.
//
// The plain kernel gives a warp to every (row, query head) and walks the visible keys 32 at a
// time, first the kept ones below the window, then the window, so the order of every sum is
// fixed by the row's own position: a row's result does not depend on the batch around it, on
// how its prompt was cut, or on which pages hold its keys.  It serves the 32-bit path and every
// size; pages that the window has passed (table entry < 0) are never touched.
#include "common.cuh"
#include <math.h>

#define WA_MAX_D 256

// ---------------------------------------------------------------- rotation + cache write
template <typename AT>
__global__ void __launch_bounds__(256) rotate_store_kv_kernel(
    AT* proj, int ld, int off_k, int off_v, const int* positions, const int* row_slot, const float* __restrict__ freq,
    float magnitude, int dims, int interleaved, AT* k_pages, AT* v_pages, const int* __restrict__ table, int max_blocks,
    int bs, int nq, int nkv, int dk, int dv, int store) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int slot = row_slot[t];                 // inputs of the step: read before the wait
    const int pos = positions[t];
    int page = -1;
    if (store && slot >= 0) page = table[(size_t)slot * max_blocks + pos / bs];
    pdl_wait();
    if (slot < 0) return;                         // padding row of a graph bucket
    AT* row = proj + (size_t)t * ld;
    const int half = dims >> 1;
    if (half > 0) {
        const int pairs = (nq + nkv) * half;
        for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
            const int head = i / half, j = i - head * half;
            AT* h = head < nq ? row + (size_t)head * dk : row + off_k + (size_t)(head - nq) * dk;
            const int ia = interleaved ? 2 * j : j;
            const int ib = interleaved ? 2 * j + 1 : j + half;
            float sn, cs;
            sincosf((float)pos * freq[j], &sn, &cs);
            sn *= magnitude;
            cs *= magnitude;
            const float a = to_f32(h[ia]), b = to_f32(h[ib]);
            h[ia] = from_f32<AT>(a * cs - b * sn);
            h[ib] = from_f32<AT>(b * cs + a * sn);
        }
    }
    if (!store || page < 0) return;               // the host guarantees a page; never write through a bad id
    __syncthreads();                              // the rotated keys are visible to all threads of the row
    const int in_page = pos % bs;
    const AT* k = row + off_k;
    const AT* v = row + off_v;
    for (int i = threadIdx.x; i < nkv * dk; i += blockDim.x) {
        const int kvh = i / dk, d = i - kvh * dk;
        k_pages[(((size_t)page * nkv + kvh) * bs + in_page) * dk + d] = k[i];
    }
    for (int i = threadIdx.x; i < nkv * dv; i += blockDim.x) {
        const int kvh = i / dv, d = i - kvh * dv;
        v_pages[(((size_t)page * nkv + kvh) * bs + in_page) * dv + d] = v[i];
    }
}

ZLLM_API int zllm_rotate_store_kv(void* proj, int ld, int off_k, int off_v, const int* positions, const int* row_slot,
                                  const float* freq, float magnitude, int dims, int interleaved, void* k_pages, void* v_pages,
                                  const int* table, int max_blocks, int bs, int T, int nq, int nkv, int dk, int dv, int store,
                                  int is_bf16, void* stream) {
    if (T <= 0) return 0;
    if (dims < 0 || dims > dk || (dims & 1) || dk <= 0 || dv <= 0 || nq <= 0 || nkv <= 0 ||
        off_k < nq * dk || off_v < off_k + nkv * dk || off_v + nkv * dv > ld || (dims > 0 && freq == nullptr))
        return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (is_bf16)
        return launch_pdl(rotate_store_kv_kernel<bf16>, dim3(T), dim3(256), 0, s, (bf16*)proj, ld, off_k, off_v, positions,
                          row_slot, freq, magnitude, dims, interleaved, (bf16*)k_pages, (bf16*)v_pages, table, max_blocks, bs,
                          nq, nkv, dk, dv, store);
    return launch_pdl(rotate_store_kv_kernel<float>, dim3(T), dim3(256), 0, s, (float*)proj, ld, off_k, off_v, positions,
                      row_slot, freq, magnitude, dims, interleaved, (float*)k_pages, (float*)v_pages, table, max_blocks, bs, nq,
                      nkv, dk, dv, store);
}

// ---------------------------------------------------------------- the plain kernel
// One warp per (row, query head).  The running state (m, l, acc) is carried over the chunks of 32
// keys of both stretches, the kept first positions below the window and then the window itself.
template <typename AT>
__global__ void __launch_bounds__(128) window_attention_plain_kernel(
    const AT* proj, int ld, int off_g, AT* out, const int* positions, const int* row_slot, const AT* k_pages,
    const AT* v_pages, const int* __restrict__ table, int max_blocks, int bs, int nq, int nkv, int dk, int dv, float scale,
    int window, int keep_first) {
    __shared__ float qs[4][WA_MAX_D];
    pdl_trigger();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * 4 + warp;
    const int slot = row_slot[t];
    const int pos = positions[t];
    pdl_wait();
    if (h >= nq) return;
    AT* o = out + ((size_t)t * nq + h) * dv;
    if (slot < 0) {
        for (int d = lane; d < dv; d += 32) o[d] = from_f32<AT>(0.f);
        return;
    }
    const int kvh = h / (nq / nkv);
    const AT* q = proj + (size_t)t * ld + (size_t)h * dk;
    for (int d = lane; d < dk; d += 32) qs[warp][d] = to_f32(q[d]);
    __syncwarp();
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int kept_end = min(keep_first, lo);               // kept positions that the window does not cover anyway
    const int* trow = table + (size_t)slot * max_blocks;
    float m = -INFINITY, l = 0.f;
    float acc[WA_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < WA_MAX_D / 32; ++i) acc[i] = 0.f;
    for (int stretch = 0; stretch < 2; ++stretch) {
        const int first = stretch == 0 ? 0 : lo;
        const int last = stretch == 0 ? kept_end - 1 : pos;         // inclusive
        for (int base = first; base <= last; base += 32) {
            const int key = base + lane;
            long long at = -1;                                      // (page * nkv + kvh) * bs + position in page
            float s = -INFINITY;
            if (key <= last) {
                const int page = trow[key / bs];
                if (page >= 0) {
                    at = ((long long)page * nkv + kvh) * bs + (key % bs);
                    const AT* k = k_pages + at * dk;
                    float dot = 0.f;
                    for (int d = 0; d < dk; ++d) dot = fmaf(qs[warp][d], to_f32(k[d]), dot);
                    s = dot * scale;
                }
            }
            const float m_new = fmaxf(m, warp_max(s));
            const float p = (at >= 0) ? expf(s - m_new) : 0.f;
            const float corr = (m_new == -INFINITY) ? 1.f : expf(m - m_new);    // first chunk: m = -inf, exp(-inf) = 0
            l = l * corr + warp_sum(p);
#pragma unroll
            for (int i = 0; i < WA_MAX_D / 32; ++i) acc[i] *= corr;
            const int n = min(32, last - base + 1);
            for (int j = 0; j < n; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
                const long long aj = __shfl_sync(0xffffffffu, at, j);
                if (aj < 0) continue;
                const AT* v = v_pages + aj * dv;
#pragma unroll
                for (int i = 0; i < WA_MAX_D / 32; ++i) {
                    const int d = lane + 32 * i;
                    if (d < dv) acc[i] = fmaf(pj, to_f32(v[d]), acc[i]);
                }
            }
            m = m_new;
        }
    }
    float inv = l > 0.f ? 1.f / l : 0.f;
    if (off_g >= 0) inv *= 1.f / (1.f + expf(-to_f32(proj[(size_t)t * ld + off_g + h])));
#pragma unroll
    for (int i = 0; i < WA_MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) o[d] = from_f32<AT>(acc[i] * inv);
    }
}

// out [T, nq * dv].  off_g < 0: no gates.
ZLLM_API int zllm_window_attention_plain(const void* proj, int ld, int off_g, void* out, const int* positions,
                                         const int* row_slot, const void* k_pages, const void* v_pages, const int* table,
                                         int max_blocks, int bs, int T, int nq, int nkv, int dk, int dv, float scale, int window,
                                         int keep_first, int is_bf16, void* stream) {
    if (T <= 0) return 0;
    if (dk > WA_MAX_D || dv > WA_MAX_D || dk <= 0 || dv <= 0 || nkv <= 0 || nq % nkv || keep_first < 0 ||
        (off_g >= 0 && off_g + nq > ld))
        return ZLLM_ERR_UNSUPPORTED;
    dim3 grid(T, (nq + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (is_bf16)
        return launch_pdl(window_attention_plain_kernel<bf16>, grid, dim3(128), 0, s, (const bf16*)proj, ld, off_g, (bf16*)out,
                          positions, row_slot, (const bf16*)k_pages, (const bf16*)v_pages, table, max_blocks, bs, nq, nkv, dk,
                          dv, scale, window, keep_first);
    return launch_pdl(window_attention_plain_kernel<float>, grid, dim3(128), 0, s, (const float*)proj, ld, off_g, (float*)out,
                      positions, row_slot, (const float*)k_pages, (const float*)v_pages, table, max_blocks, bs, nq, nkv, dk, dv,
                      scale, window, keep_first);
}
