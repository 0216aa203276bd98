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
//
// bfloat16 with key and value sizes that are multiples of 16 (up to 128) runs on tensor cores
// (mma.sync m16n8k16, float32 scores, softmax and sums):
//   prompt portions  one CTA per (tile of 128 query rows of a portion, query head), eight warps of 16
//                    rows; keys and values come in blocks of 64 through a three-stage cp.async ring,
//                    gathered through the block table; only the blocks that hold a kept first
//                    position or a key of the tile's window are visited, and only blocks that touch
//                    an edge of some row's visibility pay for the masking.
//   decoded rows     one CTA per (row, kv head); the query heads that share the kv head are the rows of
//                    the tile, so keys and values are read once for the group; the warps (eight, or four at the
//                    largest sizes) take the visible blocks of 32 keys in turn, two stages each, with their own running maximum and sums,
//                    and merge in warp order at the end.  A window bounds a row's keys, so there are no
//                    splits over CTAs and no merge kernel.
// The softmax weights stay 32-bit through the second product: a weight goes to the tensor cores as
// the sum of two bfloat16 numbers (its rounding and the rounding of what is left), two MMAs per tile.
#include "attention_common.cuh"
#include <cuda_pipeline.h>

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

// ---------------------------------------------------------------- tensor cores (bfloat16)
#define WA_PF_ROWS 128          // query rows of a tile (= the host's QUERY_TILE)
#define WA_PF_KEYS 64           // keys of a block in prompt portions
#define WA_DEC_KEYS 32          // keys of a block in decoding
#define WA_DEC_WARPS 4

template <int VMAX>
struct WaState {
    float m[2], l[2];
    float o[VMAX / 8][4];
    __device__ __forceinline__ void init() {
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
#pragma unroll
        for (int i = 0; i < VMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    }
};

// Where key ``key`` of the request lies in the pools: (page * nkv + kvh) * bs + position in the page, or -1 when
// the key is beyond ``key_hi`` or its page has gone back to the pool.
__device__ __forceinline__ long long wa_locate(const int* __restrict__ trow, int key, int key_hi, int bs, int nkv, int kvh) {
    if (key > key_hi) return -1;
    const int blk = key / bs;
    const int page = trow[blk];
    return page >= 0 ? ((long long)page * nkv + kvh) * bs + (key - blk * bs) : -1;
}

// A block of 64 keys and their values into shared tiles [64][str] by 256 threads: four threads per row, ONE table
// lookup per thread (the row's place serves its key and its value), then independent 16-byte async copies;
// a row without a page becomes zeros.
__device__ __forceinline__ void wa_gather_block64(bf16* ktile, int strk, bf16* vtile, int strv, const bf16* k_pages,
                                                  const bf16* v_pages, const int* __restrict__ trow, int key0, int key_hi,
                                                  int bs, int nkv, int kvh, int dk, int dv, int tid) {
    const int r = tid >> 2, part = tid & 3;
    const long long at = wa_locate(trow, key0 + r, key_hi, bs, nkv, kvh);
    bf16* kd = ktile + r * strk;
    bf16* vd = vtile + r * strv;
    if (at >= 0) {
        const bf16* ks = k_pages + at * dk;
        const bf16* vs = v_pages + at * dv;
        for (int c = part; c < (dk >> 3); c += 4) __pipeline_memcpy_async(kd + c * 8, ks + c * 8, 16);
        for (int c = part; c < (dv >> 3); c += 4) __pipeline_memcpy_async(vd + c * 8, vs + c * 8, 16);
    } else {
        for (int c = part; c < (dk >> 3); c += 4) *reinterpret_cast<uint4*>(kd + c * 8) = make_uint4(0, 0, 0, 0);
        for (int c = part; c < (dv >> 3); c += 4) *reinterpret_cast<uint4*>(vd + c * 8) = make_uint4(0, 0, 0, 0);
    }
}

// 32 rows of keys OR values by one warp: lane r has looked up row r's place (``at``); the lanes then walk the
// rows' 16-byte pieces in order (consecutive lanes, consecutive pieces of a row), each fetching the place of its
// piece's row from the lane that holds it.
__device__ __forceinline__ void wa_gather_rows32(bf16* tile, int str, const bf16* pages, long long at, int d, int lane) {
    const int chunks = d >> 3;
    for (int it = 0; it < chunks; ++it) {                    // 32 * chunks pieces, 32 per pass
        const int c = lane + 32 * it;
        const int r = c / chunks, ch = c - r * chunks;
        const long long a = __shfl_sync(0xffffffffu, at, r);
        bf16* dst = tile + r * str + ch * 8;
        if (a >= 0) __pipeline_memcpy_async(dst, pages + a * d + ch * 8, 16);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
}

// Scores of the warp's 16 rows against a block of NB keys.
template <int KMAX, int NB>
__device__ __forceinline__ void wa_scores(const unsigned (&qf)[KMAX / 16][4], const bf16* ks, int strk, int nk16, int lane,
                                          float (&s)[NB / 8][4]) {
    const int lrow = lane & 7, lmat = lane >> 3;
#pragma unroll
    for (int j = 0; j < NB / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KMAX / 16; ++kk) {
        if (kk < nk16) {
#pragma unroll
            for (int j = 0; j < NB / 8; j += 2) {
                // matrices: (keys 8j.., entries 16kk..), (keys 8j.., 16kk+8..), (keys 8j+8.., 16kk..), (.., +8)
                unsigned b[4];
                ldmatrix_x4(b, ks + (8 * j + (lmat >> 1) * 8 + lrow) * strk + 16 * kk + (lmat & 1) * 8);
                mma16816(s[j], qf[kk], b[0], b[1]);
                mma16816(s[j + 1], qf[kk], b[2], b[3]);
            }
        }
    }
}

// Masking, the running softmax in float32 (log2 domain; ``scale`` holds log2 e) and O += P V for one block.
// pos_r: the position of the lane's two rows (g and g + 8), -1 for a row that does not exist.
template <int VMAX, int NB>
__device__ __forceinline__ void wa_softmax_pv(float (&s)[NB / 8][4], const bf16* vs, int strv, int nv8, int key0,
                                              const int (&pos_r)[2], int window, int keep, bool masked, float scale,
                                              WaState<VMAX>& st, int lane) {
    const int t = lane & 3;
    const int lrow = lane & 7, lmat = lane >> 3;
    float mx[2] = {-INFINITY, -INFINITY};
    if (masked) {
#pragma unroll
        for (int j = 0; j < NB / 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                const int key = key0 + 8 * j + 2 * t + (e & 1);
                const int p = pos_r[r];
                const bool seen = key <= p && (window <= 0 || key > p - window || key < keep);
                if (!seen) s[j][e] = -INFINITY;
                mx[r] = fmaxf(mx[r], s[j][e]);
            }
    } else {
#pragma unroll
        for (int j = 0; j < NB / 8; ++j) {
            mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
            mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
        }
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(st.m[r], mx[r] * scale);
        corr[r] = (m_new == -INFINITY) ? 1.f : ex2_approx(st.m[r] - m_new);
        msafe[r] = (m_new == -INFINITY) ? 0.f : m_new;
        st.m[r] = m_new;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NB / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const float p = ex2_approx(fmaf(s[j][e], scale, -msafe[r]));     // 2^(-inf) = 0 for hidden keys
            s[j][e] = p;
            rs[r] += p;
        }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
        st.l[r] = st.l[r] * corr[r] + rs[r];
    }
#pragma unroll
    for (int i = 0; i < VMAX / 8; ++i) {
        st.o[i][0] *= corr[0]; st.o[i][1] *= corr[0];
        st.o[i][2] *= corr[1]; st.o[i][3] *= corr[1];
    }
    // O += P V.  A weight p goes in as hi + lo, hi = bf16(p), lo = bf16(p - hi): 16 bits of it reach the sum.
#pragma unroll
    for (int kk = 0; kk < NB / 16; ++kk) {
        unsigned hi[4], lo[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float a = s[2 * kk + (q >> 1)][(q & 1) * 2], b = s[2 * kk + (q >> 1)][(q & 1) * 2 + 1];
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(a, b);
            const float2 hf = __bfloat1622float2(h2);
            hi[q] = *reinterpret_cast<const unsigned*>(&h2);
            lo[q] = pack_bf16(a - hf.x, b - hf.y);
        }
#pragma unroll
        for (int i = 0; i < VMAX / 8; i += 2) {
            if (i < nv8) {
                // matrices: (keys 16kk.., entries 8i..), (keys 16kk+8.., 8i..), (keys 16kk.., 8i+8..), (.., +8)
                unsigned b[4];
                ldmatrix_x4_trans(b, vs + (16 * kk + (lmat & 1) * 8 + lrow) * strv + 8 * i + (lmat >> 1) * 8);
                mma16816(st.o[i], hi, b[0], b[1]);
                mma16816(st.o[i], lo, b[0], b[1]);
                mma16816(st.o[i + 1], hi, b[2], b[3]);
                mma16816(st.o[i + 1], lo, b[2], b[3]);
            }
        }
    }
}

// The A fragments of one 16-row query tile straight from global memory: row_ptr[r] points at the head's
// entries of the lane's row r (g or g + 8), or is null for a row that does not exist.
template <int KMAX>
__device__ __forceinline__ void wa_load_q(unsigned (&qf)[KMAX / 16][4], const bf16* const (&row_ptr)[2], int nk16, int lane) {
    const int t = lane & 3;
#pragma unroll
    for (int kk = 0; kk < KMAX / 16; ++kk)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const bf16* rp = row_ptr[q & 1];
            qf[kk][q] = (kk < nk16 && rp != nullptr) ? *reinterpret_cast<const unsigned*>(rp + 16 * kk + (q >> 1) * 8 + 2 * t) : 0u;
        }
}

// Visible blocks of NB keys for queries at positions p_lo..p_hi: first those that hold kept first positions
// and lie below the window's first block, then the window's blocks.  Block i of the list:
__device__ __forceinline__ int wa_block_of(int i, int n_kept, int first_win) { return i < n_kept ? i : first_win + (i - n_kept); }

#define WA_PF_STAGES 3
template <int KMAX, int VMAX>
__global__ void __launch_bounds__(256, (KMAX + VMAX <= 128) ? 2 : 1) window_attention_prefill_kernel(
    const bf16* proj, int ld, int off_g, bf16* out, const int* __restrict__ tiles, const bf16* k_pages, const bf16* v_pages,
    const int* __restrict__ table, int max_blocks, int bs, int nq, int nkv, int dk, int dv, float scale, int window, int keep) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_trigger();
    // the list runs from a portion's first tile to its last, and later tiles see more keys: the grid walks it
    // backwards, so that the longest tiles start first and the short ones fill the tail
    const int* tl = tiles + 4 * (gridDim.x - 1 - blockIdx.x);
    const int row0 = tl[0], n_rows = tl[1], slot = tl[2], p0 = tl[3];
    pdl_wait();
    if (n_rows <= 0 || slot < 0) return;                      // an empty tile of a bucketed list
    const int h = blockIdx.y, kvh = h / (nq / nkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int strk = dk + 8, strv = dv + 8, nk16 = dk >> 4, nv8 = dv >> 3;
    bf16* ksm = reinterpret_cast<bf16*>(smem_raw);                        // [stages][64][strk]
    bf16* vsm = ksm + WA_PF_STAGES * WA_PF_KEYS * strk;                   // [stages][64][strv]
    const int* trow = table + (size_t)slot * max_blocks;
    const int p_hi = p0 + n_rows - 1;
    const int lo_tile = window > 0 ? max(0, p0 - window + 1) : 0;
    const int first_win = lo_tile / WA_PF_KEYS, last_win = p_hi / WA_PF_KEYS;
    const int n_kept = min((min(keep, lo_tile) + WA_PF_KEYS - 1) / WA_PF_KEYS, first_win);
    const int nb = n_kept + last_win - first_win + 1;
    // the warp's rows
    int pos_r[2];
    const bf16* qrow[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int lr = warp * 16 + g + 8 * r;
        pos_r[r] = lr < n_rows ? p0 + lr : -1;
        qrow[r] = lr < n_rows ? proj + (size_t)(row0 + lr) * ld + (size_t)h * dk : nullptr;
    }
    unsigned qf[KMAX / 16][4];
    wa_load_q<KMAX>(qf, qrow, nk16, lane);
    const bool warp_live = warp * 16 < n_rows;
    const int wp_lo = p0 + warp * 16, wp_hi = min(p0 + warp * 16 + 15, p_hi);     // positions of the warp's rows
    WaState<VMAX> st;
    st.init();
    auto load = [&](int i, int stage) {
        const int key0 = wa_block_of(i, n_kept, first_win) * WA_PF_KEYS;
        wa_gather_block64(ksm + stage * WA_PF_KEYS * strk, strk, vsm + stage * WA_PF_KEYS * strv, strv, k_pages, v_pages, trow,
                          key0, p_hi, bs, nkv, kvh, dk, dv, tid);
        __pipeline_commit();
    };
    // a ring of three stages, two blocks ahead, ONE barrier per block: the stage that block i + 2 is copied into
    // was read last for block i - 1, which every warp has finished when it passes the barrier of block i
    load(0, 0);
    if (nb > 1) load(1, 1);
    else __pipeline_commit();
    for (int i = 0; i < nb; ++i) {
        __pipeline_wait_prior(1);                            // block i has landed (block i + 1 may still be on its way)
        __syncthreads();
        if (i + 2 < nb) load(i + 2, (i + 2) % WA_PF_STAGES);
        else __pipeline_commit();
        const int stage = i % WA_PF_STAGES;
        const int key0 = wa_block_of(i, n_kept, first_win) * WA_PF_KEYS;
        // the warp skips a block none of its rows sees; it masks only at an edge of some row's visibility
        const bool any = key0 <= wp_hi && (window <= 0 || key0 + WA_PF_KEYS - 1 > wp_lo - window || key0 < keep);
        if (warp_live && any) {
            const bool inner = key0 + WA_PF_KEYS - 1 <= wp_lo && warp * 16 + 15 < n_rows &&
                               (window <= 0 || key0 > wp_hi - window || key0 + WA_PF_KEYS - 1 < keep);
            float s[WA_PF_KEYS / 8][4];
            wa_scores<KMAX, WA_PF_KEYS>(qf, ksm + stage * WA_PF_KEYS * strk, strk, nk16, lane, s);
            wa_softmax_pv<VMAX, WA_PF_KEYS>(s, vsm + stage * WA_PF_KEYS * strv, strv, nv8, key0, pos_r, window, keep, !inner,
                                            scale, st, lane);
        }
    }
    __pipeline_wait_prior(0);
    // epilogue: 1 / l, the head's gate, bfloat16
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int lr = warp * 16 + g + 8 * r;
        if (lr >= n_rows) continue;
        float f = st.l[r] > 0.f ? 1.f / st.l[r] : 0.f;
        if (off_g >= 0) f *= 1.f / (1.f + expf(-to_f32(proj[(size_t)(row0 + lr) * ld + off_g + h])));
        bf16* o = out + ((size_t)(row0 + lr) * nq + h) * dv;
#pragma unroll
        for (int i = 0; i < VMAX / 8; ++i)
            if (i < nv8)
                *reinterpret_cast<unsigned*>(o + 8 * i + 2 * t) = pack_bf16(st.o[i][2 * r] * f, st.o[i][2 * r + 1] * f);
    }
}

template <int KMAX, int VMAX, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) window_attention_decode_kernel(
    const bf16* proj, int ld, int off_g, bf16* out, const int* rows, const int* positions, const int* row_slot,
    const bf16* k_pages, const bf16* v_pages, const int* __restrict__ table, int max_blocks, int bs, int nq, int nkv, int dk,
    int dv, float scale, int window, int keep) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_trigger();
    const int row = rows[blockIdx.x];                        // inputs of the step: read before the wait
    const int slot = row_slot[row];
    const int pos = positions[row];
    pdl_wait();
    const int kvh = blockIdx.y, G = nq / nkv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    if (slot < 0) {                                          // a padding row of a graph bucket
        for (int i = tid; i < G * dv; i += blockDim.x) out[((size_t)row * nq + (size_t)kvh * G) * dv + i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int strk = dk + 8, strv = dv + 8, nk16 = dk >> 4, nv8 = dv >> 3;
    // per warp two stages of [32][strk] keys + [32][strv] values: the next block's rows are on their way while
    // this one's are multiplied
    bf16* wsm = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * 2 * WA_DEC_KEYS * (strk + strv);
    const int* trow = table + (size_t)slot * max_blocks;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int first_win = lo / WA_DEC_KEYS, last_win = pos / WA_DEC_KEYS;
    const int n_kept = min((min(keep, lo) + WA_DEC_KEYS - 1) / WA_DEC_KEYS, first_win);
    const int nb = n_kept + last_win - first_win + 1;
    // the tile's rows are the query heads of this kv head
    int pos_r[2];
    const bf16* qrow[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int hr = g + 8 * r;
        pos_r[r] = hr < G ? pos : -1;
        qrow[r] = hr < G ? proj + (size_t)row * ld + (size_t)(kvh * G + hr) * dk : nullptr;
    }
    unsigned qf[KMAX / 16][4];
    wa_load_q<KMAX>(qf, qrow, nk16, lane);
    WaState<VMAX> st;
    st.init();
    auto issue = [&](int i, int stage) {                     // two copy groups per block: its keys, then its values
        bf16* ksm = wsm + (size_t)stage * WA_DEC_KEYS * (strk + strv);
        const int key0 = wa_block_of(i, n_kept, first_win) * WA_DEC_KEYS;
        const long long at = wa_locate(trow, key0 + lane, pos, bs, nkv, kvh);
        wa_gather_rows32(ksm, strk, k_pages, at, dk, lane);
        __pipeline_commit();
        wa_gather_rows32(ksm + WA_DEC_KEYS * strk, strv, v_pages, at, dv, lane);
        __pipeline_commit();
    };
    if (warp < nb) issue(warp, 0);
    int n = 0;
    for (int i = warp; i < nb; i += WARPS, ++n) {
        const int stage = n & 1;
        if (i + WARPS < nb) issue(i + WARPS, stage ^ 1);
        else { __pipeline_commit(); __pipeline_commit(); }
        const bf16* ksm = wsm + (size_t)stage * WA_DEC_KEYS * (strk + strv);
        const bf16* vsm = ksm + WA_DEC_KEYS * strk;
        const int key0 = wa_block_of(i, n_kept, first_win) * WA_DEC_KEYS;
        __pipeline_wait_prior(3);                           // this block's keys are there
        __syncwarp();
        float s[WA_DEC_KEYS / 8][4];
        wa_scores<KMAX, WA_DEC_KEYS>(qf, ksm, strk, nk16, lane, s);
        __pipeline_wait_prior(2);                           // and its values
        __syncwarp();
        const bool inner = key0 + WA_DEC_KEYS - 1 <= pos && G == 16 &&
                           (window <= 0 || key0 > pos - window || key0 + WA_DEC_KEYS - 1 < keep);
        wa_softmax_pv<VMAX, WA_DEC_KEYS>(s, vsm, strv, nv8, key0, pos_r, window, keep, !inner, scale, st, lane);
        __syncwarp();                                        // the stage is free for the block after next
    }
    __pipeline_wait_prior(0);
    // merge the warps' partial results in warp order through shared memory (over the tiles, which are done)
    __syncthreads();
    float* part = reinterpret_cast<float*>(smem_raw);                    // [warps][16][dv + 2]
    const int pstr = dv + 2;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float* pr = part + ((size_t)warp * 16 + g + 8 * r) * pstr;
#pragma unroll
        for (int i = 0; i < VMAX / 8; ++i)
            if (i < nv8) { pr[8 * i + 2 * t] = st.o[i][2 * r]; pr[8 * i + 2 * t + 1] = st.o[i][2 * r + 1]; }
        if (t == 0) { pr[dv] = st.m[r]; pr[dv + 1] = st.l[r]; }
    }
    __syncthreads();
    for (int i = tid; i < G * dv; i += blockDim.x) {
        const int hr = i / dv, d = i - hr * dv;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, part[((size_t)w * 16 + hr) * pstr + dv]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float* pr = part + ((size_t)w * 16 + hr) * pstr;
            const float f = pr[dv] == -INFINITY ? 0.f : exp2f(pr[dv] - M);
            num += pr[d] * f;
            den += pr[dv + 1] * f;
        }
        float f = den > 0.f ? 1.f / den : 0.f;
        const int h = kvh * G + hr;
        if (off_g >= 0) f *= 1.f / (1.f + expf(-to_f32(proj[(size_t)row * ld + off_g + h])));
        out[((size_t)row * nq + h) * dv + d] = __float2bfloat16_rn(num * f);
    }
}

// bfloat16 on tensor cores.  rows [n_decode]: the step's rows that are single decoded tokens; tiles [n_tiles][4]:
// [first row, rows, slot, position of the first row] of the portions' query tiles (empty tiles are skipped).
// Takes dk, dv multiples of 16 up to 128, nq / nkv <= 16 and scale > 0; other sizes are refused.
ZLLM_API int zllm_window_attention_bf16(const void* proj, int ld, int off_g, void* out, const int* rows, int n_decode,
                                        const int* tiles, int n_tiles, const int* positions, const int* row_slot,
                                        const void* k_pages, const void* v_pages, const int* table, int max_blocks, int bs,
                                        int nq, int nkv, int dk, int dv, float scale, int window, int keep_first, void* stream) {
    if (n_decode <= 0 && n_tiles <= 0) return 0;
    if (dk <= 0 || dv <= 0 || (dk % 16) || (dv % 16) || dk > 128 || dv > 128 || nkv <= 0 || nq % nkv || nq / nkv > 16 ||
        !(scale > 0.f) || keep_first < 0 || (ld % 2) || (off_g >= 0 && off_g + nq > ld) ||
        (((uintptr_t)proj | (uintptr_t)out | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15))
        return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const float sc = scale * 1.4426950408889634f;
    const size_t pf_smem = (size_t)WA_PF_STAGES * WA_PF_KEYS * ((dk + 8) + (dv + 8)) * sizeof(bf16);
    // decoding: eight warps per CTA while their tiles fit into 160 KB, else four (the grid is only rows x kv heads,
    // so the warps of a CTA are what keeps copies in flight)
    const size_t warp_tiles = (size_t)2 * WA_DEC_KEYS * ((dk + 8) + (dv + 8)) * sizeof(bf16);
    const int dec_warps = 8 * warp_tiles <= 160 * 1024 ? 8 : WA_DEC_WARPS;
    const size_t tiles_b = dec_warps * warp_tiles;
    const size_t merge_b = (size_t)dec_warps * 16 * (dv + 2) * sizeof(float);
    const size_t dec_smem = tiles_b > merge_b ? tiles_b : merge_b;
    static bool raised = false;
    if (!raised) {
        const int most = 160 * 1024;     // >= four warps' tiles at the largest sizes, eight warps' up to the limit above, the portions' three stages
        cudaError_t e = cudaSuccess;
#define WA_ATTR(KM, VM) \
        if (e == cudaSuccess) e = cudaFuncSetAttribute(window_attention_prefill_kernel<KM, VM>, cudaFuncAttributeMaxDynamicSharedMemorySize, most); \
        if (e == cudaSuccess) e = cudaFuncSetAttribute(window_attention_decode_kernel<KM, VM, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, most); \
        if (e == cudaSuccess) e = cudaFuncSetAttribute(window_attention_decode_kernel<KM, VM, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        WA_ATTR(64, 64) WA_ATTR(64, 128) WA_ATTR(128, 64) WA_ATTR(128, 128)
#undef WA_ATTR
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    int rc = 0;
#define WA_GO(KM, VM) do { \
        if (n_decode > 0 && dec_warps == 8) \
            rc = launch_pdl(window_attention_decode_kernel<KM, VM, 8>, dim3(n_decode, nkv), dim3(256), dec_smem, s, \
                            (const bf16*)proj, ld, off_g, (bf16*)out, rows, positions, row_slot, (const bf16*)k_pages, \
                            (const bf16*)v_pages, table, max_blocks, bs, nq, nkv, dk, dv, sc, window, keep_first); \
        else if (n_decode > 0) \
            rc = launch_pdl(window_attention_decode_kernel<KM, VM, 4>, dim3(n_decode, nkv), dim3(128), dec_smem, s, \
                            (const bf16*)proj, ld, off_g, (bf16*)out, rows, positions, row_slot, (const bf16*)k_pages, \
                            (const bf16*)v_pages, table, max_blocks, bs, nq, nkv, dk, dv, sc, window, keep_first); \
        if (rc == 0 && n_tiles > 0) \
            rc = launch_pdl(window_attention_prefill_kernel<KM, VM>, dim3(n_tiles, nq), dim3(256), pf_smem, s, (const bf16*)proj, \
                            ld, off_g, (bf16*)out, tiles, (const bf16*)k_pages, (const bf16*)v_pages, table, max_blocks, bs, nq, \
                            nkv, dk, dv, sc, window, keep_first); \
        return rc; } while (0)
    if (dk <= 64 && dv <= 64) WA_GO(64, 64);
    if (dk <= 64) WA_GO(64, 128);
    if (dv <= 64) WA_GO(128, 64);
    WA_GO(128, 128);
#undef WA_GO
}
