// Attention over a shared low-rank latent (multi-head latent attention), CUDA cores,
// everything after the loads in 32-bit.
//
// Per token the cache keeps one row of W = rank + rot elements for all heads: the latent c
// (RMS-normed down-projection) and one rotated key part r.  Head h's key is
// [Wuk_h c | r] and its value Wuv_h c; with q_h = [a_h | b_h] (b_h rotated)
//     s_hj = (a_h . Wuk_h c_j + b_h . r_j) * scale = ((Wuk_h^T a_h) . c_j + b_h . r_j) * scale
//     o_h  = Wuv_h (sum_j p_hj c_j)
// so the kernels here work on the cached rows themselves: the query is carried into the
// latent space first (`absorb`), the attention runs as many query heads over ONE key/value
// row per position (the value is the row's first `rank` elements), and the result is
// carried out through Wuv (`expand`).  Keys and values per head are never formed.
//
// Softmax: position i sees j with 0 <= i - j < window (window <= 0: all j <= i); the
// denominator also holds exp(sink_h) when sinks are given (a learned logit without key or
// value, not scaled).
//
// Kernels:
//   latent_prep    per token: c = rms(d[:rank]) * w, r = rotate(d[rank:]) at the token's
//                  position, the row [c | r] to a dense step buffer and (optionally) to the
//                  paged cache; the rotated part of every query head is rotated in place.
//   latent_store   rows of the step buffer to the paged cache (for a ring whose rows the
//                  step's own attention still had to read).
//   latent_absorb  qa[m, h] = [Wuk_h^T a_{m,h} | b_{m,h}] in float32.
//   latent_attn    the attention; a sequence's new tokens follow `seq_start[b]` positions in
//                  the cache (rows below the start are read from pages, the others from the
//                  step buffer), any mix of starts and counts in one launch.
//   latent_expand  o[m, h] = Wuv_h ol[m, h].
#include "common.cuh"
#include "attn_decode.cuh"

namespace {

struct LatentPages {
    void* pages;                 // [n_pages, page_size, W]
    const int* page_table; int table_width; int page_size; int ring_rows; int n_pages;
    const int* seq_len;          // each sequence's length after the step (for stores into a ring)
};

template <typename T>
__device__ __forceinline__ void store_row_to_pages(const LatentPages& kv, int slot, int seq, int pos, int W, const T* row_vals,
                                                   int tid, int nthreads) {
    // in a ring only the last ring_rows positions of the sequence are kept: an older row of this step
    // must not land on the place of a newer one, whichever block runs last
    if (kv.ring_rows > 0 && pos + kv.ring_rows < kv.seq_len[seq]) return;
    const int row = kv.ring_rows > 0 ? pos % kv.ring_rows : pos;
    const int pidx = row / kv.page_size;
    if (pidx >= kv.table_width) return;
    const int page = kv.page_table[(size_t)slot * kv.table_width + pidx];
    if (page < 0 || page >= kv.n_pages) return;
    T* dst = (T*)kv.pages + ((size_t)page * kv.page_size + row % kv.page_size) * W;
    for (int i = tid; i < W; i += nthreads) dst[i] = row_vals[i];
}

// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void latent_prep_body(float* sm, const T* d, long long d_stride, T* q, long long q_stride,
                                                 int n_heads, int plain, int rank, int rot, const float* __restrict__ norm_w, float eps,
                                                 const float* __restrict__ cos_t, const float* __restrict__ sin_t, int max_pos,
                                                 const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                                 const int* __restrict__ seq_slot, T* __restrict__ lat, const LatentPages& kv) {
    const int W = rank + rot;
    float* vals = sm;                    // W floats, then 33, then W values of T
    float* red = sm + W;
    T* rounded = reinterpret_cast<T*>(red + 33);
    const int m = blockIdx.x, t = threadIdx.x, nt = blockDim.x;
    const int pos = min(max(tok_pos[m], 0), max_pos - 1);
    const int half = rot >> 1;
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;
    const T* drow = d + (size_t)m * d_stride;
    float ss = 0.f;
    for (int i = t; i < W; i += nt) {
        const float x = to_f32(drow[i]);
        vals[i] = x;
        if (i < rank) ss = fmaf(x, x, ss);
    }
    ss = block_sum(ss, red);             // (also makes vals visible)
    const float inv = rsqrtf(ss / (float)rank + eps);
    for (int i = t; i < rank; i += nt) rounded[i] = from_f32<T>(vals[i] * inv * norm_w[i]);
    for (int i = t; i < half; i += nt) {
        const float u = vals[rank + i], v = vals[rank + i + half], c = cs[i], s = sn[i];
        rounded[rank + i] = from_f32<T>(u * c - v * s);
        rounded[rank + i + half] = from_f32<T>(v * c + u * s);
    }
    __syncthreads();
    if (lat)
        for (int i = t; i < W; i += nt) lat[(size_t)m * W + i] = rounded[i];
    if (kv.pages) store_row_to_pages<T>(kv, seq_slot[tok_seq[m]], tok_seq[m], tok_pos[m], W, rounded, t, nt);
    // the rotated part of every query head, in place
    if (q) {
        const int hd = plain + rot;
        for (int idx = t; idx < n_heads * half; idx += nt) {
            const int h = idx / half, i = idx - h * half;
            T* p = q + (size_t)m * q_stride + (size_t)h * hd + plain;
            const float u = to_f32(p[i]), v = to_f32(p[i + half]), c = cs[i], s = sn[i];
            p[i] = from_f32<T>(u * c - v * s);
            p[i + half] = from_f32<T>(v * c + u * s);
        }
    }
}

template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ d, long long d_stride, T* __restrict__ q, long long q_stride,
                                   int n_heads, int plain, int rank, int rot, const float* __restrict__ norm_w, float eps,
                                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, int max_pos,
                                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                   const int* __restrict__ seq_slot, T* __restrict__ lat, LatentPages kv) {
    ti_pdl_trigger();
    extern __shared__ float sm[];
    ti_pdl_sync();
    d = ti_dependent(d); q = ti_dependent(q);
    latent_prep_body<T>(sm, d, d_stride, q, q_stride, n_heads, plain, rank, rot, norm_w, eps, cos_t, sin_t, max_pos, tok_pos, tok_seq,
                        seq_slot, lat, kv);
}

// For steps of few tokens: the work of latent_prep and latent_absorb in one launch.  Grid (tokens, heads + 1): block
// (m, h) with h < heads carries head h of token m into the latent space (the rotated part is rotated on the way, q itself
// stays as it is); block (m, heads) does the token's row.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_absorb_kernel(const T* __restrict__ d, long long d_stride, const T* __restrict__ q, long long q_stride,
                          int n_heads, int plain, int rank, int rot, const float* __restrict__ norm_w, float eps,
                          const float* __restrict__ cos_t, const float* __restrict__ sin_t, int max_pos,
                          const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                          T* __restrict__ lat, LatentPages kv, const T* __restrict__ uk, float* __restrict__ qa) {
    ti_pdl_trigger();
    extern __shared__ float sm[];
    ti_pdl_sync();
    d = ti_dependent(d); q = ti_dependent(q);
    if ((int)blockIdx.y == n_heads) {
        latent_prep_body<T>(sm, d, d_stride, (T*)nullptr, 0, n_heads, plain, rank, rot, norm_w, eps, cos_t, sin_t, max_pos, tok_pos,
                            tok_seq, seq_slot, lat, kv);
        return;
    }
    const int m = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
    const int hd = plain + rot, W = rank + rot, half = rot >> 1;
    const T* qh = q + (size_t)m * q_stride + (size_t)h * hd;
    float* qs = sm;                      // [plain]
    for (int i = t; i < plain; i += 128) qs[i] = to_f32(qh[i]);
    float* dst = qa + ((size_t)m * n_heads + h) * W;
    if (rot) {
        const int pos = min(max(tok_pos[m], 0), max_pos - 1);
        for (int i = t; i < half; i += 128) {
            // (rounded to the engine's type as the rotation in place would have left it)
            const float u = to_f32(qh[plain + i]), v = to_f32(qh[plain + i + half]);
            const float c = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
            dst[rank + i] = to_f32(from_f32<T>(u * c - v * sn));
            dst[rank + i + half] = to_f32(from_f32<T>(v * c + u * sn));
        }
    }
    __syncthreads();
    const T* ukh = uk + (size_t)h * plain * rank;
    for (int r0 = 0; r0 < rank; r0 += 128 * 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
        for (int dd = 0; dd < plain; dd++) {
            const float qv = qs[dd];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int r = r0 + t + 128 * j;
                if (r < rank) acc[j] = fmaf(qv, to_f32(ukh[(size_t)dd * rank + r]), acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int r = r0 + t + 128 * j;
            if (r < rank) dst[r] = acc[j];
        }
    }
}

// For steps of few tokens: the merge of the key splits and the way out through Wuv in one launch.  Block (token, head):
// the splits' unnormalised sums are weighed and added into the latent result (shared memory), then
// o[v] = sum_r uv[h, v, r] * result[r], a warp per output element, four elements at a time.
template <typename T>
__global__ void __launch_bounds__(128)
latent_merge_expand_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const T* __restrict__ uv,
                           T* __restrict__ o, long long o_stride, int n_heads, int vdim, int rank, int n_splits) {
    ti_pdl_trigger();
    extern __shared__ float res[];       // [rank], then [64] weights
    float* w_s = res + rank;
    ti_pdl_sync();
    part_o = ti_dependent(part_o); part_ml = ti_dependent(part_ml);
    const int b = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
    const size_t base = ((size_t)b * n_heads + h) * n_splits;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; s++) m = fmaxf(m, part_ml[(base + s) * 2]);
    float l = 0.f;
    for (int s = 0; s < n_splits; s++) {
        const float ms = part_ml[(base + s) * 2];
        const float w = ms > -INFINITY ? expf(ms - m) : 0.f;
        if (t == 0) w_s[s] = w;
        l += w > 0.f ? w * part_ml[(base + s) * 2 + 1] : 0.f;
    }
    __syncthreads();
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int e = t; e < rank; e += 128) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; s++) {
            const float w = w_s[s];
            if (w > 0.f) acc = fmaf(w, part_o[(base + s) * rank + e], acc);      // an empty split's numbers were never written
        }
        res[e] = acc * inv;
    }
    __syncthreads();
    const int warp = t >> 5, lane = t & 31;
    if (sizeof(T) == 2 && (rank & 7) == 0 && (reinterpret_cast<uintptr_t>(uv) & 15) == 0) {
        // 16-byte pieces of four rows at a time: eight loads on their way per lane
        for (int v0 = warp * 4; v0 < vdim; v0 += 16) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int c = lane; c < (rank >> 3); c += 32) {
                uint4 w[4];
#pragma unroll
                for (int j = 0; j < 4; j++)
                    w[j] = v0 + j < vdim ? reinterpret_cast<const uint4*>(uv + ((size_t)h * vdim + v0 + j) * rank)[c] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const bf16* wv = reinterpret_cast<const bf16*>(&w[j]);
#pragma unroll
                    for (int e = 0; e < 8; e++) acc[j] = fmaf(to_f32(wv[e]), res[c * 8 + e], acc[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float sum = warp_sum(acc[j]);
                if (lane == 0 && v0 + j < vdim) o[(size_t)b * o_stride + (size_t)h * vdim + v0 + j] = from_f32<T>(sum);
            }
        }
        return;
    }
    for (int v0 = warp * 4; v0 < vdim; v0 += 16) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int r = lane; r < rank; r += 32) {
            const float x = res[r];
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (v0 + j < vdim) acc[j] = fmaf(to_f32(uv[((size_t)h * vdim + v0 + j) * rank + r]), x, acc[j]);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float sum = warp_sum(acc[j]);
            if (lane == 0 && v0 + j < vdim) o[(size_t)b * o_stride + (size_t)h * vdim + v0 + j] = from_f32<T>(sum);
        }
    }
}

template <typename T>
__global__ void latent_store_kernel(const T* __restrict__ lat, int W, const int* __restrict__ tok_pos,
                                    const int* __restrict__ tok_seq, const int* __restrict__ seq_slot, LatentPages kv) {
    ti_pdl_trigger();
    ti_pdl_sync();
    lat = ti_dependent(lat);
    const int m = blockIdx.x;
    store_row_to_pages<T>(kv, seq_slot[tok_seq[m]], tok_seq[m], tok_pos[m], W, lat + (size_t)m * W, threadIdx.x, blockDim.x);
}

// ---------------------------------------------------------------------------
// qa[m, h, 0:rank] = sum_d q[m, h, d] * uk[h, d, 0:rank];  qa[m, h, rank:] = q[m, h, plain:]
// uk: [heads * plain, rank] (row (h, d)).  Grid (token tiles of TM, heads), 128 threads over the rank.
constexpr int ABS_TM = 8, ABS_THREADS = 128, ABS_RPT = 2;      // a block: 8 tokens, one head, 256 elements of the latent (grid.z)

template <typename T>
__global__ void __launch_bounds__(ABS_THREADS)
latent_absorb_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ uk, float* __restrict__ qa,
                     int M, int n_heads, int plain, int rank, int rot) {
    ti_pdl_trigger();
    extern __shared__ float qs[];        // [TM][plain]
    ti_pdl_sync();
    q = ti_dependent(q);
    const int m0 = blockIdx.x * ABS_TM, h = blockIdx.y, t = threadIdx.x;
    const int hd = plain + rot, W = rank + rot;
    for (int idx = t; idx < ABS_TM * plain; idx += ABS_THREADS) {
        const int mm = idx / plain, dd = idx - mm * plain;
        qs[idx] = (m0 + mm < M) ? to_f32(q[(size_t)(m0 + mm) * q_stride + (size_t)h * hd + dd]) : 0.f;
    }
    for (int idx = t; idx < ABS_TM * rot && blockIdx.z == 0; idx += ABS_THREADS) {
        const int mm = idx / rot, dd = idx - mm * rot;
        if (m0 + mm < M)
            qa[((size_t)(m0 + mm) * n_heads + h) * W + rank + dd] = to_f32(q[(size_t)(m0 + mm) * q_stride + (size_t)h * hd + plain + dd]);
    }
    __syncthreads();
    const T* ukh = uk + (size_t)h * plain * rank;
    {
        const int r0 = blockIdx.z * ABS_THREADS * ABS_RPT;
        float acc[ABS_RPT][ABS_TM];
#pragma unroll
        for (int j = 0; j < ABS_RPT; j++)
#pragma unroll
            for (int mm = 0; mm < ABS_TM; mm++) acc[j][mm] = 0.f;
#pragma unroll 4
        for (int dd = 0; dd < plain; dd++) {
            float wv[ABS_RPT];
#pragma unroll
            for (int j = 0; j < ABS_RPT; j++) {
                const int r = r0 + t + j * ABS_THREADS;
                wv[j] = r < rank ? to_f32(ukh[(size_t)dd * rank + r]) : 0.f;
            }
#pragma unroll
            for (int mm = 0; mm < ABS_TM; mm++) {
                const float qv = qs[mm * plain + dd];
#pragma unroll
                for (int j = 0; j < ABS_RPT; j++) acc[j][mm] = fmaf(qv, wv[j], acc[j][mm]);
            }
        }
#pragma unroll
        for (int j = 0; j < ABS_RPT; j++) {
            const int r = r0 + t + j * ABS_THREADS;
            if (r < rank)
#pragma unroll
                for (int mm = 0; mm < ABS_TM; mm++)
                    if (m0 + mm < M) qa[((size_t)(m0 + mm) * n_heads + h) * W + r] = acc[j][mm];
        }
    }
}

// o[m, h, v] = sum_r uv[h, v, r] * ol[m, h, r].  uv: [heads * vdim, rank].  Grid (token tiles, heads);
// a warp per output element row v, lanes along the rank.
constexpr int EXP_TM = 8, EXP_THREADS = 128, EXP_VB = 16;      // a block: 8 tokens, one head, 16 output elements (grid.z)

template <typename T>
__global__ void __launch_bounds__(EXP_THREADS)
latent_expand_kernel(const float* __restrict__ ol, const T* __restrict__ uv, T* __restrict__ o, long long o_stride,
                     int M, int n_heads, int vdim, int rank) {
    ti_pdl_trigger();
    extern __shared__ float os[];        // [TM][rank]
    ti_pdl_sync();
    ol = ti_dependent(ol);
    const int m0 = blockIdx.x * EXP_TM, h = blockIdx.y, t = threadIdx.x;
    for (int idx = t; idx < EXP_TM * rank; idx += EXP_THREADS) {
        const int mm = idx / rank, r = idx - mm * rank;
        os[idx] = (m0 + mm < M) ? ol[((size_t)(m0 + mm) * n_heads + h) * rank + r] : 0.f;
    }
    __syncthreads();
    const int warp = t >> 5, lane = t & 31;
    const int v_end = min(vdim, (int)(blockIdx.z + 1) * EXP_VB);
    for (int v = blockIdx.z * EXP_VB + warp; v < v_end; v += EXP_THREADS / 32) {
        const T* wrow = uv + ((size_t)h * vdim + v) * rank;
        float acc[EXP_TM];
#pragma unroll
        for (int mm = 0; mm < EXP_TM; mm++) acc[mm] = 0.f;
        for (int r = lane; r < rank; r += 32) {
            const float wv = to_f32(wrow[r]);
#pragma unroll
            for (int mm = 0; mm < EXP_TM; mm++) acc[mm] = fmaf(wv, os[mm * rank + r], acc[mm]);
        }
#pragma unroll
        for (int mm = 0; mm < EXP_TM; mm++) {
            const float s = warp_sum(acc[mm]);
            if (lane == 0 && m0 + mm < M) o[(size_t)(m0 + mm) * o_stride + (size_t)h * vdim + v] = from_f32<T>(s);
        }
    }
}

// ---------------------------------------------------------------------------
// Keys and values per head after all, for steps of whole prompts on the tensor cores: from the up-projection's output
// ku[m] = [Wuk c | Wuv c] (heads * plain, then heads * vdim) and the step's rows, the padded heads
//     Q[m, h] = [q plain | q rotated | 0],  K[m, h] = [Wuk_h c | r | 0],  V[m, h] = [Wuv_h c | 0]      (D elements each)
// that a plain multi-head attention kernel takes.  One block per token.
template <typename T>
__global__ void latent_pack_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ ku, const T* __restrict__ lat,
                                   T* __restrict__ Qp, T* __restrict__ Kp, T* __restrict__ Vp, int n_heads, int plain, int rot,
                                   int vdim, int rank, int D) {
    ti_pdl_trigger();
    ti_pdl_sync();
    q = ti_dependent(q); ku = ti_dependent(ku); lat = ti_dependent(lat);
    const size_t m = blockIdx.x;
    const int hd = plain + rot, W = rank + rot;
    const T* qrow = q + m * q_stride;
    const T* krow = ku + m * ((size_t)n_heads * (plain + vdim));
    const T* vrow = krow + (size_t)n_heads * plain;
    const T* rrow = lat + m * W + rank;
    const T zero = from_f32<T>(0.f);
    for (int idx = threadIdx.x; idx < n_heads * D; idx += blockDim.x) {
        const int h = idx / D, e = idx - h * D;
        const size_t o = (m * n_heads + h) * D + e;
        Qp[o] = e < hd ? qrow[(size_t)h * hd + e] : zero;
        Kp[o] = e < plain ? krow[(size_t)h * plain + e] : e < hd ? rrow[e - plain] : zero;
        Vp[o] = e < vdim ? vrow[(size_t)h * vdim + e] : zero;
    }
}

// ---------------------------------------------------------------------------
// The attention.  A block works on 32 rows = QB consecutive queries of a sequence times HB heads
// (HB * QB == 32) against key tiles of 32 positions; thread t works on row t / 4, its 4 threads split
// a tile's keys (scores) and the latent's elements (output) between them.
constexpr int LQ = 32, LK = 32, LTHREADS = 128;

template <typename T, int MAXC>
__global__ void __launch_bounds__(LTHREADS)
latent_attn_kernel(const float* __restrict__ qa, const T* __restrict__ lat, float* __restrict__ ol,
                   const int* __restrict__ cu_new, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                   int n_heads, int hb, int rank, int rot, float scale, int window, const float* __restrict__ sink,
                   LatentPages kv, int n_splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
    ti_pdl_trigger();
    extern __shared__ float sm[];
    ti_pdl_sync();
    qa = ti_dependent(qa); lat = ti_dependent(lat);
    const int W = rank + rot, ld = W + 1;
    float* Qs = sm;                       // [LQ][ld]
    float* Ks = Qs + LQ * ld;             // [LK][ld]
    float* Ps = Ks + LK * ld;             // [LQ][LK + 1]
    const int qb = LQ / hb;
    // with n_splits > 1 the key tiles of a block's queries are shared out over n_splits blocks, which leave their
    // unnormalised sums, maxima and denominators for the merging kernel
    const int split = blockIdx.x % n_splits;
    const int b = blockIdx.z, h0 = blockIdx.y * hb, q0 = (blockIdx.x / n_splits) * qb;
    const int tok0 = cu_new[b];
    const int n = cu_new[b + 1] - tok0;
    if (q0 >= n) return;
    const int start = seq_start[b], slot = seq_slot[b], end = start + n;
    const int t = threadIdx.x, r = t >> 2, c4 = t & 3;
    // row rr: query q0 + rr / hb, head h0 + rr % hb
    for (int idx = t; idx < LQ * W; idx += LTHREADS) {
        const int rr = idx / W, e = idx - rr * W;
        const int qq = q0 + rr / hb, hh = h0 + rr % hb;
        Qs[rr * ld + e] = (qq < n && hh < n_heads) ? qa[((size_t)(tok0 + qq) * n_heads + hh) * W + e] : 0.f;
    }
    const int my_q = q0 + r / hb, my_h = h0 + r % hb;
    const bool row_ok = my_q < n && my_h < n_heads;
    const int qi = start + my_q;
    float acc[MAXC];
#pragma unroll
    for (int c = 0; c < MAXC; c++) acc[c] = 0.f;
    // the sink stands in the denominator from the start: running maximum sink_h, running sum 1
    float m_run = -INFINITY, l_run = 0.f;
    if (sink && row_ok && split == 0) { m_run = sink[my_h]; l_run = 1.f; }
    const int nc = (rank + 3) >> 2;      // elements of the latent per thread (c4 + 4 c)
    const int last_q = start + min(q0 + qb, n) - 1;
    const int lo = window > 0 ? max(0, start + q0 - window + 1) : 0;
    const int kt_first = lo / LK, kt_last = last_q / LK;
    const int per = (kt_last - kt_first + n_splits) / n_splits;
    const int kt_a = kt_first + split * per, kt_b = min(kt_last, kt_a + per - 1);
    for (int kt = kt_a; kt <= kt_b; kt++) {
        const int k0 = kt * LK;
        __syncthreads();
        // a warp fetches whole rows: where a row lives is worked out once, then the lanes run along it
        for (int rr = t >> 5; rr < LK; rr += LTHREADS / 32) {
            const int p = k0 + rr;
            const T* src = nullptr;
            if (p >= start) {
                if (p < end) src = lat + (size_t)(tok0 + p - start) * W;
            } else if (p >= lo) {
                const int row = kv.ring_rows > 0 ? p % kv.ring_rows : p;
                const int pidx = row / kv.page_size;
                const int page = pidx < kv.table_width ? kv.page_table[(size_t)slot * kv.table_width + pidx] : -1;
                if (page >= 0 && page < kv.n_pages) src = (const T*)kv.pages + ((size_t)page * kv.page_size + row % kv.page_size) * W;
            }
            for (int e = t & 31; e < W; e += 32) Ks[rr * ld + e] = src ? to_f32(src[e]) : 0.f;
        }
        __syncthreads();
        float s[8];
#pragma unroll
        for (int c = 0; c < 8; c++) s[c] = 0.f;
        const float* qrow = Qs + r * ld;
        for (int e = 0; e < W; e++) {
            const float qv = qrow[e];
#pragma unroll
            for (int c = 0; c < 8; c++) s[c] = fmaf(qv, Ks[(c4 + 4 * c) * ld + e], s[c]);
        }
        float m_tile = -INFINITY;
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const int kj = k0 + c4 + 4 * c;
            const bool ok = row_ok && kj <= qi && kj < end && (window <= 0 || kj > qi - window);
            s[c] = ok ? s[c] * scale : -INFINITY;
            m_tile = fmaxf(m_tile, s[c]);
        }
        m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
        m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 2));
        const float m_new = fmaxf(m_run, m_tile);
        float alpha = 1.f, l_tile = 0.f;
        if (m_new > -INFINITY) {
            alpha = expf(m_run - m_new);
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const float p = expf(s[c] - m_new);
                Ps[r * (LK + 1) + c4 + 4 * c] = p;
                l_tile += p;
            }
        } else {
#pragma unroll
            for (int c = 0; c < 8; c++) Ps[r * (LK + 1) + c4 + 4 * c] = 0.f;
        }
        l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 1);
        l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 2);
        l_run = l_run * alpha + l_tile;
        m_run = m_new;
        __syncwarp();
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nc) acc[c] *= alpha;
        const float* prow = Ps + r * (LK + 1);
        for (int j = 0; j < LK; j++) {
            const float p = prow[j];
            const float* vrow = Ks + j * ld + c4;
#pragma unroll
            for (int c = 0; c < MAXC; c++)
                if (c < nc) acc[c] = fmaf(p, vrow[4 * c], acc[c]);      // (an element past the rank is the rotated part: never stored)
        }
    }
    if (row_ok && n_splits > 1) {
        const size_t at = ((size_t)(tok0 + my_q) * n_heads + my_h) * n_splits + split;
        if (c4 == 0) { part_ml[at * 2] = m_run; part_ml[at * 2 + 1] = l_run; }
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nc && c4 + 4 * c < rank) part_o[at * rank + c4 + 4 * c] = acc[c];
    } else if (row_ok) {
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        float* orow = ol + ((size_t)(tok0 + my_q) * n_heads + my_h) * rank;
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nc && c4 + 4 * c < rank) orow[c4 + 4 * c] = acc[c] * inv;
    }
}

// ---------------------------------------------------------------------------
// One query per sequence, bfloat16, on the tensor cores (`mma.sync m16n8k16`, float32 accumulation).  A block takes one
// sequence, 16 * MT heads and one share of the keys, 32 positions at a time: the rows [c | r] of a tile go to shared memory
// as they are; S = Qa L^T (a warp per 8 keys), the softmax of a row by one thread in 32-bit, P rounded to bfloat16 as the
// second product's operand, O += P L[:, :rank] (the latent's columns shared out over the warps, a key pair per register
// fetched as two 16-bit loads).  Unnormalised sums, maxima and denominators go to the merging kernel when the keys are split.
// Rows of a tile outside the query's reach are zeroed: a weight of zero times whatever stood there must stay zero.
constexpr int DK = 32, D_THREADS = 128;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MT, int NTW>
__global__ void __launch_bounds__(D_THREADS)
latent_decode_mma_kernel(const float* __restrict__ qa, const bf16* __restrict__ lat, float* __restrict__ ol,
                         const int* __restrict__ cu_new, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                         int n_heads, int rank, int rot, float scale, int window, const float* __restrict__ sink,
                         LatentPages kv, int n_splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
    ti_pdl_trigger();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    ti_pdl_sync();
    qa = ti_dependent(qa); lat = ti_dependent(lat);
    constexpr int ROWS = 16 * MT;
    const int W = rank + rot, LD = W + 8;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                  // [ROWS][LD]
    bf16* Ls = Qs + ROWS * LD;                                     // [DK][LD]
    bf16* Ps = Ls + DK * LD;                                       // [ROWS][DK + 8]
    float* Ss = reinterpret_cast<float*>(Ps + ROWS * (DK + 8));    // [ROWS][DK + 1]
    float* m_s = Ss + ROWS * (DK + 1);                             // [ROWS] running maximum
    float* l_s = m_s + ROWS;                                       // [ROWS] running denominator
    float* a_s = l_s + ROWS;                                       // [ROWS] this tile's rescaling
    __shared__ const bf16* row_src[DK];
    const int split = blockIdx.x, h0 = blockIdx.y * ROWS, b = blockIdx.z;
    const int tok = cu_new[b];
    if (cu_new[b + 1] - tok <= 0) return;
    const int qi = seq_start[b], slot = seq_slot[b];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
    // (global loads in batches, so that several are on their way at a time: a block's four warps cannot hide one each)
    {
        const int per_row = W >> 2, total = ROWS * per_row;        // pieces of four floats
        for (int i0 = 0; i0 < total; i0 += 6 * D_THREADS) {
            float4 x[6];
#pragma unroll
            for (int u = 0; u < 6; u++) {
                const int idx = i0 + u * D_THREADS + tid, r = idx / per_row, e = idx - r * per_row;
                x[u] = (idx < total && h0 + r < n_heads) ? reinterpret_cast<const float4*>(qa + ((size_t)tok * n_heads + h0 + r) * W)[e]
                                                         : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 6; u++) {
                const int idx = i0 + u * D_THREADS + tid, r = idx / per_row, e = idx - r * per_row;
                if (idx < total) {
                    bf16* dst = Qs + r * LD + 4 * e;
                    dst[0] = from_f32<bf16>(x[u].x); dst[1] = from_f32<bf16>(x[u].y); dst[2] = from_f32<bf16>(x[u].z); dst[3] = from_f32<bf16>(x[u].w);
                }
            }
        }
    }
    if (tid < ROWS) {
        const bool with_sink = sink && split == 0 && h0 + tid < n_heads;
        m_s[tid] = with_sink ? sink[h0 + tid] : -INFINITY;
        l_s[tid] = with_sink ? 1.f : 0.f;
    }
    float O[MT][NTW][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int i = 0; i < NTW; i++)
#pragma unroll
            for (int c = 0; c < 4; c++) O[mt][i][c] = 0.f;
    const int lo = window > 0 ? max(0, qi - window + 1) : 0;
    const int kt_first = lo / DK, kt_last = qi / DK;
    const int per = (kt_last - kt_first + n_splits) / n_splits;
    const int kt_a = kt_first + split * per, kt_b = min(kt_last, kt_a + per - 1);
    const int n_tiles8 = rank >> 3;
    for (int kt = kt_a; kt <= kt_b; kt++) {
        const int k0 = kt * DK;
        __syncthreads();
        if (tid < DK) {              // where each of the tile's rows lives
            const int p = k0 + tid;
            const bf16* src = nullptr;
            if (p == qi) {
                src = lat + (size_t)tok * W;
            } else if (p >= lo && p < qi) {
                const int row = kv.ring_rows > 0 ? p % kv.ring_rows : p;
                const int pidx = row / kv.page_size;
                const int page = pidx < kv.table_width ? kv.page_table[(size_t)slot * kv.table_width + pidx] : -1;
                if (page >= 0 && page < kv.n_pages) src = (const bf16*)kv.pages + ((size_t)page * kv.page_size + row % kv.page_size) * W;
            }
            row_src[tid] = src;
        }
        __syncthreads();
        {
            const int per_row = W >> 3, total = DK * per_row;          // 16-byte pieces
            for (int i0 = 0; i0 < total; i0 += 6 * D_THREADS) {
                uint4 x[6];
#pragma unroll
                for (int u = 0; u < 6; u++) {
                    const int idx = i0 + u * D_THREADS + tid, rr = idx / per_row, e = idx - rr * per_row;
                    const bf16* src = idx < total ? row_src[rr] : nullptr;
                    x[u] = src ? reinterpret_cast<const uint4*>(src)[e] : make_uint4(0u, 0u, 0u, 0u);
                }
#pragma unroll
                for (int u = 0; u < 6; u++) {
                    const int idx = i0 + u * D_THREADS + tid, rr = idx / per_row, e = idx - rr * per_row;
                    if (idx < total) reinterpret_cast<uint4*>(Ls + rr * LD)[e] = x[u];
                }
            }
        }
        __syncthreads();
        // scores: this warp's 8 keys against all rows
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const bf16* qrow = Qs + (mt * 16 + g) * LD + 2 * t4;
            const bf16* krow = Ls + (warp * 8 + g) * LD + 2 * t4;
            for (int kk = 0; kk < W; kk += 16) {
                uint32_t a[4];
                a[0] = *reinterpret_cast<const uint32_t*>(qrow + kk);
                a[1] = *reinterpret_cast<const uint32_t*>(qrow + 8 * LD + kk);
                a[2] = *reinterpret_cast<const uint32_t*>(qrow + kk + 8);
                a[3] = *reinterpret_cast<const uint32_t*>(qrow + 8 * LD + kk + 8);
                mma_bf16_16816(c, a, *reinterpret_cast<const uint32_t*>(krow + kk), *reinterpret_cast<const uint32_t*>(krow + kk + 8));
            }
            float* srow = Ss + (mt * 16 + g) * (DK + 1) + warp * 8 + 2 * t4;
            srow[0] = c[0]; srow[1] = c[1];
            srow[8 * (DK + 1)] = c[2]; srow[8 * (DK + 1) + 1] = c[3];
        }
        __syncthreads();
        if (tid < ROWS) {
            const float* srow = Ss + tid * (DK + 1);
            const bool head_ok = h0 + tid < n_heads;
            float mx = -INFINITY;
            for (int j = 0; j < DK; j++) {
                const int p = k0 + j;
                if (head_ok && p >= lo && p <= qi) mx = fmaxf(mx, srow[j] * scale);
            }
            const float m_old = m_s[tid], m_new = fmaxf(m_old, mx);
            const float alpha = m_new > -INFINITY ? expf(m_old - m_new) : 1.f;
            float sum = 0.f;
            for (int j = 0; j < DK; j++) {
                const int p = k0 + j;
                float pr = 0.f;
                if (head_ok && p >= lo && p <= qi) pr = expf(srow[j] * scale - m_new);
                sum += pr;
                Ps[tid * (DK + 8) + j] = from_f32<bf16>(pr);
            }
            m_s[tid] = m_new;
            l_s[tid] = l_s[tid] * alpha + sum;
            a_s[tid] = alpha;
        }
        __syncthreads();
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const float al0 = a_s[mt * 16 + g], al1 = a_s[mt * 16 + g + 8];
            uint32_t a[2][4];
#pragma unroll
            for (int ks = 0; ks < 2; ks++) {
                const bf16* prow = Ps + (mt * 16 + g) * (DK + 8) + ks * 16 + 2 * t4;
                a[ks][0] = *reinterpret_cast<const uint32_t*>(prow);
                a[ks][1] = *reinterpret_cast<const uint32_t*>(prow + 8 * (DK + 8));
                a[ks][2] = *reinterpret_cast<const uint32_t*>(prow + 8);
                a[ks][3] = *reinterpret_cast<const uint32_t*>(prow + 8 * (DK + 8) + 8);
            }
#pragma unroll
            for (int i = 0; i < NTW; i++) {
                const int nt = warp + 4 * i;
                if (nt >= n_tiles8) continue;
                O[mt][i][0] *= al0; O[mt][i][1] *= al0; O[mt][i][2] *= al1; O[mt][i][3] *= al1;
                const unsigned short* col = reinterpret_cast<const unsigned short*>(Ls) + nt * 8 + g;
#pragma unroll
                for (int ks = 0; ks < 2; ks++) {
                    const int kr = ks * 16 + 2 * t4;
                    const uint32_t b0 = (uint32_t)col[(size_t)kr * LD] | ((uint32_t)col[(size_t)(kr + 1) * LD] << 16);
                    const uint32_t b1 = (uint32_t)col[(size_t)(kr + 8) * LD] | ((uint32_t)col[(size_t)(kr + 9) * LD] << 16);
                    mma_bf16_16816(O[mt][i], a[ks], b0, b1);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int r = mt * 16 + g + 8 * half, h = h0 + r;
            if (h >= n_heads) continue;
            const float l = l_s[r];
            if (part_o != nullptr) {
                const size_t at = ((size_t)tok * n_heads + h) * n_splits + split;
                if (t4 == 0 && warp == 0) { part_ml[at * 2] = m_s[r]; part_ml[at * 2 + 1] = l; }
#pragma unroll
                for (int i = 0; i < NTW; i++) {
                    const int nt = warp + 4 * i;
                    if (nt >= n_tiles8) continue;
                    float* dst = part_o + at * rank + nt * 8 + 2 * t4;
                    dst[0] = O[mt][i][2 * half]; dst[1] = O[mt][i][2 * half + 1];
                }
            } else {
                const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
                for (int i = 0; i < NTW; i++) {
                    const int nt = warp + 4 * i;
                    if (nt >= n_tiles8) continue;
                    float* dst = ol + ((size_t)tok * n_heads + h) * rank + nt * 8 + 2 * t4;
                    dst[0] = O[mt][i][2 * half] * inv; dst[1] = O[mt][i][2 * half + 1] * inv;
                }
            }
        }
}

template <int MT, int NTW>
int launch_decode_mma(const float* qa, const void* lat, float* ol, const int* cu_new, const int* seq_start, const int* seq_slot,
                      int n_seq, int n_heads, int rank, int rot, float scale, int window, const float* sink,
                      const LatentPages& kv, int n_splits, float* part_o, float* part_ml, int n_tok, cudaStream_t stream,
                      const void* uv = nullptr, void* o = nullptr, long long o_stride = 0, int vdim = 0) {
    constexpr int ROWS = 16 * MT;
    const int W = rank + rot, LD = W + 8;
    const size_t smem = (size_t)(ROWS + DK) * LD * 2 + (size_t)ROWS * (DK + 8) * 2 + ((size_t)ROWS * (DK + 1) + 3 * ROWS) * 4;
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        TI_CUDA(cudaFuncSetAttribute(latent_decode_mma_kernel<MT, NTW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    dim3 grid(n_splits, (n_heads + ROWS - 1) / ROWS, n_seq);
    TI_CUDA(ti_launch_class<3>(latent_decode_mma_kernel<MT, NTW>, grid, dim3(D_THREADS), smem, stream, qa, (const bf16*)lat, ol, cu_new,
                               seq_start, seq_slot, n_heads, rank, rot, scale, window, sink, kv, n_splits, part_o, part_ml));
    TI_CHECK_LAUNCH("latent_attention (one token, tensor cores)");
    if (uv) {
        const size_t sm2 = (size_t)(rank + 64) * sizeof(float);
        TI_CUDA(ti_launch_class<4>(latent_merge_expand_kernel<bf16>, dim3(n_tok, n_heads), dim3(128), sm2, stream, (const float*)part_o,
                                   (const float*)part_ml, (const bf16*)uv, (bf16*)o, o_stride, n_heads, vdim, rank, n_splits));
        TI_CHECK_LAUNCH("latent_merge_expand");
        return 0;
    }
    if (n_splits > 1) {
        int threads = ((rank + 3) / 4 + 31) / 32 * 32;
        TI_CUDA(ti_launch_class<4>(tiattn::attn_decode_combine_kernel<float>, dim3(n_tok, n_heads), dim3(threads), 0, stream,
                                   (const float*)part_o, (const float*)part_ml, ol, (long long)n_heads * rank, n_heads, rank, n_splits));
        TI_CHECK_LAUNCH("latent_attention_combine");
    }
    return 0;
}

template <typename T, int MAXC>
int launch_attn(const float* qa, const void* lat, float* ol, const int* cu_new, const int* seq_start, const int* seq_slot,
                int n_seq, int max_new, int n_heads, int hb, int rank, int rot, float scale, int window, const float* sink,
                const LatentPages& kv, int n_splits, float* part_o, float* part_ml, int n_tok, cudaStream_t stream) {
    const int W = rank + rot;
    const size_t smem = ((size_t)(LQ + LK) * (W + 1) + (size_t)LQ * (LK + 1)) * sizeof(float);
    TI_REQUIRE(smem <= 227 * 1024, "latent_attention: rows of %d elements need %zu bytes of shared memory", W, smem);
    static size_t configured = 0;
    if (smem > configured) {
        TI_CUDA(cudaFuncSetAttribute(latent_attn_kernel<T, MAXC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    const int qb = LQ / hb;
    dim3 grid(((max_new + qb - 1) / qb) * n_splits, (n_heads + hb - 1) / hb, n_seq);
    TI_CUDA(ti_launch(latent_attn_kernel<T, MAXC>, grid, dim3(LTHREADS), smem, stream, qa, (const T*)lat, ol, cu_new, seq_start,
                      seq_slot, n_heads, hb, rank, rot, scale, window, sink, kv, n_splits, part_o, part_ml));
    TI_CHECK_LAUNCH("latent_attention");
    if (n_splits > 1) {
        // the splits' sums meet: one block per (token, head), the latent's elements over its threads
        int threads = ((rank + 3) / 4 + 31) / 32 * 32;
        TI_CUDA(ti_launch_class<4>(tiattn::attn_decode_combine_kernel<float>, dim3(n_tok, n_heads), dim3(threads), 0, stream,
                                   (const float*)part_o, (const float*)part_ml, ol, (long long)n_heads * rank, n_heads, rank, n_splits));
        TI_CHECK_LAUNCH("latent_attention_combine");
    }
    return 0;
}

}  // namespace

// d[M, rank + rot] (row stride d_stride) is the down-projection's output; q[M, heads, plain + rot] or null;
// cos/sin: float32 [max_pos, rot / 2]; lat: [M, rank + rot] dense or null; pages null: no store.
extern "C" int ti_latent_prep(const void* d, long long d_stride, void* q, long long q_stride, int n_heads, int plain,
                              int rank, int rot, const float* norm_w, float eps, const float* cos_t, const float* sin_t,
                              int max_pos, const int* tok_pos, const int* tok_seq, const int* seq_slot, const int* seq_len,
                              void* lat, void* pages, const int* page_table, int table_width, int page_size, int ring_rows, int n_pages,
                              int M, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && rank > 0 && rot >= 0 && rot % 2 == 0 && plain >= 0, "latent_prep: bad sizes");
    TI_REQUIRE(rot == 0 || (cos_t && sin_t && max_pos > 0), "latent_prep: a rotated part needs cos and sin tables");
    TI_REQUIRE(!pages || (page_table && seq_len && page_size > 0 && table_width > 0 && n_pages > 0 && ring_rows % page_size == 0),
               "latent_prep: incomplete cache description");
    LatentPages kv{pages, page_table, table_width, page_size, ring_rows, n_pages, seq_len};
    const int W = rank + rot;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        const size_t smem = (size_t)(W + 33) * sizeof(float) + (size_t)W * sizeof(T);
        TI_REQUIRE(smem <= 48 * 1024, "latent_prep: rows of %d elements are too long", W);
        TI_CUDA(ti_launch_class<2>(latent_prep_kernel<T>, dim3(M), dim3(128), smem, stream, (const T*)d, d_stride, (T*)q, q_stride,
                                   n_heads, plain, rank, rot, norm_w, eps, cos_t, sin_t, max_pos, tok_pos, tok_seq, seq_slot,
                                   (T*)lat, kv));
        TI_CHECK_LAUNCH("latent_prep");
        return 0;
    });
}

extern "C" int ti_latent_store(const void* lat, int W, const int* tok_pos, const int* tok_seq, const int* seq_slot,
                               const int* seq_len, void* pages, const int* page_table, int table_width, int page_size, int ring_rows, int n_pages,
                               int M, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(pages && page_table && seq_len && page_size > 0 && table_width > 0 && n_pages > 0 && ring_rows % page_size == 0,
               "latent_store: incomplete cache description");
    LatentPages kv{pages, page_table, table_width, page_size, ring_rows, n_pages, seq_len};
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<2>(latent_store_kernel<T>, dim3(M), dim3(128), 0, stream, (const T*)lat, W, tok_pos, tok_seq,
                                   seq_slot, kv));
        TI_CHECK_LAUNCH("latent_store");
        return 0;
    });
}

// A step of single tokens in two launches before and two after the projections... the latent's part of it: this one does
// latent_prep's and latent_absorb's work (q is left unrotated; qa gets the rotated part).
extern "C" int ti_latent_prep_absorb(const void* d, long long d_stride, const void* q, long long q_stride, int n_heads, int plain,
                                     int rank, int rot, const float* norm_w, float eps, const float* cos_t, const float* sin_t,
                                     int max_pos, const int* tok_pos, const int* tok_seq, const int* seq_slot, const int* seq_len,
                                     void* lat, void* pages, const int* page_table, int table_width, int page_size, int ring_rows,
                                     int n_pages, const void* uk, float* qa, int M, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_heads > 0 && n_heads < 65535 && rank > 0 && rot >= 0 && rot % 2 == 0 && plain >= 0 && q && uk && qa && lat,
               "latent_prep_absorb: bad arguments");
    TI_REQUIRE(rot == 0 || (cos_t && sin_t && max_pos > 0), "latent_prep_absorb: a rotated part needs cos and sin tables");
    TI_REQUIRE(!pages || (page_table && seq_len && page_size > 0 && table_width > 0 && n_pages > 0 && ring_rows % page_size == 0),
               "latent_prep_absorb: incomplete cache description");
    LatentPages kv{pages, page_table, table_width, page_size, ring_rows, n_pages, seq_len};
    const int W = rank + rot;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        size_t smem = (size_t)(W + 33) * sizeof(float) + (size_t)W * sizeof(T);
        if ((size_t)plain * sizeof(float) > smem) smem = (size_t)plain * sizeof(float);
        TI_REQUIRE(smem <= 48 * 1024, "latent_prep_absorb: rows of %d elements are too long", W);
        TI_CUDA(ti_launch_class<2>(latent_prep_absorb_kernel<T>, dim3(M, n_heads + 1), dim3(128), smem, stream, (const T*)d, d_stride,
                                   (const T*)q, q_stride, n_heads, plain, rank, rot, norm_w, eps, cos_t, sin_t, max_pos, tok_pos, tok_seq,
                                   seq_slot, (T*)lat, kv, (const T*)uk, qa));
        TI_CHECK_LAUNCH("latent_prep_absorb");
        return 0;
    });
}

// Whether ti_latent_decode takes these sizes (bfloat16 only): rows in 16-element steps, a latent in 8-element tiles up to 512.
extern "C" int ti_latent_decode_takes(int rank, int rot) { return (rank + rot) % 16 == 0 && rank % 8 == 0 && rank <= 512; }

// One query per sequence, bfloat16, tensor cores; the key splits' merge and the way out through uv[heads * vdim, rank] in
// the second launch: o[n_seq, heads * vdim].  part_o: float32 [n_seq, heads, n_splits, rank], part_ml: [n_seq, heads, n_splits, 2].
extern "C" int ti_latent_decode(const float* qa, const void* lat, const int* cu_new, const int* seq_start, const int* seq_slot,
                                int n_seq, int n_heads, int rank, int rot, float scale, int window, const float* sink,
                                const void* pages, const int* page_table, int table_width, int page_size, int ring_rows, int n_pages,
                                int n_splits, float* part_o, float* part_ml, const void* uv, void* o, long long o_stride, int vdim,
                                cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_seq <= 65535 && n_heads > 0 && vdim > 0 && ti_latent_decode_takes(rank, rot), "latent_decode: sizes not taken");
    TI_REQUIRE(n_splits >= 1 && n_splits <= 64 && part_o && part_ml && uv && o, "latent_decode: bad arguments");
    TI_REQUIRE(pages && page_table && page_size > 0 && table_width > 0 && n_pages > 0 && ring_rows % page_size == 0,
               "latent_decode: incomplete cache description");
    TI_REQUIRE(ring_rows == 0 || (window > 0 && ring_rows >= window), "latent_decode: a ring of %d rows needs a window of at most as many", ring_rows);
    TI_REQUIRE((((uintptr_t)lat | (uintptr_t)pages | (uintptr_t)qa) & 15) == 0, "latent_decode: rows are not 16-byte aligned");
    LatentPages kv{const_cast<void*>(pages), page_table, table_width, page_size, ring_rows, n_pages, nullptr};
    const bool two = n_heads > 16;
#define TI_LATENT_DECODE(MT, NTW) launch_decode_mma<MT, NTW>(qa, lat, nullptr, cu_new, seq_start, seq_slot, n_seq, n_heads, rank, rot, scale, \
                                                            window, sink, kv, n_splits, part_o, part_ml, n_seq, stream, uv, o, o_stride, vdim)
    if (rank <= 128) return two ? TI_LATENT_DECODE(2, 4) : TI_LATENT_DECODE(1, 4);
    if (rank <= 256) return two ? TI_LATENT_DECODE(2, 8) : TI_LATENT_DECODE(1, 8);
    return two ? TI_LATENT_DECODE(2, 16) : TI_LATENT_DECODE(1, 16);
#undef TI_LATENT_DECODE
}

extern "C" int ti_latent_pack(const void* q, long long q_stride, const void* ku, const void* lat, void* Qp, void* Kp, void* Vp,
                              int M, int n_heads, int plain, int rot, int vdim, int rank, int D, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_heads > 0 && plain >= 0 && rot >= 0 && vdim > 0 && rank > 0 && D >= plain + rot && D >= vdim,
               "latent_pack: heads of %d + %d and %d elements do not fit %d", plain, rot, vdim, D);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<2>(latent_pack_kernel<T>, dim3(M), dim3(256), 0, stream, (const T*)q, q_stride, (const T*)ku,
                                   (const T*)lat, (T*)Qp, (T*)Kp, (T*)Vp, n_heads, plain, rot, vdim, rank, D));
        TI_CHECK_LAUNCH("latent_pack");
        return 0;
    });
}

extern "C" int ti_latent_absorb(const void* q, long long q_stride, const void* uk, float* qa, int M, int n_heads, int plain,
                                int rank, int rot, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_heads > 0 && n_heads <= 65535 && plain >= 0 && rank > 0 && rot >= 0, "latent_absorb: bad sizes");
    const size_t smem = (size_t)ABS_TM * (plain > 0 ? plain : 1) * sizeof(float);
    TI_REQUIRE(smem <= 48 * 1024, "latent_absorb: heads of %d unrotated elements are too long", plain);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        const int zs = (rank + ABS_THREADS * ABS_RPT - 1) / (ABS_THREADS * ABS_RPT);
        TI_CUDA(ti_launch(latent_absorb_kernel<T>, dim3((M + ABS_TM - 1) / ABS_TM, n_heads, zs), dim3(ABS_THREADS), smem, stream,
                          (const T*)q, q_stride, (const T*)uk, qa, M, n_heads, plain, rank, rot));
        TI_CHECK_LAUNCH("latent_absorb");
        return 0;
    });
}

extern "C" int ti_latent_expand(const float* ol, const void* uv, void* o, long long o_stride, int M, int n_heads, int vdim,
                                int rank, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_heads > 0 && n_heads <= 65535 && vdim > 0 && rank > 0, "latent_expand: bad sizes");
    const size_t smem = (size_t)EXP_TM * rank * sizeof(float);
    TI_REQUIRE(smem <= 48 * 1024, "latent_expand: a latent of %d elements is too long", rank);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch(latent_expand_kernel<T>, dim3((M + EXP_TM - 1) / EXP_TM, n_heads, (vdim + EXP_VB - 1) / EXP_VB), dim3(EXP_THREADS), smem, stream, ol,
                          (const T*)uv, (T*)o, o_stride, M, n_heads, vdim, rank));
        TI_CHECK_LAUNCH("latent_expand");
        return 0;
    });
}

// qa: float32 [M, heads, rank + rot]; lat: the step's rows [M, rank + rot]; ol: float32 [M, heads, rank].
// hb: heads per block, a power of two up to 32.  sink: float32 [heads] or null.
extern "C" int ti_latent_attn(const float* qa, const void* lat, float* ol, const int* cu_new, const int* seq_start,
                              const int* seq_slot, int n_seq, int max_new, int n_heads, int hb, int rank, int rot, float scale,
                              int window, const float* sink, const void* pages, const int* page_table, int table_width,
                              int page_size, int ring_rows, int n_pages, int n_splits, float* part_o, float* part_ml, int n_tok,
                              int dtype, cudaStream_t stream) {
    if (n_seq == 0 || max_new == 0) return 0;
    TI_REQUIRE(n_seq > 0 && max_new > 0 && n_heads > 0 && rank > 0 && rot >= 0, "latent_attention: bad sizes");
    TI_REQUIRE(hb >= 1 && hb <= LQ && (hb & (hb - 1)) == 0, "latent_attention: %d heads per block (a power of two up to %d)", hb, LQ);
    TI_REQUIRE(n_seq <= 65535, "latent_attention: too many sequences for one launch");
    TI_REQUIRE(pages && page_table && page_size > 0 && table_width > 0 && n_pages > 0 && ring_rows % page_size == 0,
               "latent_attention: incomplete cache description");
    TI_REQUIRE(ring_rows == 0 || (window > 0 && ring_rows >= window),
               "latent_attention: a ring of %d rows needs a window of at most as many positions (got %d)", ring_rows, window);
    TI_REQUIRE(rank <= 1024, "latent_attention: a latent of %d elements is not supported (up to 1,024)", rank);
    TI_REQUIRE(n_splits >= 1 && (n_splits == 1 || (part_o && part_ml && n_tok > 0 && n_tok <= 65535 * 32768)),
               "latent_attention: %d splits need room for their partial results", n_splits);
    LatentPages kv{const_cast<void*>(pages), page_table, table_width, page_size, ring_rows, n_pages, nullptr};
    // every sequence brings one token, bfloat16, rows in 16-byte pieces: the tensor-core kernel
    if (dtype == TI_BF16 && max_new == 1 && n_tok == n_seq && (rank + rot) % 16 == 0 && rank % 8 == 0 && rank <= 512 &&
        ((uintptr_t)lat & 15) == 0 && ((uintptr_t)pages & 15) == 0) {
        const bool two = n_heads > 16;
#define TI_LATENT_DECODE(MT, NTW) launch_decode_mma<MT, NTW>(qa, lat, ol, cu_new, seq_start, seq_slot, n_seq, n_heads, rank, rot, scale, \
                                                            window, sink, kv, n_splits, part_o, part_ml, n_tok, stream)
        if (rank <= 128) return two ? TI_LATENT_DECODE(2, 4) : TI_LATENT_DECODE(1, 4);
        if (rank <= 256) return two ? TI_LATENT_DECODE(2, 8) : TI_LATENT_DECODE(1, 8);
        return two ? TI_LATENT_DECODE(2, 16) : TI_LATENT_DECODE(1, 16);
#undef TI_LATENT_DECODE
    }
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        if (rank <= 64)
            return launch_attn<T, 16>(qa, lat, ol, cu_new, seq_start, seq_slot, n_seq, max_new, n_heads, hb, rank, rot, scale, window, sink, kv, n_splits, part_o, part_ml, n_tok, stream);
        if (rank <= 128)
            return launch_attn<T, 32>(qa, lat, ol, cu_new, seq_start, seq_slot, n_seq, max_new, n_heads, hb, rank, rot, scale, window, sink, kv, n_splits, part_o, part_ml, n_tok, stream);
        if (rank <= 256)
            return launch_attn<T, 64>(qa, lat, ol, cu_new, seq_start, seq_slot, n_seq, max_new, n_heads, hb, rank, rot, scale, window, sink, kv, n_splits, part_o, part_ml, n_tok, stream);
        if (rank <= 512)
            return launch_attn<T, 128>(qa, lat, ol, cu_new, seq_start, seq_slot, n_seq, max_new, n_heads, hb, rank, rot, scale, window, sink, kv, n_splits, part_o, part_ml, n_tok, stream);
        return launch_attn<T, 256>(qa, lat, ol, cu_new, seq_start, seq_slot, n_seq, max_new, n_heads, hb, rank, rot, scale, window, sink, kv, n_splits, part_o, part_ml, n_tok, stream);
    });
}
