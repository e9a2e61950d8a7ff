// Causal grouped-query attention with a soft cap on the scores and a learned bias by distance,
// over keys and values of different sizes, read from the paged cache.  CUDA cores, everything
// after the loads in 32-bit.
//
// For the query at position i and the key at position j <= i of a sequence:
//     s_ij = (q_i . k_j) * scale;   s_ij <- cap * tanh(s_ij / cap)  (cap > 0);   s_ij <- s_ij + bias[h][min(i - j, far)]
// then the ordinary softmax over j and o_i = sum_j p_ij v_j.  `bias` [heads, far + 1] is the
// distance's bucket already looked up (the host folds the bucket rule into the table; every
// distance from `far` on shares one entry).  Query head h reads kv head h / (heads / kv_heads); a
// query or key has `dim` elements, a value `vdim`.
//
// attn_bias_prepare: from the projection's output row [q | k | v]: adds the projections' biases,
// norms every query and key head (x * rsqrt(mean(x^2) + eps) * w, plain weight), leaves all three
// in place and stores key and value at the token's position in the sequence's pages.
// attn_bias: any number of new tokens per sequence after any number of cached ones; all keys are
// read from the pages, so the step's own must be stored first.  Grid (query tiles of 32, heads,
// sequences), 128 threads: thread t works on query row t / 4; its 4 threads split the tile's 32
// keys (scores) and the value's elements (output) between them.
// attn_bias_decode: one query per sequence; a block takes up to four query heads of one kv head and
// one of `splits` ranges of keys, a warp 32 keys at a time (a lane a key for the scores, then the
// lanes the value's elements); ranges are merged by a second kernel when there are several.
#include "common.cuh"

#include <type_traits>

namespace {

struct Pages {
    const void* k_pages; const void* v_pages;      // [pages, kv_heads, page_size, dim] and [.., vdim]
    const int* page_table; int table_width; int page_size; int n_pages;
};

__device__ __forceinline__ float capped(float s, float cap, float inv_cap) { return cap > 0.f ? cap * tanhf(s * inv_cap) : s; }

// one warp per (token, unit): units 0 .. H - 1 query heads, then G key heads, then G value heads
template <typename T>
__global__ void attn_bias_prepare_kernel(T* __restrict__ qkv, long long ld, const float* __restrict__ bias,
                                         const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                         const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                         const int* __restrict__ seq_slot, Pages pg, int M, int H, int G, int dim, int vdim) {
    ti_pdl_trigger();
    ti_pdl_sync();
    qkv = ti_dependent(qkv);
    const int units = H + 2 * G;
    const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= (long long)M * units) return;
    const int lane = threadIdx.x & 31;
    const int m = (int)(r / units), unit = (int)(r - (long long)m * units);
    T* row = qkv + (size_t)m * ld;
    const bool is_q = unit < H, is_k = !is_q && unit < H + G;
    const int head = is_q ? unit : is_k ? unit - H : unit - H - G;
    const int n = (is_q || is_k) ? dim : vdim;
    const int col0 = is_q ? head * dim : is_k ? H * dim + head * dim : (H + G) * dim + head * vdim;
    T* dst = nullptr;
    if (!is_q) {
        const int p = tok_pos[m], slot = seq_slot[tok_seq[m]];
        const int pidx = p / pg.page_size;
        const int page = pidx < pg.table_width ? pg.page_table[(size_t)slot * pg.table_width + pidx] : 0;
        const int pp = (page >= 0 && page < pg.n_pages) ? page : 0;       // page 0 is scratch
        dst = (T*)(is_k ? pg.k_pages : pg.v_pages) + (((size_t)pp * G + head) * pg.page_size + p % pg.page_size) * n;
    }
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) {
        const float x = to_f32(row[col0 + i]) + (bias ? bias[col0 + i] : 0.f);
        ss = fmaf(x, x, ss);
    }
    const float* w = is_q ? q_w : is_k ? k_w : nullptr;
    float inv = 1.f;
    if (w) inv = rsqrtf(warp_sum(ss) / (float)n + eps);
    for (int i = lane; i < n; i += 32) {
        float x = to_f32(row[col0 + i]) + (bias ? bias[col0 + i] : 0.f);
        if (w) x = x * inv * w[i];
        row[col0 + i] = from_f32<T>(x);              // in place too: a kernel that reads the step's own keys and values finds them ready
        if (!is_q) dst[i] = from_f32<T>(x);
    }
}

constexpr int BQ = 32, BKV = 32, THREADS = 128;

template <typename T, int MAXC>
__global__ void __launch_bounds__(THREADS)
attn_bias_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long o_stride,
                 const int* __restrict__ cu_new, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                 Pages pg, const float* __restrict__ dist_bias, int far, int n_heads, int n_kv_heads, int dim, int vdim,
                 float scale, float cap) {
    ti_pdl_trigger();
    extern __shared__ float sm[];
    ti_pdl_sync();
    q = ti_dependent(q);
    const int ldk = dim + 1, ldv = vdim + 1;
    float* Qs = sm;                      // [BQ][dim + 1]
    float* Ks = Qs + BQ * ldk;           // [BKV][dim + 1]
    float* Vs = Ks + BKV * ldk;          // [BKV][vdim + 1]
    float* Ps = Vs + BKV * ldv;          // [BQ][BKV + 1]
    const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BQ;
    const int tok0 = cu_new[b];
    const int n = cu_new[b + 1] - tok0;
    if (q0 >= n) return;
    const int kvh = h / (n_heads / n_kv_heads);
    const int t = threadIdx.x, r = t >> 2, c4 = t & 3;
    const int start = seq_start[b], slot = seq_slot[b];
    const int end = start + n;
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    const float* hb = dist_bias ? dist_bias + (size_t)h * (far + 1) : nullptr;

    for (int idx = t; idx < BQ * dim; idx += THREADS) {
        const int rr = idx / dim, d = idx - rr * dim;
        Qs[rr * ldk + d] = (q0 + rr < n) ? to_f32(q[(size_t)(tok0 + q0 + rr) * q_stride + (size_t)h * dim + d]) : 0.f;
    }
    float acc[MAXC];
#pragma unroll
    for (int c = 0; c < MAXC; c++) acc[c] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const int qi = start + q0 + r;      // this thread's query position
    const int nc = (vdim + 3) >> 2;     // value elements per thread (c4, c4 + 4, ...)
    const int last_q = start + min(q0 + BQ, n) - 1;
    for (int k0 = 0; k0 <= last_q; k0 += BKV) {
        __syncthreads();  // previous tile fully consumed (and Qs written, first time)
        for (int rr = t >> 3; rr < BKV; rr += THREADS >> 3) {
            const int p = k0 + rr;
            const T* kp = nullptr;
            const T* vp = nullptr;
            if (p < end) {
                const int pidx = p / pg.page_size;
                const int page = pidx < pg.table_width ? pg.page_table[(size_t)slot * pg.table_width + pidx] : -1;
                if (page >= 0 && page < pg.n_pages) {
                    const size_t at = ((size_t)page * n_kv_heads + kvh) * pg.page_size + p % pg.page_size;
                    kp = (const T*)pg.k_pages + at * dim;
                    vp = (const T*)pg.v_pages + at * vdim;
                }
            }
            for (int d = t & 7; d < dim; d += 8) Ks[rr * ldk + d] = kp ? to_f32(kp[d]) : 0.f;
            for (int d = t & 7; d < vdim; d += 8) Vs[rr * ldv + d] = vp ? to_f32(vp[d]) : 0.f;
        }
        __syncthreads();
        float s[8];
#pragma unroll
        for (int c = 0; c < 8; c++) s[c] = 0.f;
        const float* qrow = Qs + r * ldk;
        for (int d = 0; d < dim; d++) {
            const float qv = qrow[d];
#pragma unroll
            for (int c = 0; c < 8; c++) s[c] = fmaf(qv, Ks[(c4 + 4 * c) * ldk + d], s[c]);
        }
        float m_tile = -INFINITY;
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const int kj = k0 + c4 + 4 * c;
            const bool ok = kj <= qi && kj < end;
            float x = capped(s[c] * scale, cap, inv_cap);
            if (hb && ok) x += hb[min(qi - kj, far)];
            s[c] = ok ? x : -INFINITY;
            m_tile = fmaxf(m_tile, s[c]);
        }
        m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
        m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 2));
        const float m_new = fmaxf(m_run, m_tile);
        float alpha = 1.f, l_tile = 0.f;
        if (m_new > -INFINITY) {
            alpha = expf(m_run - m_new);  // exp(-inf) = 0 on the first useful tile
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const float p = expf(s[c] - m_new);
                Ps[r * (BKV + 1) + c4 + 4 * c] = p;
                l_tile += p;
            }
        } else {
#pragma unroll
            for (int c = 0; c < 8; c++) Ps[r * (BKV + 1) + c4 + 4 * c] = 0.f;
        }
        l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 1);
        l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 2);
        l_run = l_run * alpha + l_tile;
        m_run = m_new;
        __syncwarp();  // the four threads of a row are in one warp
#pragma unroll
        for (int c = 0; c < MAXC; c++) acc[c] *= alpha;
        const float* prow = Ps + r * (BKV + 1);
        for (int j = 0; j < BKV; j++) {
            const float p = prow[j];
            const float* vrow = Vs + j * ldv + c4;
#pragma unroll
            for (int c = 0; c < MAXC; c++)
                if (c < nc && c4 + 4 * c < vdim) acc[c] = fmaf(p, vrow[4 * c], acc[c]);
        }
    }
    if (qi < end) {
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        T* orow = out + (size_t)(tok0 + qi - start) * o_stride + (size_t)h * vdim;
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nc && c4 + 4 * c < vdim) orow[c4 + 4 * c] = from_f32<T>(acc[c] * inv);
    }
}

constexpr int DEC_WARPS = 4, DEC_MAXE = 8;      // up to 256 elements per head, lane + 32 e

// `n` consecutive elements of a row as floats, by one load where size and address allow it
template <typename T, int N>
__device__ __forceinline__ void load_run(const T* __restrict__ p, float (&x)[N], bool vec) {
    constexpr int BYTES = N * (int)sizeof(T);
    if (vec && (BYTES == 16 || BYTES == 8 || BYTES == 4)) {
        T raw[N];
        if constexpr (BYTES == 16) *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(p);
        else if constexpr (BYTES == 8) *reinterpret_cast<uint2*>(raw) = *reinterpret_cast<const uint2*>(p);
        else if constexpr (BYTES == 4) *reinterpret_cast<uint32_t*>(raw) = *reinterpret_cast<const uint32_t*>(p);
#pragma unroll
        for (int e = 0; e < N; e++) x[e] = to_f32(raw[e]);
    } else {
#pragma unroll
        for (int e = 0; e < N; e++) x[e] = to_f32(p[e]);
    }
}

// A block takes GH query heads that share a kv head, and one range of keys; a warp 32 keys at a time: a lane a key for
// the scores of all GH heads (the key's row is read once, 16 bytes at a time where it allows; no sums across lanes), then
// the lanes VPL consecutive elements of the value each, while the 32 weights and rows go round by shuffles.
// part_o [n_seq, heads, splits, vdim], part_ml [n_seq, heads, splits, 2] when splits > 1.
template <typename T, int GH, int VPL>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_bias_decode_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long o_stride,
                        const int* __restrict__ seq_len, const int* __restrict__ seq_slot, Pages pg,
                        const float* __restrict__ dist_bias, int far, int n_heads, int n_kv_heads, int dim, int vdim,
                        float scale, float cap, int splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
    ti_pdl_trigger();
    extern __shared__ __align__(16) float dsm[];         // q: [GH][dim]; o: [DEC_WARPS][GH][32 * VPL]; m, l: [DEC_WARPS][GH][2]
    float* q_sh = dsm;
    float* o_sh = q_sh + GH * dim;
    float* ml_sh = o_sh + DEC_WARPS * GH * 32 * VPL;
    ti_pdl_sync();
    q = ti_dependent(q);
    const int b = blockIdx.z, h0 = blockIdx.y * GH, sp = blockIdx.x;
    const int len = seq_len[b], slot = seq_slot[b];
    const int qi = len - 1;
    const int kvh = h0 / (n_heads / n_kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tiles = (len + 31) / 32, per = (tiles + splits - 1) / splits;          // ranges of whole tiles of 32 keys
    const int t_lo = sp * per, t_hi = min(tiles, t_lo + per);
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    for (int i = threadIdx.x; i < GH * dim; i += DEC_WARPS * 32)
        q_sh[i] = to_f32(q[(size_t)b * q_stride + (size_t)h0 * dim + i]) * scale;
    __syncthreads();
    const bool kvec = (dim * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(pg.k_pages) & 15) == 0;
    const bool vvec = vdim % VPL == 0 && (reinterpret_cast<uintptr_t>(pg.v_pages) & 15) == 0;
    constexpr int KPER = 16 / sizeof(T);
    float acc[GH][VPL], m_run[GH], l_run[GH];
#pragma unroll
    for (int g = 0; g < GH; g++) {
        m_run[g] = -INFINITY; l_run[g] = 0.f;
#pragma unroll
        for (int e = 0; e < VPL; e++) acc[g][e] = 0.f;
    }
    for (int t = t_lo + warp; t < t_hi; t += DEC_WARPS) {
        const int j = t * 32 + lane;
        int at = -1;                                     // the key's row among all rows of the pages
        if (j < len) {
            const int pidx = j / pg.page_size;
            const int page = pidx < pg.table_width ? pg.page_table[(size_t)slot * pg.table_width + pidx] : -1;
            if (page >= 0 && page < pg.n_pages) at = (page * n_kv_heads + kvh) * pg.page_size + j % pg.page_size;
        }
        float s[GH];
#pragma unroll
        for (int g = 0; g < GH; g++) s[g] = 0.f;
        if (at >= 0) {
            const T* kp = (const T*)pg.k_pages + (size_t)at * dim;
            if (kvec) {
                for (int d = 0; d < dim; d += KPER) {
                    float x[KPER];
                    load_run<T, KPER>(kp + d, x, true);
#pragma unroll
                    for (int g = 0; g < GH; g++)
#pragma unroll
                        for (int e = 0; e < KPER; e++) s[g] = fmaf(q_sh[g * dim + d + e], x[e], s[g]);
                }
            } else {
                for (int d = 0; d < dim; d++) {
                    const float x = to_f32(kp[d]);
#pragma unroll
                    for (int g = 0; g < GH; g++) s[g] = fmaf(q_sh[g * dim + d], x, s[g]);
                }
            }
        }
        float p[GH];
        bool any = false;
#pragma unroll
        for (int g = 0; g < GH; g++) {
            float x = -INFINITY;
            if (at >= 0) {
                x = capped(s[g], cap, inv_cap);
                if (dist_bias) x += dist_bias[(size_t)(h0 + g) * (far + 1) + min(qi - j, far)];
            }
            const float m_new = fmaxf(m_run[g], warp_max(x));
            p[g] = 0.f;
            if (m_new > -INFINITY) {                     // (the same for all lanes)
                const float alpha = expf(m_run[g] - m_new);
                p[g] = at >= 0 ? expf(x - m_new) : 0.f;
                l_run[g] = l_run[g] * alpha + warp_sum(p[g]);
                m_run[g] = m_new;
#pragma unroll
                for (int e = 0; e < VPL; e++) acc[g][e] *= alpha;
                any = true;
            }
        }
        if (!any) continue;
#pragma unroll 4
        for (int jj = 0; jj < 32; jj++) {
            const int aj = __shfl_sync(0xffffffffu, at, jj);
            float x[VPL];
            const T* vp = (const T*)pg.v_pages + (size_t)max(aj, 0) * vdim + lane * VPL;
            if (vvec) {
                if (lane * VPL < vdim) load_run<T, VPL>(vp, x, true);
            } else {
#pragma unroll
                for (int e = 0; e < VPL; e++) x[e] = lane * VPL + e < vdim ? to_f32(vp[e]) : 0.f;
            }
#pragma unroll
            for (int g = 0; g < GH; g++) {
                const float pj = __shfl_sync(0xffffffffu, p[g], jj);       // 0 where the lane's key does not exist
#pragma unroll
                for (int e = 0; e < VPL; e++)
                    if (aj >= 0 && lane * VPL + e < vdim) acc[g][e] = fmaf(pj, x[e], acc[g][e]);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < GH; g++) {
#pragma unroll
        for (int e = 0; e < VPL; e++) o_sh[(warp * GH + g) * 32 * VPL + lane * VPL + e] = acc[g][e];
        if (lane == 0) { ml_sh[(warp * GH + g) * 2] = m_run[g]; ml_sh[(warp * GH + g) * 2 + 1] = l_run[g]; }
    }
    __syncthreads();
    for (int g = 0; g < GH; g++) {
        const int h = h0 + g;
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; w++) m_all = fmaxf(m_all, ml_sh[(w * GH + g) * 2]);
        float l_all = 0.f, f[DEC_WARPS];
#pragma unroll
        for (int w = 0; w < DEC_WARPS; w++) {
            const float mw = ml_sh[(w * GH + g) * 2];
            f[w] = mw > -INFINITY ? expf(mw - m_all) : 0.f;
            l_all += ml_sh[(w * GH + g) * 2 + 1] * f[w];
        }
        for (int d = threadIdx.x; d < vdim; d += DEC_WARPS * 32) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; w++) o = fmaf(o_sh[(w * GH + g) * 32 * VPL + d], f[w], o);
            if (splits == 1) out[(size_t)b * o_stride + (size_t)h * vdim + d] = from_f32<T>(l_all > 0.f ? o / l_all : 0.f);
            else part_o[(((size_t)b * n_heads + h) * splits + sp) * vdim + d] = o;
        }
        if (splits > 1 && threadIdx.x == 0) {
            float* ml = part_ml + (((size_t)b * n_heads + h) * splits + sp) * 2;
            ml[0] = m_all; ml[1] = l_all;
        }
    }
}

template <typename T>
__global__ void attn_bias_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, T* __restrict__ out,
                                       long long o_stride, int n_heads, int vdim, int splits) {
    ti_pdl_trigger();
    ti_pdl_sync();
    part_o = ti_dependent(part_o); part_ml = ti_dependent(part_ml);
    const int b = blockIdx.y, h = blockIdx.x;
    const float* ml = part_ml + ((size_t)b * n_heads + h) * splits * 2;
    float m_all = -INFINITY;
    for (int s = 0; s < splits; s++) m_all = fmaxf(m_all, ml[2 * s]);
    float l_all = 0.f;
    for (int s = 0; s < splits; s++) l_all += ml[2 * s] > -INFINITY ? ml[2 * s + 1] * expf(ml[2 * s] - m_all) : 0.f;
    for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < splits; s++)
            if (ml[2 * s] > -INFINITY) o = fmaf(part_o[(((size_t)b * n_heads + h) * splits + s) * vdim + d], expf(ml[2 * s] - m_all), o);
        out[(size_t)b * o_stride + (size_t)h * vdim + d] = from_f32<T>(l_all > 0.f ? o / l_all : 0.f);
    }
}

int check_pages(const char* what, const void* k_pages, const void* v_pages, const int* page_table, int table_width, int page_size,
                int n_pages) {
    TI_REQUIRE(k_pages && v_pages && page_table && page_size > 0 && table_width > 0 && n_pages > 0, "%s: incomplete cache description", what);
    return 0;
}

}  // namespace

// qkv: [M, heads * dim + kv_heads * (dim + vdim)] of the engine's type, row stride ld; bias: float32 of a row's length or
// null; q_w, k_w: float32 [dim] or null (no norm).
extern "C" int ti_attn_bias_prepare(void* qkv, long long ld, const float* bias, const float* q_w, const float* k_w, float eps,
                                    const int* tok_pos, const int* tok_seq, const int* seq_slot, void* k_pages, void* v_pages,
                                    const int* page_table, int table_width, int page_size, int n_pages, int M, int n_heads,
                                    int n_kv_heads, int dim, int vdim, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_heads > 0 && n_kv_heads > 0 && dim > 0 && vdim > 0, "attn_bias_prepare: bad sizes");
    if (check_pages("attn_bias_prepare", k_pages, v_pages, page_table, table_width, page_size, n_pages)) return 1;
    Pages pg{k_pages, v_pages, page_table, table_width, page_size, n_pages};
    const long long rows = (long long)M * (n_heads + 2 * n_kv_heads);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<2>(attn_bias_prepare_kernel<T>, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, stream, (T*)qkv, ld, bias,
                                   q_w, k_w, eps, tok_pos, tok_seq, seq_slot, pg, M, n_heads, n_kv_heads, dim, vdim));
        TI_CHECK_LAUNCH("attn_bias_prepare");
        return 0;
    });
}

// q: [M, heads, dim] (row stride q_stride); out: [M, heads, vdim] (row stride o_stride); dist_bias: float32
// [heads, far + 1] or null; cap <= 0: no soft cap.
extern "C" int ti_attn_bias(const void* q, long long q_stride, void* out, long long o_stride, const int* cu_new,
                            const int* seq_start, const int* seq_slot, int n_seq, int max_new, const void* k_pages,
                            const void* v_pages, const int* page_table, int table_width, int page_size, int n_pages,
                            const float* dist_bias, int far, int n_heads, int n_kv_heads, int dim, int vdim, float scale,
                            float cap, int dtype, cudaStream_t stream) {
    if (n_seq == 0 || max_new == 0) return 0;
    TI_REQUIRE(n_seq > 0 && max_new > 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attn_bias: bad sizes");
    TI_REQUIRE(dim >= 1 && dim <= 256 && vdim >= 1 && vdim <= 256, "attn_bias: heads of %d and %d elements are not supported (up to 256)", dim, vdim);
    TI_REQUIRE(n_seq <= 65535 && n_heads <= 65535, "attn_bias: too many sequences or heads for one launch");
    TI_REQUIRE(!dist_bias || far >= 0, "attn_bias: a distance table needs its last distance");
    if (check_pages("attn_bias", k_pages, v_pages, page_table, table_width, page_size, n_pages)) return 1;
    Pages pg{k_pages, v_pages, page_table, table_width, page_size, n_pages};
    const size_t smem = ((size_t)(BQ + BKV) * (dim + 1) + (size_t)BKV * (vdim + 1) + (size_t)BQ * (BKV + 1)) * sizeof(float);
    dim3 grid((max_new + BQ - 1) / BQ, n_heads, n_seq);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        auto go = [&](auto mc) -> int {
            constexpr int MAXC = decltype(mc)::value;
            static size_t configured = 0;
            if (smem > configured) {
                TI_CUDA(cudaFuncSetAttribute(attn_bias_kernel<T, MAXC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                configured = smem;
            }
            TI_CUDA(ti_launch(attn_bias_kernel<T, MAXC>, grid, dim3(THREADS), smem, stream, (const T*)q, q_stride, (T*)out, o_stride,
                              cu_new, seq_start, seq_slot, pg, dist_bias, far, n_heads, n_kv_heads, dim, vdim, scale, cap));
            TI_CHECK_LAUNCH("attn_bias");
            return 0;
        };
        if (vdim <= 64) return go(std::integral_constant<int, 16>());
        if (vdim <= 128) return go(std::integral_constant<int, 32>());
        return go(std::integral_constant<int, 64>());
    });
}

// One query per sequence (its last position, seq_len - 1).  part_o: float32 [n_seq, heads, splits, vdim] and part_ml:
// float32 [n_seq, heads, splits, 2], both only when splits > 1.
extern "C" int ti_attn_bias_decode(const void* q, long long q_stride, void* out, long long o_stride, const int* seq_len,
                                   const int* seq_slot, int n_seq, const void* k_pages, const void* v_pages,
                                   const int* page_table, int table_width, int page_size, int n_pages, const float* dist_bias,
                                   int far, int n_heads, int n_kv_heads, int dim, int vdim, float scale, float cap, int splits,
                                   float* part_o, float* part_ml, int dtype, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && splits >= 1, "attn_bias_decode: bad sizes");
    TI_REQUIRE(dim >= 1 && dim <= 32 * DEC_MAXE && vdim >= 1 && vdim <= 32 * DEC_MAXE,
               "attn_bias_decode: heads of %d and %d elements are not supported (up to %d)", dim, vdim, 32 * DEC_MAXE);
    TI_REQUIRE(n_seq <= 65535 && n_heads <= 65535, "attn_bias_decode: too many sequences or heads for one launch");
    TI_REQUIRE(splits == 1 || (part_o && part_ml), "attn_bias_decode: split keys need scratch");
    if (check_pages("attn_bias_decode", k_pages, v_pages, page_table, table_width, page_size, n_pages)) return 1;
    Pages pg{k_pages, v_pages, page_table, table_width, page_size, n_pages};
    // query heads of one kv head per block: as many of 4, 2, 1 as divide the group; value elements per lane: 1, 2, 4 or 8
    const int group = n_heads / n_kv_heads;
    const int gh = group % 4 == 0 ? 4 : group % 2 == 0 ? 2 : 1;
    const int vpl = vdim <= 32 ? 1 : vdim <= 64 ? 2 : vdim <= 128 ? 4 : 8;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        auto go = [&](auto ghv, auto vplv) -> int {
            constexpr int GH = decltype(ghv)::value, VPL = decltype(vplv)::value;
            const size_t smem = ((size_t)GH * dim + (size_t)DEC_WARPS * GH * 32 * VPL + (size_t)DEC_WARPS * GH * 2) * sizeof(float);
            static size_t configured = 0;
            if (smem > 48 * 1024 && smem > configured) {
                TI_CUDA(cudaFuncSetAttribute(attn_bias_decode_kernel<T, GH, VPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                configured = smem;
            }
            TI_CUDA(ti_launch_class<3>(attn_bias_decode_kernel<T, GH, VPL>, dim3(splits, n_heads / GH, n_seq), dim3(DEC_WARPS * 32), smem, stream,
                                       (const T*)q, q_stride, (T*)out, o_stride, seq_len, seq_slot, pg, dist_bias, far, n_heads, n_kv_heads,
                                       dim, vdim, scale, cap, splits, part_o, part_ml));
            TI_CHECK_LAUNCH("attn_bias_decode");
            return 0;
        };
        auto with_vpl = [&](auto ghv) -> int {
            switch (vpl) {
                case 1: return go(ghv, std::integral_constant<int, 1>());
                case 2: return go(ghv, std::integral_constant<int, 2>());
                case 4: return go(ghv, std::integral_constant<int, 4>());
                default: return go(ghv, std::integral_constant<int, 8>());
            }
        };
        int rc = gh == 4 ? with_vpl(std::integral_constant<int, 4>()) : gh == 2 ? with_vpl(std::integral_constant<int, 2>())
                                                                                 : with_vpl(std::integral_constant<int, 1>());
        if (rc) return rc;
        if (splits > 1) {
            TI_CUDA(ti_launch_class<4>(attn_bias_merge_kernel<T>, dim3(n_heads, n_seq), dim3(64), 0, stream, (const float*)part_o,
                                       (const float*)part_ml, (T*)out, o_stride, n_heads, vdim, splits));
            TI_CHECK_LAUNCH("attn_bias_merge");
        }
        return 0;
    });
}
