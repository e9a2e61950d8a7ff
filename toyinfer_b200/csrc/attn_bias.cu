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
// attn_bias_decode: one query per sequence; a block takes one head and one of `splits` ranges of
// keys, a warp 32 keys at a time (a lane a key for the scores, then the lanes the value's
// elements); ranges are merged by a second kernel when there are several.
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

// a key row times the query (float32 in shared memory, scaled): 16-byte loads where the row allows them
template <typename T>
__device__ __forceinline__ float key_dot(const T* __restrict__ kp, const float* __restrict__ qs, int dim, bool vec) {
    float s = 0.f;
    if (vec) {
        constexpr int PER = 16 / sizeof(T);
        for (int d = 0; d < dim; d += PER) {
            const uint4 raw = *reinterpret_cast<const uint4*>(kp + d);
            const T* x = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int e = 0; e < PER; e++) s = fmaf(qs[d + e], to_f32(x[e]), s);
        }
    } else {
        for (int d = 0; d < dim; d++) s = fmaf(qs[d], to_f32(kp[d]), s);
    }
    return s;
}

// A warp takes 32 keys at a time: a lane a key for the scores (no sums across lanes), then the lanes the value's elements
// while the 32 weights and rows go round by shuffles.  part_o [n_seq, heads, splits, vdim], part_ml [n_seq, heads, splits, 2]
// when splits > 1.
template <typename T>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_bias_decode_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long o_stride,
                        const int* __restrict__ seq_len, const int* __restrict__ seq_slot, Pages pg,
                        const float* __restrict__ dist_bias, int far, int n_heads, int n_kv_heads, int dim, int vdim,
                        float scale, float cap, int splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
    ti_pdl_trigger();
    __shared__ float o_sh[DEC_WARPS][DEC_MAXE * 32];
    __shared__ float ml_sh[DEC_WARPS][2];
    __shared__ __align__(16) float q_sh[DEC_MAXE * 32];
    ti_pdl_sync();
    q = ti_dependent(q);
    const int b = blockIdx.z, h = blockIdx.y, sp = blockIdx.x;
    const int len = seq_len[b], slot = seq_slot[b];
    const int qi = len - 1;
    const int kvh = h / (n_heads / n_kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // ranges of whole tiles of 32 keys
    const int tiles = (len + 31) / 32, per = (tiles + splits - 1) / splits;
    const int t_lo = sp * per, t_hi = min(tiles, t_lo + per);
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    const float* hb = dist_bias ? dist_bias + (size_t)h * (far + 1) : nullptr;
    for (int d = threadIdx.x; d < dim; d += DEC_WARPS * 32) q_sh[d] = to_f32(q[(size_t)b * q_stride + (size_t)h * dim + d]) * scale;
    __syncthreads();
    const bool vec = (dim * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(pg.k_pages) & 15) == 0;
    float acc[DEC_MAXE];
#pragma unroll
    for (int e = 0; e < DEC_MAXE; e++) acc[e] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    for (int t = t_lo + warp; t < t_hi; t += DEC_WARPS) {
        const int j = t * 32 + lane;
        int at = -1;                                     // the key's row among all rows of the pages
        if (j < len) {
            const int pidx = j / pg.page_size;
            const int page = pidx < pg.table_width ? pg.page_table[(size_t)slot * pg.table_width + pidx] : -1;
            if (page >= 0 && page < pg.n_pages) at = (page * n_kv_heads + kvh) * pg.page_size + j % pg.page_size;
        }
        float s = -INFINITY;
        if (at >= 0) {
            s = capped(key_dot((const T*)pg.k_pages + (size_t)at * dim, q_sh, dim, vec), cap, inv_cap);
            if (hb) s += hb[min(qi - j, far)];
        }
        const float m_new = fmaxf(m_run, warp_max(s));
        if (m_new == -INFINITY) continue;                // (the same for all lanes)
        const float alpha = expf(m_run - m_new), p = at >= 0 ? expf(s - m_new) : 0.f;
        l_run = l_run * alpha + warp_sum(p);
        m_run = m_new;
#pragma unroll
        for (int e = 0; e < DEC_MAXE; e++) acc[e] *= alpha;
#pragma unroll 4
        for (int jj = 0; jj < 32; jj++) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int aj = __shfl_sync(0xffffffffu, at, jj);
            if (aj < 0) continue;
            const T* vp = (const T*)pg.v_pages + (size_t)aj * vdim;
#pragma unroll
            for (int e = 0; e < DEC_MAXE; e++) {
                const int d = lane + 32 * e;
                if (d < vdim) acc[e] = fmaf(pj, to_f32(vp[d]), acc[e]);
            }
        }
    }
#pragma unroll
    for (int e = 0; e < DEC_MAXE; e++) o_sh[warp][lane + 32 * e] = acc[e];
    if (lane == 0) { ml_sh[warp][0] = m_run; ml_sh[warp][1] = l_run; }
    __syncthreads();
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; w++) m_all = fmaxf(m_all, ml_sh[w][0]);
    float l_all = 0.f, f[DEC_WARPS];
#pragma unroll
    for (int w = 0; w < DEC_WARPS; w++) {
        f[w] = ml_sh[w][0] > -INFINITY ? expf(ml_sh[w][0] - m_all) : 0.f;
        l_all += ml_sh[w][1] * f[w];
    }
    for (int d = threadIdx.x; d < vdim; d += DEC_WARPS * 32) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; w++) o = fmaf(o_sh[w][d], f[w], o);
        if (splits == 1) out[(size_t)b * o_stride + (size_t)h * vdim + d] = from_f32<T>(l_all > 0.f ? o / l_all : 0.f);
        else part_o[(((size_t)b * n_heads + h) * splits + sp) * vdim + d] = o;
    }
    if (splits > 1 && threadIdx.x == 0) {
        float* ml = part_ml + (((size_t)b * n_heads + h) * splits + sp) * 2;
        ml[0] = m_all; ml[1] = l_all;
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
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<3>(attn_bias_decode_kernel<T>, dim3(splits, n_heads, n_seq), dim3(DEC_WARPS * 32), 0, stream, (const T*)q,
                                   q_stride, (T*)out, o_stride, seq_len, seq_slot, pg, dist_bias, far, n_heads, n_kv_heads, dim, vdim,
                                   scale, cap, splits, part_o, part_ml));
        TI_CHECK_LAUNCH("attn_bias_decode");
        if (splits > 1) {
            TI_CUDA(ti_launch_class<4>(attn_bias_merge_kernel<T>, dim3(n_heads, n_seq), dim3(64), 0, stream, (const float*)part_o,
                                       (const float*)part_ml, (T*)out, o_stride, n_heads, vdim, splits));
            TI_CHECK_LAUNCH("attn_bias_merge");
        }
        return 0;
    });
}
