// Linear attention with a per-head decay ("lightning" attention) and the gated norm after it.
//
// Per head, with a state S [dim, vdim] in float32 that a sequence carries from token to token
// (zero when the sequence starts):
//     S_t = decay_h * S_{t-1} + k_t v_t^T,      o_t = S_t^T q_t
// where q, k, v are the projections' outputs after silu (z / (1 + exp(-z)), applied here as
// the values are loaded).  Everything of the recurrence is 32-bit.
//
// lightning_scan: a sequence's new tokens are scanned in order from the state in its slot,
// which is updated in place: whole prompts, single tokens and anything between are one
// kernel.  Grid (heads * column groups, sequences): a thread owns one column of S
// (dim registers) and needs no other thread's work; q and k of a run of tokens are staged in
// shared memory.
//
// lightning_chunk_*: the same for long runs of new tokens, in three kernels that work on
// chunks of C tokens in parallel: (1) every chunk's own contribution
// U_c = sum_s decay^(C-1-s) k_s v_s^T, (2) the states before every chunk by a scan over the
// chunks, S_c = decay^C S_{c-1} + U_c, (3) every token's output from the state before its
// chunk and the tokens of the chunk up to itself,
// o_t = decay^(t+1) S^T q_t + sum_{s<=t} decay^(t-s) (q_t . k_s) v_s.
//
// gated_rmsnorm: y = rms(o) * w * sigmoid(g) over all heads' outputs of a token together.
#include "common.cuh"

#include <type_traits>

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

constexpr int SCAN_TOK = 16;     // tokens staged at a time

template <typename T, int MAXD>
__global__ void lightning_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                      long long q_stride, long long k_stride, long long v_stride,
                                      float* __restrict__ o, float* __restrict__ state, const float* __restrict__ decay,
                                      const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                                      int n_heads, int dim, int vdim, int groups) {
    ti_pdl_trigger();
    extern __shared__ float sm[];        // q: [SCAN_TOK][dim], k: [SCAN_TOK][dim]
    ti_pdl_sync();
    q = ti_dependent(q); k = ti_dependent(k); v = ti_dependent(v);
    float* qs = sm;
    float* ks = sm + SCAN_TOK * dim;
    const int h = blockIdx.x / groups, g = blockIdx.x - h * groups;
    const int b = blockIdx.y;
    const int tok0 = cu_new[b], n = cu_new[b + 1] - tok0;
    if (n <= 0) return;
    const int slot = seq_slot[b];
    const int col = g * blockDim.x + threadIdx.x;
    const bool live = col < vdim;
    const float lam = decay[h];
    float S[MAXD];
    float* srow = state + ((size_t)slot * n_heads + h) * dim * vdim;
#pragma unroll
    for (int i = 0; i < MAXD; i++) S[i] = (live && i < dim) ? srow[(size_t)i * vdim + col] : 0.f;
    for (int t0 = 0; t0 < n; t0 += SCAN_TOK) {
        const int nt = min(SCAN_TOK, n - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * dim; idx += blockDim.x) {
            const int tt = idx / dim, i = idx - tt * dim;
            const size_t tok = (size_t)(tok0 + t0 + tt);
            qs[idx] = silu_f(to_f32(q[tok * q_stride + (size_t)h * dim + i]));
            ks[idx] = silu_f(to_f32(k[tok * k_stride + (size_t)h * dim + i]));
        }
        __syncthreads();
        if (live) {
            for (int tt = 0; tt < nt; tt++) {
                const size_t tok = (size_t)(tok0 + t0 + tt);
                const float vv = silu_f(to_f32(v[tok * v_stride + (size_t)h * vdim + col]));
                const float* kr = ks + tt * dim;
                const float* qr = qs + tt * dim;
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < MAXD; i++) {
                    if (i < dim) {
                        S[i] = fmaf(lam, S[i], kr[i] * vv);
                        acc = fmaf(S[i], qr[i], acc);
                    }
                }
                o[tok * ((size_t)n_heads * vdim) + (size_t)h * vdim + col] = acc;
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < MAXD; i++)
            if (i < dim) srow[(size_t)i * vdim + col] = S[i];
    }
}

// ---------------------------------------------------------------------------
// chunked form
// ---------------------------------------------------------------------------
constexpr int CH = 64;           // tokens per chunk

// chunk c of sequence b covers its new tokens [c * CH, min(n, (c + 1) * CH)); chunk_of[b] is the index of
// the sequence's first chunk among all chunks of the step (a prefix sum of ceil(n / CH)).
struct Chunks { const int* cu_new; const int* seq_slot; int n_seq; };

__device__ __forceinline__ bool find_chunk(const Chunks& cz, int chunk, int& b, int& c, int& tok0, int& n) {
    // a linear walk over the sequences: steps have few of them
    int seen = 0;
    for (int s = 0; s < cz.n_seq; s++) {
        const int a = cz.cu_new[s], len = cz.cu_new[s + 1] - a;
        const int nchunks = (len + CH - 1) / CH;
        if (chunk < seen + nchunks) { b = s; c = chunk - seen; tok0 = a; n = len; return true; }
        seen += nchunks;
    }
    return false;
}

// (1) U[chunk, h] = sum_s lam^(len-1-s) k_s v_s^T over the chunk's tokens; thread owns a column.
template <typename T, int MAXD>
__global__ void lightning_chunk_local_kernel(const T* __restrict__ k, const T* __restrict__ v, long long k_stride,
                                             long long v_stride, float* __restrict__ U, const float* __restrict__ decay,
                                             Chunks cz, int n_heads, int dim, int vdim, int groups) {
    ti_pdl_trigger();
    extern __shared__ float ks[];        // [CH][dim]
    ti_pdl_sync();
    k = ti_dependent(k); v = ti_dependent(v);
    const int h = blockIdx.x / groups, g = blockIdx.x - h * groups;
    int b, c, tok0, n;
    if (!find_chunk(cz, blockIdx.y, b, c, tok0, n)) return;
    const int t0 = c * CH, nt = min(CH, n - t0);
    const int col = g * blockDim.x + threadIdx.x;
    const bool live = col < vdim;
    const float lam = decay[h];
    for (int idx = threadIdx.x; idx < nt * dim; idx += blockDim.x) {
        const int tt = idx / dim, i = idx - tt * dim;
        ks[idx] = silu_f(to_f32(k[(size_t)(tok0 + t0 + tt) * k_stride + (size_t)h * dim + i]));
    }
    __syncthreads();
    if (!live) return;
    float S[MAXD];
#pragma unroll
    for (int i = 0; i < MAXD; i++) S[i] = 0.f;
    for (int tt = 0; tt < nt; tt++) {
        const float vv = silu_f(to_f32(v[(size_t)(tok0 + t0 + tt) * v_stride + (size_t)h * vdim + col]));
        const float* kr = ks + tt * dim;
#pragma unroll
        for (int i = 0; i < MAXD; i++)
            if (i < dim) S[i] = fmaf(lam, S[i], kr[i] * vv);
    }
    float* u = U + ((size_t)blockIdx.y * n_heads + h) * dim * vdim;
#pragma unroll
    for (int i = 0; i < MAXD; i++)
        if (i < dim) u[(size_t)i * vdim + col] = S[i];
}

// (2) per sequence and head, over its chunks in order: U[chunk] <- state before the chunk, state <- state after the
// last chunk.  One thread per element of the state.
__global__ void lightning_chunk_scan_kernel(float* __restrict__ U, float* __restrict__ state, const float* __restrict__ decay,
                                            Chunks cz, int n_heads, int dim, int vdim) {
    ti_pdl_trigger();
    ti_pdl_sync();
    const int b = blockIdx.z, h = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= dim * vdim) return;
    int first = 0;
    for (int s = 0; s < b; s++) first += (cz.cu_new[s + 1] - cz.cu_new[s] + CH - 1) / CH;
    const int n = cz.cu_new[b + 1] - cz.cu_new[b];
    if (n <= 0) return;
    const int nchunks = (n + CH - 1) / CH;
    const float lam = decay[h];
    float* sp = state + ((size_t)cz.seq_slot[b] * n_heads + h) * dim * vdim + e;
    float S = *sp;
    for (int c = 0; c < nchunks; c++) {
        const int nt = min(CH, n - c * CH);
        float* u = U + ((size_t)(first + c) * n_heads + h) * dim * vdim + e;
        const float own = *u;
        *u = S;
        S = fmaf(powf(lam, (float)nt), S, own);
    }
    *sp = S;
}

// (3) outputs of a chunk: thread owns an output column (the state's column in registers, the chunk's values of
// the column in shared memory); A[t][s] = lam^(t-s) (q_t . k_s) for s <= t is formed by the whole block first.
template <typename T, int MAXD>
__global__ void lightning_chunk_out_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                           long long q_stride, long long k_stride, long long v_stride,
                                           const float* __restrict__ U, float* __restrict__ o,
                                           const float* __restrict__ decay, Chunks cz, int n_heads, int dim, int vdim, int groups) {
    ti_pdl_trigger();
    extern __shared__ float sm[];
    ti_pdl_sync();
    q = ti_dependent(q); k = ti_dependent(k); v = ti_dependent(v); U = ti_dependent(U);
    const int ldq = dim + 1;
    float* qs = sm;                      // [CH][dim + 1]
    float* ks = qs + CH * ldq;           // [CH][dim + 1]
    float* A = ks + CH * ldq;            // [CH][CH + 1]
    float* pw = A + CH * (CH + 1);       // lam^0 .. lam^CH
    float* vs = pw + CH + 1;             // [CH][blockDim.x]
    const int h = blockIdx.x / groups, g = blockIdx.x - h * groups;
    int b, c, tok0, n;
    if (!find_chunk(cz, blockIdx.y, b, c, tok0, n)) return;
    const int t0 = c * CH, nt = min(CH, n - t0);
    const float lam = decay[h];
    const int col = g * blockDim.x + threadIdx.x;
    const bool live = col < vdim;
    for (int idx = threadIdx.x; idx < nt * dim; idx += blockDim.x) {
        const int tt = idx / dim, i = idx - tt * dim;
        const size_t tok = (size_t)(tok0 + t0 + tt);
        qs[tt * ldq + i] = silu_f(to_f32(q[tok * q_stride + (size_t)h * dim + i]));
        ks[tt * ldq + i] = silu_f(to_f32(k[tok * k_stride + (size_t)h * dim + i]));
    }
    for (int tt = 0; tt < nt; tt++)
        vs[tt * blockDim.x + threadIdx.x] = live ? silu_f(to_f32(v[(size_t)(tok0 + t0 + tt) * v_stride + (size_t)h * vdim + col])) : 0.f;
    for (int i = threadIdx.x; i <= CH; i += blockDim.x) pw[i] = powf(lam, (float)i);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * nt; idx += blockDim.x) {
        const int tt = idx / nt, ss = idx - tt * nt;
        float a = 0.f;
        if (ss <= tt) {
            for (int i = 0; i < dim; i++) a = fmaf(qs[tt * ldq + i], ks[ss * ldq + i], a);
            a *= pw[tt - ss];
        }
        A[tt * (CH + 1) + ss] = a;
    }
    __syncthreads();
    if (!live) return;
    const float* Sg = U + ((size_t)blockIdx.y * n_heads + h) * dim * vdim;      // the state before this chunk
    float S[MAXD];
#pragma unroll
    for (int i = 0; i < MAXD; i++) S[i] = i < dim ? Sg[(size_t)i * vdim + col] : 0.f;
    for (int tt = 0; tt < nt; tt++) {
        float acc = 0.f;
        const float* qr = qs + tt * ldq;
#pragma unroll
        for (int i = 0; i < MAXD; i++)
            if (i < dim) acc = fmaf(S[i], qr[i], acc);
        acc *= pw[tt + 1];
        const float* arow = A + tt * (CH + 1);
        for (int ss = 0; ss <= tt; ss++) acc = fmaf(arow[ss], vs[ss * blockDim.x + threadIdx.x], acc);
        o[(size_t)(tok0 + t0 + tt) * ((size_t)n_heads * vdim) + (size_t)h * vdim + col] = acc;
    }
}

// ---------------------------------------------------------------------------
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ g, long long g_stride,
                                     const float* __restrict__ w, T* __restrict__ out, int N, float eps) {
    ti_pdl_trigger();
    __shared__ float red[33];
    ti_pdl_sync();
    o = ti_dependent(o); g = ti_dependent(g);
    const size_t m = blockIdx.x;
    const float* orow = o + m * N;
    float ss = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) ss = fmaf(orow[i], orow[i], ss);
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)N + eps);
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const float gate = 1.0f / (1.0f + expf(-to_f32(g[m * g_stride + i])));
        out[m * N + i] = from_f32<T>(orow[i] * inv * w[i] * gate);
    }
}

template <typename F>
int dispatch_dim(int dim, F&& f) {
    if (dim <= 32) return f(std::integral_constant<int, 32>());
    if (dim <= 64) return f(std::integral_constant<int, 64>());
    if (dim <= 128) return f(std::integral_constant<int, 128>());
    ti_set_error("lightning: heads of %d query/key elements are not supported (up to 128)", dim);
    return 1;
}

int column_threads(int vdim) { return vdim <= 32 ? 32 : vdim <= 64 ? 64 : 128; }

}  // namespace

// q, k: [M, heads, dim], v: [M, heads, vdim] (token strides given), before silu.  o: float32 [M, heads * vdim].
// state: float32 [slots, heads, dim, vdim].
extern "C" int ti_lightning_scan(const void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                 long long v_stride, float* o, float* state, const float* decay, const int* cu_new,
                                 const int* seq_slot, int n_seq, int n_heads, int dim, int vdim, int dtype, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_seq <= 65535 && n_heads > 0 && dim > 0 && vdim > 0, "lightning_scan: bad sizes");
    const int threads = column_threads(vdim), groups = (vdim + threads - 1) / threads;
    const size_t smem = (size_t)2 * SCAN_TOK * dim * sizeof(float);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        return dispatch_dim(dim, [&](auto md) -> int {
            constexpr int MAXD = decltype(md)::value;
            TI_CUDA(ti_launch(lightning_scan_kernel<T, MAXD>, dim3(n_heads * groups, n_seq), dim3(threads), smem, stream,
                              (const T*)q, (const T*)k, (const T*)v, q_stride, k_stride, v_stride, o, state, decay, cu_new,
                              seq_slot, n_heads, dim, vdim, groups));
            TI_CHECK_LAUNCH("lightning_scan");
            return 0;
        });
    });
}

// The chunked form: n_chunks >= sum over sequences of ceil(new tokens / 64) (an upper bound is enough);
// U: float32 scratch [n_chunks, heads, dim, vdim].
extern "C" int ti_lightning_chunked(const void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                    long long v_stride, float* o, float* state, float* U, const float* decay,
                                    const int* cu_new, const int* seq_slot, int n_seq, int n_chunks, int n_heads, int dim,
                                    int vdim, int dtype, cudaStream_t stream) {
    if (n_seq == 0 || n_chunks == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_seq <= 65535 && n_chunks > 0 && n_chunks <= 65535 && n_heads > 0 && n_heads <= 65535 && dim > 0 && vdim > 0,
               "lightning_chunked: bad sizes");
    const int threads = column_threads(vdim), groups = (vdim + threads - 1) / threads;
    Chunks cz{cu_new, seq_slot, n_seq};
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        return dispatch_dim(dim, [&](auto md) -> int {
            constexpr int MAXD = decltype(md)::value;
            const size_t smem1 = (size_t)CH * dim * sizeof(float);
            TI_CUDA(ti_launch(lightning_chunk_local_kernel<T, MAXD>, dim3(n_heads * groups, n_chunks), dim3(threads), smem1, stream,
                              (const T*)k, (const T*)v, k_stride, v_stride, U, decay, cz, n_heads, dim, vdim, groups));
            TI_CHECK_LAUNCH("lightning_chunk_local");
            TI_CUDA(ti_launch(lightning_chunk_scan_kernel, dim3((dim * vdim + 127) / 128, n_heads, n_seq), dim3(128), 0, stream,
                              U, state, decay, cz, n_heads, dim, vdim));
            TI_CHECK_LAUNCH("lightning_chunk_scan");
            const size_t smem3 = ((size_t)2 * CH * (dim + 1) + (size_t)CH * (CH + 1) + CH + 1 + (size_t)CH * threads) * sizeof(float);
            static size_t configured = 0;
            if (smem3 > 48 * 1024 && smem3 > configured) {
                TI_CUDA(cudaFuncSetAttribute(lightning_chunk_out_kernel<T, MAXD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3));
                configured = smem3;
            }
            TI_CUDA(ti_launch(lightning_chunk_out_kernel<T, MAXD>, dim3(n_heads * groups, n_chunks), dim3(threads), smem3, stream,
                              (const T*)q, (const T*)k, (const T*)v, q_stride, k_stride, v_stride, (const float*)U, o, decay, cz,
                              n_heads, dim, vdim, groups));
            TI_CHECK_LAUNCH("lightning_chunk_out");
            return 0;
        });
    });
}

// o: float32 [M, N]; g: [M, N] of the engine's type with row stride g_stride; w: float32 [N]; out: [M, N].
extern "C" int ti_gated_rmsnorm(const float* o, const void* g, long long g_stride, const float* w, void* out, int M, int N,
                                float eps, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && N > 0 && g_stride >= N, "gated_rmsnorm: bad sizes M=%d N=%d", M, N);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        const int threads = N <= 256 ? 64 : N <= 1024 ? 128 : 256;
        TI_CUDA(ti_launch_class<1>(gated_rmsnorm_kernel<T>, dim3(M), dim3(threads), 0, stream, o, (const T*)g, g_stride, w, (T*)out, N, eps));
        TI_CHECK_LAUNCH("gated_rmsnorm");
        return 0;
    });
}
