// The real-gated linear recurrent unit of a Griffin-style recurrent block.
//
// Per channel c, with the convolved input u_t, the gate logits p_t (recurrence gate) and n_t (input
// gate) that block-diagonal matrices made from u_t, and the other branch's projection z_t:
//     r = sigmoid(p_t + bp[c]),  i = sigmoid(n_t + bn[c]),  a = exp(-rate[c] * r)   (rate = 8 softplus(lam), made once),
//     S_t = a * S_{t-1} + sqrt(1 - a^2) * (i * u_t),        out_t = S_t * gelu_tanh(z_t + bz[c]).
// S is float32, one value per channel and sequence, zero when the sequence starts (the first token
// is no special case) and updated in place; everything of the recurrence is 32-bit.  A thread owns
// a channel of a sequence and walks the step's tokens in order: whole prompts, single tokens and
// anything between are one kernel.  The loads of the next tokens do not wait for the recurrence.  Long runs of new tokens
// take the chunked form further down instead.
#include "common.cuh"

namespace {

constexpr int LRU_THREADS = 128, LRU_AHEAD = 4;

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// gates: float32 [M, 2 C]; channel c of gate block k = c / bs sits at column k * 2 bs + (c % bs) (recurrence gate)
// and bs columns further (input gate).
template <typename T>
__global__ void __launch_bounds__(LRU_THREADS)
rglru_scan_kernel(const float* __restrict__ gates, const T* __restrict__ u, long long ldu, const T* __restrict__ z, long long ldz,
                  const float* __restrict__ bp, const float* __restrict__ bn, const float* __restrict__ bz,
                  const float* __restrict__ rate, float* __restrict__ state, long long slot_stride, T* __restrict__ out,
                  const int* __restrict__ cu_new, const int* __restrict__ seq_slot, int C, int bs) {
    ti_pdl_trigger();
    const int c = blockIdx.x * LRU_THREADS + threadIdx.x;
    float b_p = 0.f, b_n = 0.f, b_z = 0.f, rt = 0.f;
    if (c < C) { b_p = bp[c]; b_n = bn[c]; b_z = bz ? bz[c] : 0.f; rt = rate[c]; }
    ti_pdl_sync();
    gates = ti_dependent(gates); u = ti_dependent(u); z = ti_dependent(z);
    const int b = blockIdx.y;
    const int tok0 = cu_new[b], n = cu_new[b + 1] - tok0;
    if (n <= 0 || c >= C) return;
    const int gcol = (c / bs) * 2 * bs + (c % bs);
    float* sp = state + (size_t)seq_slot[b] * slot_stride + c;
    float S = *sp;
    for (int t0 = 0; t0 < n; t0 += LRU_AHEAD) {
        float p[LRU_AHEAD], q[LRU_AHEAD], uu[LRU_AHEAD], zz[LRU_AHEAD];
#pragma unroll
        for (int k = 0; k < LRU_AHEAD; k++) {
            const size_t tok = (size_t)(tok0 + min(t0 + k, n - 1));
            p[k] = gates[tok * 2 * C + gcol];
            q[k] = gates[tok * 2 * C + gcol + bs];
            uu[k] = to_f32(u[tok * ldu + c]);
            zz[k] = to_f32(z[tok * ldz + c]);
        }
#pragma unroll
        for (int k = 0; k < LRU_AHEAD; k++) {
            if (t0 + k < n) {
                const float a = expf(-rt * sigmoid_f(p[k] + b_p));
                const float in = sigmoid_f(q[k] + b_n) * uu[k];
                S = fmaf(a, S, sqrtf(fmaxf(1.0f - a * a, 0.f)) * in);
                out[(size_t)(tok0 + t0 + k) * C + c] = from_f32<T>(S * gelu_tanh_f(zz[k] + b_z));
            }
        }
    }
    *sp = S;
}

// The same recurrence for long runs of new tokens, in three kernels over chunks of LRU_CHUNK tokens: (1) every chunk's own
// effect on the state, S_out = A S_in + B with A the product of its decays and B what it leaves from S_in = 0; (2) per
// channel, the states before every chunk by a walk over the chunks' (A, B), which also leaves the sequence's state for the
// next step; (3) every chunk again from the state before it, now writing the outputs.  Chunks work in parallel; the
// inputs are read twice.
constexpr int LRU_CHUNK = 128;

template <typename T>
__device__ __forceinline__ void lru_coeffs(const float* __restrict__ gates, const T* __restrict__ u, long long ldu, size_t tok, int C,
                                           int gcol, int bs, int c, float b_p, float b_n, float rt, float& a, float& in) {
    a = expf(-rt * sigmoid_f(gates[tok * 2 * C + gcol] + b_p));
    in = sqrtf(fmaxf(1.0f - a * a, 0.f)) * sigmoid_f(gates[tok * 2 * C + gcol + bs] + b_n) * to_f32(u[tok * ldu + c]);
}

// AB: float32 [n_seq, chunks, 2, C]
template <typename T>
__global__ void __launch_bounds__(LRU_THREADS)
rglru_chunk_effect_kernel(const float* __restrict__ gates, const T* __restrict__ u, long long ldu, const float* __restrict__ bp,
                          const float* __restrict__ bn, const float* __restrict__ rate, float* __restrict__ AB,
                          const int* __restrict__ cu_new, int C, int bs, int chunks) {
    ti_pdl_trigger();
    const int c = blockIdx.x * LRU_THREADS + threadIdx.x;
    ti_pdl_sync();
    gates = ti_dependent(gates); u = ti_dependent(u);
    const int b = blockIdx.z, ch = blockIdx.y;
    const int tok0 = cu_new[b], n = cu_new[b + 1] - tok0;
    const int t0 = ch * LRU_CHUNK;
    if (t0 >= n || c >= C) return;
    const int nt = min(LRU_CHUNK, n - t0), gcol = (c / bs) * 2 * bs + (c % bs);
    const float b_p = bp[c], b_n = bn[c], rt = rate[c];
    float A = 1.f, B = 0.f;
#pragma unroll 4
    for (int t = 0; t < nt; t++) {
        float a, in;
        lru_coeffs(gates, u, ldu, (size_t)(tok0 + t0 + t), C, gcol, bs, c, b_p, b_n, rt, a, in);
        A *= a;
        B = fmaf(a, B, in);
    }
    float* ab = AB + ((size_t)b * chunks + ch) * 2 * C;
    ab[c] = A;
    ab[C + c] = B;
}

// AB's A entries become the states before the chunks; the sequence's state moves on to after its last token
__global__ void rglru_chunk_carry_kernel(float* __restrict__ AB, float* __restrict__ state, long long slot_stride,
                                         const int* __restrict__ cu_new, const int* __restrict__ seq_slot, int C, int chunks) {
    ti_pdl_trigger();
    ti_pdl_sync();
    AB = ti_dependent(AB);
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    const int n = cu_new[b + 1] - cu_new[b];
    if (n <= 0 || c >= C) return;
    float* sp = state + (size_t)seq_slot[b] * slot_stride + c;
    float S = *sp;
    const int used = (n + LRU_CHUNK - 1) / LRU_CHUNK;
    for (int ch = 0; ch < used; ch++) {
        float* ab = AB + ((size_t)b * chunks + ch) * 2 * C;
        const float A = ab[c], B = ab[C + c];
        ab[c] = S;
        S = fmaf(A, S, B);
    }
    *sp = S;
}

template <typename T>
__global__ void __launch_bounds__(LRU_THREADS)
rglru_chunk_out_kernel(const float* __restrict__ gates, const T* __restrict__ u, long long ldu, const T* __restrict__ z, long long ldz,
                       const float* __restrict__ bp, const float* __restrict__ bn, const float* __restrict__ bz,
                       const float* __restrict__ rate, const float* __restrict__ AB, T* __restrict__ out,
                       const int* __restrict__ cu_new, int C, int bs, int chunks) {
    ti_pdl_trigger();
    const int c = blockIdx.x * LRU_THREADS + threadIdx.x;
    ti_pdl_sync();
    gates = ti_dependent(gates); u = ti_dependent(u); z = ti_dependent(z); AB = ti_dependent(AB);
    const int b = blockIdx.z, ch = blockIdx.y;
    const int tok0 = cu_new[b], n = cu_new[b + 1] - tok0;
    const int t0 = ch * LRU_CHUNK;
    if (t0 >= n || c >= C) return;
    const int nt = min(LRU_CHUNK, n - t0), gcol = (c / bs) * 2 * bs + (c % bs);
    const float b_p = bp[c], b_n = bn[c], b_z = bz ? bz[c] : 0.f, rt = rate[c];
    float S = AB[((size_t)b * chunks + ch) * 2 * C + c];
#pragma unroll 4
    for (int t = 0; t < nt; t++) {
        const size_t tok = (size_t)(tok0 + t0 + t);
        float a, in;
        lru_coeffs(gates, u, ldu, tok, C, gcol, bs, c, b_p, b_n, rt, a, in);
        S = fmaf(a, S, in);
        out[tok * C + c] = from_f32<T>(S * gelu_tanh_f(to_f32(z[tok * ldz + c]) + b_z));
    }
}

// A block-diagonal product for few tokens: out[m, b * N + n] = sum_k x[m, b * K + k] * W[b][n][k], float32 results.
// One warp per output column (b, n): its weight row is read once, the lanes over k, up to BD_TOK tokens at a time.
constexpr int BD_TOK = 16, BD_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(BD_WARPS * 32)
block_diag_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ W, float* __restrict__ out, long long ldo, int M,
                  int n_blocks, int N, int K) {
    ti_pdl_trigger();
    ti_pdl_sync();
    x = ti_dependent(x);
    const int lane = threadIdx.x & 31;
    const long long col = (long long)blockIdx.x * BD_WARPS + (threadIdx.x >> 5);
    if (col >= (long long)n_blocks * N) return;
    const int b = (int)(col / N);
    const T* w = W + (size_t)col * K;
    for (int m0 = 0; m0 < M; m0 += BD_TOK) {
        float acc[BD_TOK];
#pragma unroll
        for (int i = 0; i < BD_TOK; i++) acc[i] = 0.f;
        for (int k = lane; k < K; k += 32) {
            const float wv = to_f32(w[k]);
#pragma unroll
            for (int i = 0; i < BD_TOK; i++)
                if (m0 + i < M) acc[i] = fmaf(wv, to_f32(x[(size_t)(m0 + i) * ldx + (size_t)b * K + k]), acc[i]);
        }
#pragma unroll
        for (int i = 0; i < BD_TOK; i++) {
            const float v = warp_sum(acc[i]);
            if (lane == 0 && m0 + i < M) out[(size_t)(m0 + i) * ldo + col] = v;
        }
    }
}

}  // namespace

// gates: float32 [M, 2 C] (see the kernel); u: [M, C] row stride ldu; z: [M, C] row stride ldz; bp, bn, rate: float32 [C];
// bz: float32 [C] or null; state: float32, slot s at state + s * slot_stride holds [C]; out: [M, C] dense.
extern "C" int ti_rglru_scan(const float* gates, const void* u, long long ldu, const void* z, long long ldz, const float* bp,
                             const float* bn, const float* bz, const float* rate, float* state, long long slot_stride, void* out,
                             const int* cu_new, const int* seq_slot, int n_seq, int C, int bs, int dtype, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_seq <= 65535 && C > 0 && bs > 0 && C % bs == 0, "rglru_scan: bad sizes (channels %d, gate blocks of %d)", C, bs);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch(rglru_scan_kernel<T>, dim3((C + LRU_THREADS - 1) / LRU_THREADS, n_seq), dim3(LRU_THREADS), 0, stream, gates,
                          (const T*)u, ldu, (const T*)z, ldz, bp, bn, bz, rate, state, slot_stride, (T*)out, cu_new, seq_slot, C, bs));
        TI_CHECK_LAUNCH("rglru_scan");
        return 0;
    });
}

// x: [M, n_blocks * K] of the engine's type (row stride ldx); W: [n_blocks, N, K]; out: float32 [M, n_blocks * N] (row stride ldo).
extern "C" int ti_block_diag_linear(const void* x, long long ldx, const void* W, float* out, long long ldo, int M, int n_blocks,
                                    int N, int K, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_blocks > 0 && N > 0 && K > 0, "block_diag_linear: bad sizes");
    const long long cols = (long long)n_blocks * N;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch(block_diag_kernel<T>, dim3((unsigned)((cols + BD_WARPS - 1) / BD_WARPS)), dim3(BD_WARPS * 32), 0, stream,
                          (const T*)x, ldx, (const T*)W, out, ldo, M, n_blocks, N, K));
        TI_CHECK_LAUNCH("block_diag_linear");
        return 0;
    });
}

// The chunked form of ti_rglru_scan for steps whose longest run of new tokens is `max_new`; AB: float32 scratch
// [n_seq, ceil(max_new / 128), 2, C].
extern "C" int ti_rglru_scan_chunked(const float* gates, const void* u, long long ldu, const void* z, long long ldz, const float* bp,
                                     const float* bn, const float* bz, const float* rate, float* state, long long slot_stride,
                                     void* out, float* AB, const int* cu_new, const int* seq_slot, int n_seq, int max_new, int C,
                                     int bs, int dtype, cudaStream_t stream) {
    if (n_seq == 0 || max_new == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_seq <= 65535 && max_new > 0 && C > 0 && bs > 0 && C % bs == 0 && AB, "rglru_scan_chunked: bad sizes");
    const int chunks = (max_new + LRU_CHUNK - 1) / LRU_CHUNK, groups = (C + LRU_THREADS - 1) / LRU_THREADS;
    TI_REQUIRE(chunks <= 65535, "rglru_scan_chunked: %d new tokens are too many for one launch", max_new);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch(rglru_chunk_effect_kernel<T>, dim3(groups, chunks, n_seq), dim3(LRU_THREADS), 0, stream, gates, (const T*)u, ldu,
                          bp, bn, rate, AB, cu_new, C, bs, chunks));
        TI_CHECK_LAUNCH("rglru_chunk_effect");
        TI_CUDA(ti_launch(rglru_chunk_carry_kernel, dim3(groups, n_seq), dim3(LRU_THREADS), 0, stream, AB, state, slot_stride, cu_new,
                          seq_slot, C, chunks));
        TI_CHECK_LAUNCH("rglru_chunk_carry");
        TI_CUDA(ti_launch(rglru_chunk_out_kernel<T>, dim3(groups, chunks, n_seq), dim3(LRU_THREADS), 0, stream, gates, (const T*)u, ldu,
                          (const T*)z, ldz, bp, bn, bz, rate, (const float*)AB, (T*)out, cu_new, C, bs, chunks));
        TI_CHECK_LAUNCH("rglru_chunk_out");
        return 0;
    });
}
