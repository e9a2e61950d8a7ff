// The real-gated linear recurrent unit of a Griffin-style recurrent block.
//
// Per channel c, with the convolved input u_t, the gate logits p_t (recurrence gate) and n_t (input
// gate) that block-diagonal matrices made from u_t, and the other branch's projection z_t:
//     r = sigmoid(p_t + bp[c]),  i = sigmoid(n_t + bn[c]),  a = exp(-rate[c] * r)   (rate = 8 softplus(lam), made once),
//     S_t = a * S_{t-1} + sqrt(1 - a^2) * (i * u_t),        out_t = S_t * gelu_tanh(z_t + bz[c]).
// S is float32, one value per channel and sequence, zero when the sequence starts (the first token
// is no special case) and updated in place; everything of the recurrence is 32-bit.  A thread owns
// a channel of a sequence and walks the step's tokens in order: whole prompts, single tokens and
// anything between are one kernel.  The loads of the next tokens do not wait for the recurrence.
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
