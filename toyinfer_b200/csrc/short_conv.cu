// A short causal convolution over time, one filter per channel, with the last inputs of every
// sequence kept as state.
//
// For channel c of a sequence whose inputs are x_0, x_1, ... (x_t = projection + input bias):
//     y_t = act(sum_{j < n} taps[c][j] * x_{t - (n - 1 - j)} + out_bias[c]),    x_s = 0 for s < 0,
// so the last column of `taps` weighs the current token.  The state of a sequence is its last
// n - 1 inputs, float32 [n - 1, C] (oldest first), zero when the sequence starts; a step reads it
// for its first tokens and leaves it holding the step's last inputs, however many tokens the
// step brings.  act: 0 none, 1 silu.
//
// short_conv: grid (token chunks of 64, channel groups, sequences); a thread owns one channel and
// walks its chunk's tokens with the window in registers.  A sequence whose new tokens fit one
// chunk gets its state updated by the same block; for longer ones short_conv_tail runs afterwards
// (other blocks still read the old state while the chunk with the last tokens is at work).
#include "common.cuh"

#include <type_traits>

namespace {

constexpr int CONV_CHUNK = 64, CONV_THREADS = 128, MAX_TAPS = 8;

__device__ __forceinline__ float conv_act(float z, int act) { return act == 1 ? z / (1.0f + expf(-z)) : z; }

template <typename T, int N>
__global__ void __launch_bounds__(CONV_THREADS)
short_conv_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ in_bias, const float* __restrict__ taps,
                  const float* __restrict__ out_bias, int act, float* __restrict__ state, long long slot_stride,
                  T* __restrict__ out, long long ldo, const int* __restrict__ cu_new, const int* __restrict__ seq_slot, int C) {
    ti_pdl_trigger();
    const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
    float w[N];
    float ib = 0.f, ob = 0.f;
    if (c < C) {
#pragma unroll
        for (int j = 0; j < N; j++) w[j] = taps[(size_t)c * N + j];
        if (in_bias) ib = in_bias[c];
        if (out_bias) ob = out_bias[c];
    }
    ti_pdl_sync();
    x = ti_dependent(x);
    const int b = blockIdx.z;
    const int tok0 = cu_new[b], n = cu_new[b + 1] - tok0;
    const int t0 = blockIdx.x * CONV_CHUNK;
    if (t0 >= n || c >= C) return;
    const int nt = min(CONV_CHUNK, n - t0);
    float* st = state + (size_t)seq_slot[b] * slot_stride;      // [N - 1, C]
    // win[j]: the input N - 1 - j tokens before the one at hand
    float win[N > 1 ? N - 1 : 1];
#pragma unroll
    for (int j = 0; j < N - 1; j++) {
        const int s = t0 - (N - 1 - j);                 // index among the step's tokens; negative: from the state
        win[j] = s >= 0 ? to_f32(x[(size_t)(tok0 + s) * ldx + c]) + ib : st[(size_t)(N - 1 + s) * C + c];
    }
    for (int t = 0; t < nt; t++) {
        const float cur = to_f32(x[(size_t)(tok0 + t0 + t) * ldx + c]) + ib;
        float a = ob;
#pragma unroll
        for (int j = 0; j < N - 1; j++) a = fmaf(w[j], win[j], a);
        a = fmaf(w[N - 1], cur, a);
        out[(size_t)(tok0 + t0 + t) * ldo + c] = from_f32<T>(conv_act(a, act));
#pragma unroll
        for (int j = 0; j + 1 < N - 1; j++) win[j] = win[j + 1];
        if constexpr (N > 1) win[N - 2] = cur;
    }
    if (n <= CONV_CHUNK) {
#pragma unroll
        for (int j = 0; j < N - 1; j++) st[(size_t)j * C + c] = win[j];
    }
}

// The state of the sequences with more than one chunk of new tokens: their last N - 1 inputs.
template <typename T, int N>
__global__ void short_conv_tail_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ in_bias,
                                       float* __restrict__ state, long long slot_stride, const int* __restrict__ cu_new,
                                       const int* __restrict__ seq_slot, int C) {
    ti_pdl_trigger();
    ti_pdl_sync();
    x = ti_dependent(x);
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    const int tok0 = cu_new[b], n = cu_new[b + 1] - tok0;
    if (n <= CONV_CHUNK || c >= C) return;
    float* st = state + (size_t)seq_slot[b] * slot_stride;
    const float ib = in_bias ? in_bias[c] : 0.f;
#pragma unroll
    for (int j = 0; j < N - 1; j++) st[(size_t)j * C + c] = to_f32(x[(size_t)(tok0 + n - (N - 1) + j) * ldx + c]) + ib;
}

template <typename F>
int dispatch_taps(int n, F&& f) {
    switch (n) {
        case 1: return f(std::integral_constant<int, 1>());
        case 2: return f(std::integral_constant<int, 2>());
        case 3: return f(std::integral_constant<int, 3>());
        case 4: return f(std::integral_constant<int, 4>());
        case 5: return f(std::integral_constant<int, 5>());
        case 6: return f(std::integral_constant<int, 6>());
        case 7: return f(std::integral_constant<int, 7>());
        default: return f(std::integral_constant<int, 8>());
    }
}

}  // namespace

// x: [M, C] of the engine's type with row stride ldx; in_bias, out_bias: float32 [C] or null; taps: float32 [C, n];
// state: float32, sequence slot s at state + s * slot_stride holds [n - 1, C]; out: [M, C] with row stride ldo.
extern "C" int ti_short_conv(const void* x, long long ldx, const float* in_bias, const float* taps, const float* out_bias,
                             int act, float* state, long long slot_stride, void* out, long long ldo, const int* cu_new,
                             const int* seq_slot, int n_seq, int max_new, int C, int n_taps, int dtype, cudaStream_t stream) {
    if (n_seq == 0 || max_new == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_seq <= 65535 && max_new > 0 && C > 0, "short_conv: bad sizes");
    TI_REQUIRE(n_taps >= 1 && n_taps <= MAX_TAPS, "short_conv: %d taps are not supported (1 to %d)", n_taps, MAX_TAPS);
    TI_REQUIRE(act == 0 || act == 1, "short_conv: unknown activation %d", act);
    const int chunks = (max_new + CONV_CHUNK - 1) / CONV_CHUNK, groups = (C + CONV_THREADS - 1) / CONV_THREADS;
    TI_REQUIRE(groups <= 65535, "short_conv: %d channels are too many for one launch", C);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        return dispatch_taps(n_taps, [&](auto nv) -> int {
            constexpr int N = decltype(nv)::value;
            TI_CUDA(ti_launch(short_conv_kernel<T, N>, dim3(chunks, groups, n_seq), dim3(CONV_THREADS), 0, stream, (const T*)x, ldx,
                              in_bias, taps, out_bias, act, state, slot_stride, (T*)out, ldo, cu_new, seq_slot, C));
            TI_CHECK_LAUNCH("short_conv");
            if (chunks > 1 && N > 1) {
                TI_CUDA(ti_launch(short_conv_tail_kernel<T, N>, dim3(groups, n_seq), dim3(CONV_THREADS), 0, stream, (const T*)x, ldx,
                                  in_bias, state, slot_stride, cu_new, seq_slot, C));
                TI_CHECK_LAUNCH("short_conv_tail");
            }
            return 0;
        });
    });
}
