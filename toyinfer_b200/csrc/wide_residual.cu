// A residual stream kept in float32 beside activations of the engine's type.
//
// Some designs ask for the sum over layers in 32-bit while projections run in bfloat16.
// The stream h[M, H] is then float32 whatever the engine's type, and what the layers add
// (up to three terms d0, d1, d2 of the engine's type, any of them absent) is added here, in
// the order ((d0 + d1) + h) + d2, without rounding.  One kernel does what a layer boundary
// needs: the sum (written back to h when asked), and the RMS norm of the new row,
// y = x * rsqrt(mean(x^2) + eps) * w, rounded once into the engine's type.  With `rows` it
// works on the gathered rows h[rows[r]] only and leaves h alone (the head's rows).
// The embedding gather into a float32 stream is here too.
#include "common.cuh"

namespace {

template <typename T>
__global__ void embed_wide_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                  int H, int vocab, float scale, int copies) {
    ti_pdl_trigger();
    ti_pdl_sync();
    ids = ti_dependent(ids);
    const int m = blockIdx.x;
    const int id = ids[m];
    const bool ok = id >= 0 && id < vocab;
    const T* src = table + (size_t)(ok ? id : 0) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float x = ok ? to_f32(src[i]) * scale : 0.f;
        for (int c = 0; c < copies; c++) out[((size_t)m * copies + c) * H + i] = x;
    }
}

// One block per output row.  W: type of the norm weight (float or T).
template <typename T, typename W>
__global__ void add_norm_wide_kernel(float* __restrict__ h, const T* __restrict__ d0, const T* __restrict__ d1,
                                     const T* __restrict__ d2, const int* __restrict__ rows, const W* __restrict__ w,
                                     T* __restrict__ out, float* __restrict__ sum_out, int H, int M, float eps, int write_back) {
    ti_pdl_trigger();
    extern __shared__ float row[];      // H floats + 33
    float* red = row + H;
    ti_pdl_sync();
    h = ti_dependent(h); d0 = ti_dependent(d0); d1 = ti_dependent(d1); d2 = ti_dependent(d2);
    const int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    const bool ok = src >= 0 && src < M;
    if (!ok) src = 0;
    const size_t base = (size_t)src * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x = h[base + i];
        if (d0 || d1) {
            float s = 0.f;
            if (d0) s = to_f32(d0[base + i]);
            if (d1) s = d0 ? s + to_f32(d1[base + i]) : to_f32(d1[base + i]);
            x += s;
        }
        if (d2) x += to_f32(d2[base + i]);
        if (!ok) x = 0.f;
        row[i] = x;
        if (write_back) h[base + i] = x;
        if (sum_out) sum_out[(size_t)r * H + i] = x;
        ss = fmaf(x, x, ss);
    }
    if (!out) return;
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float y = w ? row[i] * inv * to_f32(w[i]) : row[i];
        out[(size_t)r * H + i] = from_f32<T>(y);
    }
}

}  // namespace

// out: float32 [M, copies, H]: every token's row `copies` times over (the streams of a model with several).
extern "C" int ti_embed_wide(const void* table, const int* ids, float* out, int M, int H, int vocab, float scale,
                             int copies, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && H > 0 && vocab > 0 && copies >= 1, "embed_wide: bad sizes M=%d H=%d vocab=%d copies=%d", M, H, vocab, copies);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<1>(embed_wide_kernel<T>, dim3(M), dim3(128), 0, stream, (const T*)table, ids, out, H, vocab, scale, copies));
        TI_CHECK_LAUNCH("embed_wide");
        return 0;
    });
}

// h: float32 [M, H].  d0, d1, d2: [M, H] of the engine's type or null.  rows: null (every row of h, R == M)
// or R row indices.  w: norm weight (null: `out` is the rounded sum itself), float32 when w_f32.
// out: [R, H] of the engine's type or null.  sum_out: float32 [R, H] or null.  write_back: store the sum into h.
extern "C" int ti_add_norm_wide(float* h, const void* d0, const void* d1, const void* d2, const int* rows, const void* w,
                                int w_f32, void* out, float* sum_out, int R, int H, int M, float eps, int write_back,
                                int dtype, cudaStream_t stream) {
    if (R == 0) return 0;
    TI_REQUIRE(R > 0 && H > 0 && M > 0, "add_norm_wide: bad sizes R=%d H=%d M=%d", R, H, M);
    TI_REQUIRE(rows || R == M, "add_norm_wide: without row indices every row is taken (R=%d, M=%d)", R, M);
    TI_REQUIRE(!(rows && write_back), "add_norm_wide: gathered rows are not written back");
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    TI_REQUIRE(smem <= 200 * 1024, "add_norm_wide: rows of %d elements do not fit shared memory", H);
    int threads = 256;
    if (H <= 256) threads = 64;
    else if (H <= 1024) threads = 128;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        auto go = [&](auto wt) -> int {
            using W = decltype(wt);
            static size_t configured = 0;
            if (smem > 48 * 1024 && smem > configured) {
                TI_CUDA(cudaFuncSetAttribute(add_norm_wide_kernel<T, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                configured = smem;
            }
            TI_CUDA(ti_launch_class<1>(add_norm_wide_kernel<T, W>, dim3(R), dim3(threads), smem, stream, h, (const T*)d0,
                                       (const T*)d1, (const T*)d2, rows, (const W*)w, (T*)out, sum_out, H, M, eps, write_back));
            TI_CHECK_LAUNCH("add_norm_wide");
            return 0;
        };
        if (w_f32) return go(float());
        return go(T());
    });
}
