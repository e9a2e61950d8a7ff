// The gated delta rule with one decay per key channel, and the per-head gated norm after it.
//
// Per head, with a state S [dim, vdim] in float32 that a sequence carries from token to token
// (zero when the sequence starts), a unit query q and key k [dim], a value v [vdim], a write
// strength beta and a decay g [dim] per token:
//     S <- diag(g) S;   e = beta * (v - S^T k);   S <- S + k e^T;   o = S^T q
// in this order, so that the read-out sees the token's own write.  Query and key arrive unnormalised
// (after their short convolution and silu) and are made unit vectors here, x / sqrt(sum x^2 + 1e-6),
// the query also times dim^-1/2.  The decay comes as the logit l of a low-rank projection:
// g = exp(-rate_h * softplus(l + dt)), rate_h = exp(A_h) made once.  beta = sigmoid of its logit.
// Value head h reads query/key head h / (heads / qk_heads).  Everything of the recurrence is 32-bit.
//
// delta_rule_scan: a sequence's new tokens are scanned in order from the state in its slot, which
// is updated in place: whole prompts, single tokens and anything between are one kernel.  Grid
// (heads * column groups of 32, sequences): four neighbouring lanes share one column of S (a quarter
// of its rows in registers each) and add up their parts of the two sums over the column by shuffles;
// q, k, g and v of a run of tokens are staged in shared memory, where a warp per token makes them ready.
//
// head_gated_rmsnorm: y = o / rms(o) * w * sigmoid(gate) per token and head over vdim, w [vdim]
// shared by the heads.
#include "common.cuh"

#include <type_traits>

namespace {

constexpr int DR_TOK = 16;       // tokens staged at a time

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

constexpr int DR_SPLIT = 4, DR_COLS = 32;       // a column of S is shared by 4 lanes; a block holds 32 columns

// Lane r of a column's four holds the rows i = 16 jj + 4 r + e (e < 4): its q, k and g come as one 16-byte read per jj
// from shared memory, the four lanes' reads side by side.  Staged rows are MAXD long, zero past dim, so that the inner
// loops have no bounds to check (rows of S past dim stay zero).
template <typename T, int MAXD>
__global__ void __launch_bounds__(DR_SPLIT * DR_COLS)
delta_rule_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                       long long q_stride, long long k_stride, long long v_stride,
                       const float* __restrict__ decay_logit, const float* __restrict__ dt_bias,
                       const float* __restrict__ rate, const T* __restrict__ beta_logit, long long beta_stride,
                       float* __restrict__ o, float* __restrict__ state, long long slot_stride,
                       const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                       int n_heads, int qk_heads, int dim, int vdim, int groups) {
    ti_pdl_trigger();
    extern __shared__ __align__(16) float sm[];        // q, k, g: [DR_TOK][MAXD] each; v: [DR_TOK][DR_COLS]; beta: [DR_TOK]
    ti_pdl_sync();
    q = ti_dependent(q); k = ti_dependent(k); v = ti_dependent(v);
    decay_logit = ti_dependent(decay_logit); beta_logit = ti_dependent(beta_logit);
    constexpr int J = MAXD / 16;
    float* qs = sm;
    float* ks = qs + DR_TOK * MAXD;
    float* gs = ks + DR_TOK * MAXD;
    float* vs = gs + DR_TOK * MAXD;
    float* bs = vs + DR_TOK * DR_COLS;
    const int h = blockIdx.x / groups, g = blockIdx.x - h * groups;
    const int b = blockIdx.y;
    const int tok0 = cu_new[b], n = cu_new[b + 1] - tok0;
    if (n <= 0) return;
    const int hq = h / (n_heads / qk_heads);
    const int r = threadIdx.x & (DR_SPLIT - 1);
    const int col = g * DR_COLS + (threadIdx.x >> 2);
    const bool live = col < vdim;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const float rt = rate[h], q_scale = rsqrtf((float)dim);
    float S[J][4];
    float* srow = state + (size_t)seq_slot[b] * slot_stride + (size_t)h * dim * vdim;
#pragma unroll
    for (int jj = 0; jj < J; jj++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int i = 16 * jj + 4 * r + e;
            S[jj][e] = (live && i < dim) ? srow[(size_t)i * vdim + col] : 0.f;
        }
    // A run's operands are fetched into registers while the run before it is worked off: a warp brings TPW tokens'
    // q, k and decay logits (EPL elements a lane each), a thread VPT of the run's values.
    constexpr int TPW = DR_TOK / DR_SPLIT, EPL = MAXD / 32, VPT = DR_TOK * DR_COLS / (DR_SPLIT * DR_COLS);
    float rq[TPW][EPL], rk[TPW][EPL], rl[TPW][EPL], rb[TPW], rv[VPT], dtb[EPL];
#pragma unroll
    for (int e = 0; e < EPL; e++) dtb[e] = lane + 32 * e < dim ? dt_bias[(size_t)h * dim + lane + 32 * e] : 0.f;
    auto fetch = [&](int t0) {
        const int nt = min(DR_TOK, n - t0);
#pragma unroll
        for (int j = 0; j < TPW; j++) {
            const int tt = warp + n_warps * j;
            const size_t tok = (size_t)(tok0 + t0 + min(tt, nt - 1));
#pragma unroll
            for (int e = 0; e < EPL; e++) {
                const int i = lane + 32 * e;
                const bool ok = i < dim && tt < nt;
                rq[j][e] = ok ? to_f32(q[tok * q_stride + (size_t)hq * dim + i]) : 0.f;
                rk[j][e] = ok ? to_f32(k[tok * k_stride + (size_t)hq * dim + i]) : 0.f;
                rl[j][e] = ok ? decay_logit[tok * ((size_t)n_heads * dim) + (size_t)h * dim + i] : 0.f;
            }
            rb[j] = to_f32(beta_logit[tok * beta_stride + h]);
        }
#pragma unroll
        for (int m = 0; m < VPT; m++) {
            const int idx = threadIdx.x + DR_SPLIT * DR_COLS * m, tt = idx / DR_COLS, c = g * DR_COLS + (idx - tt * DR_COLS);
            rv[m] = (tt < nt && c < vdim) ? to_f32(v[(size_t)(tok0 + t0 + tt) * v_stride + (size_t)h * vdim + c]) : 0.f;
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < n; t0 += DR_TOK) {
        const int nt = min(DR_TOK, n - t0);
        __syncthreads();             // the run before is worked off
#pragma unroll
        for (int j = 0; j < TPW; j++) {
            const int tt = warp + n_warps * j;
            float sq = 0.f, sk = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; e++) { sq = fmaf(rq[j][e], rq[j][e], sq); sk = fmaf(rk[j][e], rk[j][e], sk); }
            sq = warp_sum(sq);
            sk = warp_sum(sk);
            const float iq = rsqrtf(sq + 1e-6f) * q_scale, ik = rsqrtf(sk + 1e-6f);
            if (tt < nt) {
#pragma unroll
                for (int e = 0; e < EPL; e++) {
                    const int i = lane + 32 * e;
                    qs[tt * MAXD + i] = rq[j][e] * iq;
                    ks[tt * MAXD + i] = rk[j][e] * ik;
                    gs[tt * MAXD + i] = i < dim ? expf(-rt * softplus_f(rl[j][e] + dtb[e])) : 0.f;
                }
                if (lane == 0) bs[tt] = 1.0f / (1.0f + expf(-rb[j]));
            }
        }
#pragma unroll
        for (int m = 0; m < VPT; m++) vs[threadIdx.x + DR_SPLIT * DR_COLS * m] = rv[m];
        __syncthreads();
        if (t0 + DR_TOK < n) fetch(t0 + DR_TOK);          // on its way while this run is worked off
        for (int tt = 0; tt < nt; tt++) {            // (all lanes take part in the sums over a column's four lanes)
            const float4* k4 = reinterpret_cast<const float4*>(ks + tt * MAXD) + r;
            const float4* q4 = reinterpret_cast<const float4*>(qs + tt * MAXD) + r;
            const float4* g4 = reinterpret_cast<const float4*>(gs + tt * MAXD) + r;
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
            float4 kk[J];
#pragma unroll
            for (int jj = 0; jj < J; jj++) {
                const float4 gg = g4[4 * jj];
                kk[jj] = k4[4 * jj];
                S[jj][0] *= gg.x; S[jj][1] *= gg.y; S[jj][2] *= gg.z; S[jj][3] *= gg.w;
                d0 = fmaf(S[jj][0], kk[jj].x, d0); d1 = fmaf(S[jj][1], kk[jj].y, d1);
                d2 = fmaf(S[jj][2], kk[jj].z, d2); d3 = fmaf(S[jj][3], kk[jj].w, d3);
            }
            float dot = (d0 + d1) + (d2 + d3);
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            const float e = bs[tt] * (vs[tt * DR_COLS + (threadIdx.x >> 2)] - dot);
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int jj = 0; jj < J; jj++) {
                const float4 qq = q4[4 * jj];
                S[jj][0] = fmaf(kk[jj].x, e, S[jj][0]); S[jj][1] = fmaf(kk[jj].y, e, S[jj][1]);
                S[jj][2] = fmaf(kk[jj].z, e, S[jj][2]); S[jj][3] = fmaf(kk[jj].w, e, S[jj][3]);
                a0 = fmaf(S[jj][0], qq.x, a0); a1 = fmaf(S[jj][1], qq.y, a1);
                a2 = fmaf(S[jj][2], qq.z, a2); a3 = fmaf(S[jj][3], qq.w, a3);
            }
            float acc = (a0 + a1) + (a2 + a3);
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (live && r == 0) o[(size_t)(tok0 + t0 + tt) * ((size_t)n_heads * vdim) + (size_t)h * vdim + col] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int jj = 0; jj < J; jj++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = 16 * jj + 4 * r + e;
                if (i < dim) srow[(size_t)i * vdim + col] = S[jj][e];
            }
    }
}

// one warp per (token, head)
template <typename T>
__global__ void head_gated_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long gate_stride,
                                          const float* __restrict__ w, T* __restrict__ out, long long rows, int n_heads, int vdim,
                                          float eps) {
    ti_pdl_trigger();
    ti_pdl_sync();
    o = ti_dependent(o); gate = ti_dependent(gate);
    const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const long long m = r / n_heads;
    const int h = (int)(r - m * n_heads);
    const float* orow = o + (size_t)r * vdim;
    float ss = 0.f;
    for (int i = lane; i < vdim; i += 32) ss = fmaf(orow[i], orow[i], ss);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)vdim + eps);
    for (int i = lane; i < vdim; i += 32) {
        const float gl = to_f32(gate[(size_t)m * gate_stride + (size_t)h * vdim + i]);
        out[(size_t)r * vdim + i] = from_f32<T>(orow[i] * inv * w[i] / (1.0f + expf(-gl)));
    }
}

template <typename F>
int dispatch_dim(int dim, F&& f) {
    if (dim <= 32) return f(std::integral_constant<int, 32>());
    if (dim <= 64) return f(std::integral_constant<int, 64>());
    return f(std::integral_constant<int, 128>());
}

}  // namespace

// q, k: [M, qk_heads, dim] and v: [M, heads, vdim] of the engine's type (row strides given, heads dense); decay_logit:
// float32 [M, heads * dim]; dt_bias: float32 [heads * dim]; rate: float32 [heads]; beta_logit: [M, heads] (row stride
// given); o: float32 [M, heads * vdim]; state: float32, slot s at state + s * slot_stride holds [heads, dim, vdim].
extern "C" int ti_delta_rule_scan(const void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                  long long v_stride, const float* decay_logit, const float* dt_bias, const float* rate,
                                  const void* beta_logit, long long beta_stride, float* o, float* state, long long slot_stride,
                                  const int* cu_new, const int* seq_slot, int n_seq, int n_heads, int qk_heads, int dim,
                                  int vdim, int dtype, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_seq <= 65535 && n_heads > 0 && qk_heads > 0 && n_heads % qk_heads == 0 && dim > 0 && vdim > 0,
               "delta_rule_scan: bad sizes");
    TI_REQUIRE(dim <= 128, "delta_rule: heads of %d query/key elements are not supported (up to 128)", dim);
    const int threads = DR_SPLIT * DR_COLS, groups = (vdim + DR_COLS - 1) / DR_COLS;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        return dispatch_dim(dim, [&](auto md) -> int {
            constexpr int MAXD = decltype(md)::value;
            constexpr size_t smem = (size_t)(3 * DR_TOK * MAXD + DR_TOK + DR_TOK * DR_COLS) * sizeof(float);
            TI_CUDA(ti_launch(delta_rule_scan_kernel<T, MAXD>, dim3(n_heads * groups, n_seq), dim3(threads), smem, stream,
                              (const T*)q, (const T*)k, (const T*)v, q_stride, k_stride, v_stride, decay_logit, dt_bias, rate,
                              (const T*)beta_logit, beta_stride, o, state, slot_stride, cu_new, seq_slot, n_heads, qk_heads, dim,
                              vdim, groups));
            TI_CHECK_LAUNCH("delta_rule_scan");
            return 0;
        });
    });
}

// o: float32 [M, heads * vdim]; gate: [M, heads * vdim] of the engine's type with row stride gate_stride; w: float32 [vdim];
// out: [M, heads * vdim] dense.
extern "C" int ti_head_gated_rmsnorm(const float* o, const void* gate, long long gate_stride, const float* w, void* out, int M,
                                     int n_heads, int vdim, float eps, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_heads > 0 && vdim > 0, "head_gated_rmsnorm: bad sizes");
    const long long rows = (long long)M * n_heads;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<1>(head_gated_rmsnorm_kernel<T>, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, stream, o, (const T*)gate,
                                   gate_stride, w, (T*)out, rows, n_heads, vdim, eps));
        TI_CHECK_LAUNCH("head_gated_rmsnorm");
        return 0;
    });
}
