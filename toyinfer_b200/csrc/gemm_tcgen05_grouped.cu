// The tcgen05 matrix product over groups of rows that each meet a matrix of their own (the experts of a mixture):
// out[i, :] = a[i, :] W[group of i]^T.  The rows of a group stand together, every group padded to whole tiles of 128
// rows (the padding rows hold zeros), and `tile_group[t]` names the group of tile t (or -1: nothing to do).  The
// matrices are one tensor [groups * N, K]; a block's weight tile starts at row group * N + its column tile.  Otherwise
// the kernel is the one-block-per-tile product of gemm_tcgen05_tile.cu without the split contraction: TMA into an
// mbarrier ring, one elected thread issuing `tcgen05.mma`, accumulator in tensor memory, four epilogue warps.
// Which group a tile has is known only on the device, so nothing is requested before the wait for the earlier kernels.
#include "gemm_tcgen05.cuh"

namespace tigemm {
namespace {
constexpr int GBN = 128, GSTAGES = 6;

__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_grouped_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
                       GemmArgs g, const int* __restrict__ tile_group, int rows_per_group, int* status) {
    ti_pdl_trigger();
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = GBN * BK * 2;
    constexpr uint32_t TMEM_COLS = 128;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full[GSTAGES], empty[GSTAGES], acc_ready;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_gave_up;
    if (threadIdx.x == 0) s_gave_up = *reinterpret_cast<volatile int*>(status);
    __syncthreads();
    if (s_gave_up) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a0 = blockIdx.x * BM, b0 = blockIdx.y * GBN;
    if (threadIdx.x == 0) {
        for (int s = 0; s < GSTAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(&acc_ready, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        __syncwarp();
        tmem_alloc(&tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    ti_pdl_sync();
    const int group = ti_dependent(tile_group)[blockIdx.x];
    const int n_iter = group >= 0 ? (g.K + BK - 1) / BK : 0;
    const int warp_u = warp_uniform();
    if (warp_u == 0) {
        if (elect_one()) {
            const int brow = group * rows_per_group + b0;
            for (int it = 0; it < n_iter; it++) {
                const int s = it % GSTAGES;
                if (it >= GSTAGES && !mbar_wait(&empty[s], (uint32_t)(((it / GSTAGES) & 1) ^ 1))) { ti_report(status, TI_STATUS_PIPE_WAIT); break; }
                unsigned char* sa = smem + (size_t)s * (A_BYTES + B_BYTES);
                mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                tma_load_2d(sa, &a_map, it * BK, a0, &full[s]);
                tma_load_2d(sa + A_BYTES, &b_map, it * BK, brow, &full[s]);
            }
        }
    } else if (warp_u == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = instr_desc<GBN>();
            bool ok = true;
            for (int it = 0; it < n_iter && ok; it++) {
                const int s = it % GSTAGES;
                if (!mbar_wait(&full[s], (uint32_t)((it / GSTAGES) & 1))) { ti_report(status, TI_STATUS_TMA_WAIT); ok = false; break; }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + (size_t)s * (A_BYTES + B_BYTES));
                const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; k++)
                    tc_mma_bf16(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (it > 0 || k > 0) ? 1u : 0u);
                tc_commit(&empty[s]);
            }
            if (ok && n_iter > 0) tc_commit(&acc_ready);
        }
    } else {
        const int q = warp & 3;
        const int i = a0 + q * 32 + lane;
        bool ok = n_iter > 0;
        if (n_iter > 0) {
            if (!mbar_wait(&acc_ready, 0)) { ti_report(status, TI_STATUS_MMA_WAIT); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
        }
        const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16);
        if (ok) {
#pragma unroll 1
            for (int c = 0; c < GBN; c += 16) {
                float r[16];
                tmem_ld16(taddr + c, r);
                store_chunk(g, i, b0, c, r, lane);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}
}  // namespace
}  // namespace tigemm

// a: bfloat16 [rows, K] dense, rows a multiple of 128 (groups padded to whole tiles); W: bfloat16 [groups, N, K] dense;
// out: bfloat16 [rows, N] with row stride ld_out; tile_group: int32 [rows / 128] on the device.
extern "C" int ti_linear_grouped_tc(const void* a, const void* W, void* out, const int* tile_group, int rows, int groups, int N,
                                    int K, long long ld_out, cudaStream_t stream) {
    using namespace tigemm;
    if (rows == 0) return 0;
    TI_REQUIRE(rows > 0 && rows % BM == 0 && groups > 0 && N > 0 && K > 0, "linear_grouped: bad sizes rows=%d groups=%d N=%d K=%d", rows, groups, N, K);
    TI_REQUIRE(K % 8 == 0, "linear_grouped: rows of %d elements are not whole 16-byte pieces", K);
    CUtensorMap am, bm;
    if (int rc = ti_make_tensor_map_2d_bf16(&am, a, (uint64_t)rows, (uint64_t)K, (uint64_t)K * 2, BM, BK)) return rc;
    if (int rc = ti_make_tensor_map_2d_bf16(&bm, W, (uint64_t)groups * N, (uint64_t)K, (uint64_t)K * 2, GBN, BK)) return rc;
    GemmArgs g = {};
    g.rows_a = rows; g.rows_b = N; g.K = K; g.out = out; g.ld_out = ld_out; g.out_f32 = 0; g.transposed = 0; g.splits = 1;
    constexpr size_t smem = (size_t)GSTAGES * (BM * BK * 2 + GBN * BK * 2) + 1024;
    static bool configured = false;
    if (!configured) {
        TI_CUDA(cudaFuncSetAttribute(gemm_tc_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    int* status = ti_status_ptr();
    TI_REQUIRE(status != nullptr, "linear_grouped: no status word");
    dim3 grid(rows / BM, (N + GBN - 1) / GBN);
    TI_REQUIRE(grid.y <= 65535, "linear_grouped: %d weight rows are too many for one launch", N);
    TI_CUDA(ti_launch_class<5>(gemm_tc_grouped_kernel, grid, dim3(THREADS), smem, stream, am, bm, g, tile_group, N, status));
    TI_CHECK_LAUNCH("linear_grouped (tcgen05)");
    return 0;
}
