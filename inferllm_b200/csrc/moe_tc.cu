// The experts' products of a prompt step on the 5th-generation tensor cores: one block per (row tile of ONE expert,
// BN columns of that expert's matrix), D[128, BN] = A[128 rows, K] . B[BN rows, K]^T in tensor memory, the block of
// gemm_tc.cu (a TMA loader thread, an MMA thread, four epilogue warps, a ring of shared-memory stages, bounded waits)
// with the tile's place taken from the list that moe_layout_kernel made on the device:
//   A  the step's rows in the experts' order [P, K] (moe_gather_rows_kernel for the first product, the hidden rows for
//      the second); a tile starts at any row (TMA rows need no alignment) and holds up to 128 rows of its expert; what
//      the box reads beyond them (the next expert's rows, zeros beyond P) is computed and not stored;
//   B  the experts' matrices stacked [E * N, K]; the tile's rows start at expert * N + column offset.
// GATED: the matrix's rows 2i, 2i + 1 are gate and up of output i; a thread of the epilogue holds neighbouring
// columns and stores act(gate) * up.  The tile list is written by the kernel before this one, so every thread waits
// for it (griddepcontrol.wait) before anything else, and a block whose tile is empty leaves at once.
#include "tc_common.cuh"

#define MT_MAX_STAGES 8

// act(gate) * up; act 4: g = min(gate, limit), u = clamp(up, -limit, limit), g sigmoid(1.702 g) (u + 1)
__device__ __forceinline__ float mt_gated(float v, float u, int act, float limit) {
    if (act == 1) return v / (1.0f + __expf(-v)) * u;
    if (act == 2) return fmaxf(v, 0.f) * u;
    if (act == 3) return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v))) * u;
    if (act == 4) {
        const float g = fminf(v, limit), c = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + __expf(-1.702f * g)) * (c + 1.0f);
    }
    return v * u;
}

template <int BN, typename TOut, bool GATED>
__global__ void __launch_bounds__(TC_THREADS)
moe_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TOut* __restrict__ C, int ldc,
                   int n_per_expert, int n_k, int STAGES, int act, float act_limit, const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                   const int* __restrict__ tile_rows, int* __restrict__ err) {
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(TC_BM >> 4) << 24);
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * MT_MAX_STAGES + 1];
    __shared__ unsigned tmem_holder;

    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int tile = blockIdx.x;
    const int rows = tile_rows[tile];
    if (rows <= 0 || n_k <= 0) return;                      // the same for every thread of the block
    const int ra0 = tile_row0[tile], nb0 = blockIdx.y * BN;
    const int rb0 = tile_expert[tile] * n_per_expert + nb0;

    const unsigned a_base = (tc_smem_u32(smem_raw) + 1023u) & ~1023u, b_base = a_base + STAGES * A_BYTES;
    const unsigned full0 = tc_smem_u32(&bars[0]), empty0 = tc_smem_u32(&bars[MT_MAX_STAGES]);
    const unsigned done_bar = tc_smem_u32(&bars[2 * MT_MAX_STAGES]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tc_smem_u32(&tmem_holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_holder;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            bool alive = true;
            for (int i = 0; i < n_k && alive; i++) {
                const int s = i % STAGES;
                if (i >= STAGES) alive = mbar_wait(empty0 + 8 * s, ((i / STAGES) - 1) & 1, err);
                if (!alive) break;
                mbar_expect_tx(full0 + 8 * s, A_BYTES + B_BYTES);
                tma_load_2d(a_base + s * A_BYTES, &map_a, i * TC_BK, ra0, full0 + 8 * s);
                tma_load_2d(b_base + s * B_BYTES, &map_b, i * TC_BK, rb0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool alive = true;
            for (int i = 0; i < n_k && alive; i++) {
                const int s = i % STAGES;
                alive = mbar_wait(full0 + 8 * s, (i / STAGES) & 1, err);
                if (!alive) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; kk++) {
                    const unsigned long long da = umma_desc_sw128(a_base + s * A_BYTES + kk * 32);
                    const unsigned long long db = umma_desc_sw128(b_base + s * B_BYTES + kk * 32);
                    umma_bf16(tmem, da, db, IDESC, (i > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(empty0 + 8 * s);
            }
            umma_commit(done_bar);
        }
    } else {
        const int quad = warp & 3;
        const bool ok = __all_sync(0xffffffffu, mbar_wait(done_bar, 0, err));
        tc_fence_after();
        const int m = quad * 32 + lane;
        const size_t ra = (size_t)ra0 + m;
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (nb0 + c0 >= n_per_expert) break;        // uniform over the warp
                float v[16];
                tmem_ld16(tmem + ((unsigned)(quad * 32) << 16) + (unsigned)c0, v);
                if (m >= rows) continue;
                if (GATED) {
                    TOut* dst = C + ra * ldc + (nb0 + c0) / 2;
                    float o[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) o[j] = mt_gated(v[2 * j], v[2 * j + 1], act, act_limit);
                    if (nb0 + c0 + 16 <= n_per_expert && (ldc & 7) == 0) {
                        store8(dst, o);
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            if (nb0 + c0 + 2 * j + 1 < n_per_expert) store_out<TOut>(dst + j, o[j]);
                    }
                } else {
                    TOut* dst = C + ra * ldc + nb0 + c0;
                    if (nb0 + c0 + 16 <= n_per_expert && (ldc & 7) == 0) {
                        store8(dst, v);
                        store8(dst + 8, v + 8);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (nb0 + c0 + j < n_per_expert) store_out<TOut>(dst + j, v[j]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*MtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map of a row-major bfloat16 matrix [rows, K]; boxes of [box_rows, 64], 128-byte swizzle, zeros outside.
static int mt_make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, int box_rows) {
    static MtEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (MtEncodeFn)p;
    }
    if (!fn) return ILLM_ERR_BAD_ARG;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ILLM_ERR_BAD_ARG;
}

template <int BN, typename TOut, bool GATED>
static int mt_launch(const CUtensorMap& ma, const CUtensorMap& mb, TOut* y, int ldc, int N, int k_iters, int tiles, int act, float act_limit, const int* tile_expert,
                     const int* tile_row0, const int* tile_rows, int* err, cudaStream_t s) {
    const int stage_bytes = TC_BM * TC_BK * 2 + BN * TC_BK * 2;
    // a ring that leaves room for TWO blocks on an SM (two stages of 48 KB, three of 32 KB): one block's epilogue then runs
    // under the other's products (experts of a 2,048-token prompt at width 4096: 2.79 ms against 3.03 ms with one block of
    // four stages and 3.29 ms with one of three)
    int stages = (227 * 1024 / 2 - 2560) / stage_bytes;
    if (stages > MT_MAX_STAGES) stages = MT_MAX_STAGES;
    if (stages > k_iters) stages = k_iters;
    if (stages < 2) stages = 2;
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    auto kern = moe_gemm_tc_kernel<BN, TOut, GATED>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    illm_launch(kern, dim3(tiles, (N + BN - 1) / BN), dim3(TC_THREADS), smem, s, ma, mb, y, ldc, N, k_iters, stages, act, act_limit, tile_expert, tile_row0,
                tile_rows, err);
    return illm_launch_status();
}

// xs [P, K] bfloat16: the rows in the experts' order; w [E * N, K] bfloat16; the tile list with tiles of up to 128 rows
// (`tiles` entries).  gated != 0: y [P, N / 2] bfloat16 = act(gate) * up of the matrix's row pairs; else y [P, N] float32.
extern "C" int illm_moe_gemm_tc_ex(const void* xs, const void* w, void* y, int P, int E, int N, int K, int gated, int act, float act_limit, int tiles,
                                   const int* tile_expert, const int* tile_row0, const int* tile_rows, int* err, void* stream);
extern "C" int illm_moe_gemm_tc(const void* xs, const void* w, void* y, int P, int E, int N, int K, int gated, int act, int tiles,
                                const int* tile_expert, const int* tile_row0, const int* tile_rows, int* err, void* stream) {
    return illm_moe_gemm_tc_ex(xs, w, y, P, E, N, K, gated, act, 0.f, tiles, tile_expert, tile_row0, tile_rows, err, stream);
}
// act_limit: the limit of the clamped activation (act 4)
extern "C" int illm_moe_gemm_tc_ex(const void* xs, const void* w, void* y, int P, int E, int N, int K, int gated, int act, float act_limit, int tiles,
                                   const int* tile_expert, const int* tile_row0, const int* tile_rows, int* err, void* stream) {
    if (P <= 0) return 0;
    if (N <= 0 || K <= 0 || (K & 7) || (gated && (N & 1)) || ((uintptr_t)xs & 15) || ((uintptr_t)w & 15) || tiles <= 0) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int k_iters = (K + TC_BK - 1) / TC_BK;
    const int bn = N >= 256 ? 256 : 128;
    CUtensorMap ma, mb;
    int rc;
    if ((rc = mt_make_map(&ma, xs, P, K, TC_BM)) != 0) return rc;
    if ((rc = mt_make_map(&mb, w, (long long)E * N, K, bn)) != 0) return rc;
    if (gated) {
        if (bn == 256) return mt_launch<256, bf16, true>(ma, mb, (bf16*)y, N / 2, N, k_iters, tiles, act, act_limit, tile_expert, tile_row0, tile_rows, err, s);
        return mt_launch<128, bf16, true>(ma, mb, (bf16*)y, N / 2, N, k_iters, tiles, act, act_limit, tile_expert, tile_row0, tile_rows, err, s);
    }
    if (bn == 256) return mt_launch<256, float, false>(ma, mb, (float*)y, N, N, k_iters, tiles, act, act_limit, tile_expert, tile_row0, tile_rows, err, s);
    return mt_launch<128, float, false>(ma, mb, (float*)y, N, N, k_iters, tiles, act, act_limit, tile_expert, tile_row0, tile_rows, err, s);
}
