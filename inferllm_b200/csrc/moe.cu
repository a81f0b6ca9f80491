// Routed feed-forward (mixture of experts): every token goes through its `top` experts with the largest router
// logits, weighted by the softmax over those logits alone.
//
//   moe_route_kernel   a warp per token: logits + bias (float32), `top` rounds of arg-max (the lowest index among
//                      equal values), softmax over the chosen -> expert [T, top], weight [T, top]
//   moe_layout_kernel  one block: rows per expert, their offsets, the (token, choice) pairs placed expert by expert
//                      (row_of_pair, pair_of_row), and the list of row tiles (tile -> expert, first row, rows)
//   moe_gemm_kernel    one block per (row tile, 64 columns): rows of one expert against that expert's matrix; GATED:
//                      the matrix's rows 2i, 2i + 1 are gate and up of output i (packed so at load), x is gathered by
//                      token and hid = act(gate) * up; else the down product into float32 rows.  One chain of fused multiply-adds over the inner index per
//                      output, so a row's bits depend neither on its place among the rows nor on the step.
//   moe_combine_kernel out[t] = sum over the choices, in their order, of weight * row
//
// Which row a pair gets within its expert is decided by atomics in shared memory and may differ from run to run;
// no result depends on it.
#include "common.cuh"

__global__ void moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int top,
                                 int* __restrict__ expert, float* __restrict__ weight) {
    pdl_grid_sync();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    const float* z = logits + (size_t)t * E;
    float best0 = 0.f, sum = 0.f;
    for (int k = 0; k < top; k++) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            bool taken = false;
            for (int j = 0; j < k; j++) taken |= expert[(size_t)t * top + j] == e;
            if (taken) continue;
            const float v = z[e] + (bias ? bias[e] : 0.f);
            if (v > bv) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (k == 0) best0 = bv;
        const float w = expf(bv - best0);
        sum += w;
        if (lane == 0) {
            expert[(size_t)t * top + k] = bi;
            weight[(size_t)t * top + k] = w;
        }
        __syncwarp();
    }
    if (lane < top) weight[(size_t)t * top + lane] /= sum;
    for (int k = lane + 32; k < top; k += 32) weight[(size_t)t * top + k] /= sum;
}

// Routing by scores over ALL experts: s = softmax(z), or with `sigmoid` s_e = 1 / (1 + exp(-z_e)); the choice looks at
// s + choice_bias (the bias never enters the weights), optionally confined to the `keep` best of `groups` equal groups
// of neighbouring experts (a group's score is the sum of its `group_top` largest choice scores, 1: the largest;
// experts of other groups cannot be chosen, whatever their score); the weights are the chosen experts' s, divided by
// their sum (+ sum_eps) only if `renorm`, then times weight_scale.  Among equal scores the lowest index wins.  A warp
// per token; up to 32 groups, group_top up to 4.
__global__ void moe_route_scored_kernel(const float* __restrict__ logits, const float* __restrict__ choice_bias, int T, int E, int top, int groups,
                                        int keep, int renorm, int sigmoid, int group_top, float sum_eps, float weight_scale,
                                        int* __restrict__ expert, float* __restrict__ weight) {
    pdl_grid_sync();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    const float* z = logits + (size_t)t * E;
    float zmax = 0.f, den = 1.f;
    if (!sigmoid) {
        zmax = -INFINITY;
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
        zmax = warp_max(zmax);
        den = 0.f;
        for (int e = lane; e < E; e += 32) den += expf(z[e] - zmax);
        den = warp_sum(den);
    }
    auto score = [&](int e) { return sigmoid ? 1.0f / (1.0f + expf(-z[e])) : expf(z[e] - zmax) / den; };
    const int per = E / groups;
    unsigned kept = 0xffffffffu;       // bit g: group g may be chosen from
    if (groups > 1 && keep < groups) {
        float mine = -INFINITY;        // lane g holds group g's score
        for (int g = 0; g < groups; g++) {
            float gs = 0.f;
            int took[4] = {-1, -1, -1, -1};
            for (int r = 0; r < group_top && r < per; r++) {       // the group's r-th largest choice score
                float bv = -INFINITY;
                int bi = 0x7fffffff;
                for (int e = g * per + lane; e < (g + 1) * per; e += 32) {
                    if (e == took[0] || e == took[1] || e == took[2] || e == took[3]) continue;
                    const float v = score(e) + (choice_bias ? choice_bias[e] : 0.f);
                    if (v > bv || bi == 0x7fffffff) { bv = v; bi = e; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
                }
                took[r] = bi;
                gs = r == 0 ? bv : gs + bv;
            }
            if (lane == g) mine = gs;
        }
        kept = 0;
        for (int k = 0; k < keep; k++) {
            float bv = (lane < groups && !((kept >> lane) & 1)) ? mine : -INFINITY;
            int bi = (lane < groups && !((kept >> lane) & 1)) ? lane : 0x7fffffff;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            kept |= 1u << bi;
        }
    }
    float sum = 0.f;
    for (int k = 0; k < top; k++) {
        float bv = -INFINITY, bs = 0.f;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            if (!((kept >> (e / per)) & 1)) continue;
            bool taken = false;
            for (int j = 0; j < k; j++) taken |= expert[(size_t)t * top + j] == e;
            if (taken) continue;
            const float sc = score(e);
            const float v = sc + (choice_bias ? choice_bias[e] : 0.f);
            if (v > bv || bi == 0x7fffffff) { bv = v; bi = e; bs = sc; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o), os = __shfl_xor_sync(0xffffffffu, bs, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; bs = os; }
        }
        sum += bs;
        if (lane == 0) {
            expert[(size_t)t * top + k] = bi;
            weight[(size_t)t * top + k] = bs;
        }
        __syncwarp();
    }
    if (renorm || weight_scale != 1.f)
        for (int k = lane; k < top; k += 32) {
            float w = weight[(size_t)t * top + k];
            if (renorm) w /= sum + sum_eps;
            weight[(size_t)t * top + k] = w * weight_scale;
        }
}

// dynamic shared memory: 3 E + 1 ints
__global__ void __launch_bounds__(1024)
moe_layout_kernel(const int* __restrict__ expert, int P, int E, int bm, int* __restrict__ row_of_pair, int* __restrict__ pair_of_row,
                  int* __restrict__ tile_expert, int* __restrict__ tile_row0, int* __restrict__ tile_rows, int max_tiles) {
    pdl_grid_sync();
    extern __shared__ int si[];
    int* count = si;
    int* offset = si + E;
    int* cursor = si + 2 * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = cursor[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < P; i += blockDim.x) atomicAdd(&count[expert[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int rows = 0, tiles = 0;
        for (int e = 0; e < E; e++) {
            offset[e] = rows;
            for (int r = 0; r < count[e]; r += bm, tiles++) {
                tile_expert[tiles] = e;
                tile_row0[tiles] = rows + r;
                tile_rows[tiles] = min(bm, count[e] - r);
            }
            rows += count[e];
        }
        for (; tiles < max_tiles; tiles++) tile_rows[tiles] = 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < P; i += blockDim.x) {
        const int e = expert[i];
        const int row = offset[e] + atomicAdd(&cursor[e], 1);
        row_of_pair[i] = row;
        pair_of_row[row] = i;
    }
}

// act(gate) * up; act 4 is the clamped form g = min(gate, limit), u = clamp(up, -limit, limit): g sigmoid(1.702 g) (u + 1)
__device__ __forceinline__ float moe_gated(float v, float u, int act, float limit) {
    if (act == 1) return v / (1.0f + expf(-v)) * u;
    if (act == 2) return fmaxf(v, 0.f) * u;
    if (act == 3) return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v))) * u;
    if (act == 4) {
        const float g = fminf(v, limit), c = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-1.702f * g)) * (c + 1.0f);
    }
    return v * u;
}

#define MOE_BN 64
#define MOE_BK 16

// grid (ceil(Nw / 64), max_tiles); 256 threads = 16 x 16, a (BM / 16) x 4 patch of outputs each.  w [E, Nw, K].
// GATED: x [T, K] gathered through pair_of_row / top; the matrix's rows 2i, 2i + 1 are gate and up of output i, and
// y [P, Nw / 2] = act(gate) * up; else x [P, K] by row and y [P, Nw].
template <typename TX, typename TW, typename TY, int BM, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y, int Nw, int K, int top, int act, float act_limit,
                const int* __restrict__ pair_of_row, const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                const int* __restrict__ tile_rows) {
    pdl_grid_sync();
    constexpr int RM = BM / 16;
    __shared__ float xs[MOE_BK][BM + 4];
    __shared__ float ws[MOE_BK][MOE_BN + 4];
    __shared__ int src_row[BM];
    const int tile = blockIdx.y;
    const int rows = tile_rows[tile];
    if (rows == 0) return;
    const int e = tile_expert[tile], row0 = tile_row0[tile], n0 = blockIdx.x * MOE_BN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    for (int m = threadIdx.x; m < BM; m += 256) src_row[m] = m < rows ? (GATED ? pair_of_row[row0 + m] / top : row0 + m) : -1;
    const TW* we = w + (size_t)e * Nw * K;
    float acc[RM][4];
#pragma unroll
    for (int i = 0; i < RM; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    __syncthreads();
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
        for (int el = threadIdx.x; el < BM * MOE_BK; el += 256) {
            const int m = el / MOE_BK, k = el % MOE_BK;
            const int r = src_row[m];
            xs[k][m] = (r >= 0 && k0 + k < K) ? to_f32(x[(size_t)r * K + k0 + k]) : 0.f;
        }
        for (int el = threadIdx.x; el < MOE_BN * MOE_BK; el += 256) {
            const int n = el / MOE_BK, k = el % MOE_BK;
            ws[k][n] = (n0 + n < Nw && k0 + k < K) ? to_f32(we[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < MOE_BK; k++) {
            float a[RM], b[4];
#pragma unroll
            for (int i = 0; i < RM; i++) a[i] = xs[k][ty * RM + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < RM; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RM; i++) {
        const int m = ty * RM + i;
        if (m >= rows) continue;
        if (GATED) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int n = n0 + tx * 4 + j;
                if (n + 1 < Nw) y[(size_t)(row0 + m) * (Nw / 2) + n / 2] = from_f32<TY>(moe_gated(acc[i][j], acc[i][j + 1], act, act_limit));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int n = n0 + tx * 4 + j;
                if (n < Nw) y[(size_t)(row0 + m) * Nw + n] = from_f32<TY>(acc[i][j]);
            }
        }
    }
}

// ---- the same product on tensor cores (bfloat16, K a multiple of 8)
//
// A 64 x 128 tile per block, 8 warps of 32 x 32, K in slabs of 32 through a ring of three shared-memory stages filled
// by cp.async (rows padded to 80 bytes, so that ldmatrix reads without bank conflicts); rows of the tile beyond the
// expert's rows and columns beyond N are zero-filled on the way in and masked on the way out.  GATED: the matrix's
// rows 2i, 2i + 1 are gate and up of output i, which neighbouring accumulator columns of a thread hold.
#define MM_BM 64
#define MM_BN 128
#define MM_BK 32
#define MM_LD 40            // bf16 elements per padded row
#define MM_STAGES 3

__device__ __forceinline__ unsigned mm_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mm_cp16(unsigned dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void mm_ldsm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mm_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename TY, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_mma_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, TY* __restrict__ y, int N, int K, int top, int act, float act_limit,
                    const int* __restrict__ pair_of_row, const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                    const int* __restrict__ tile_rows) {
    pdl_grid_sync();
    extern __shared__ __align__(16) unsigned char mm_raw[];
    constexpr int NB = 1;
    constexpr int A_ELEMS = MM_BM * MM_LD, B_ELEMS = MM_BN * MM_LD, STAGE_ELEMS = A_ELEMS + NB * B_ELEMS;
    bf16* sm = reinterpret_cast<bf16*>(mm_raw);
    __shared__ int src_row[MM_BM];
    const int tile = blockIdx.y;
    const int rows = tile_rows[tile];
    if (rows == 0) return;
    const int e = tile_expert[tile], row0 = tile_row0[tile], n0 = blockIdx.x * MM_BN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, wm = warp >> 2, wn = warp & 3;
    for (int m = tid; m < MM_BM; m += 256) src_row[m] = m < rows ? (GATED ? pair_of_row[row0 + m] / top : row0 + m) : -1;
    __syncthreads();
    const bf16* wg = w + (size_t)e * N * K;
    const int KT = (K + MM_BK - 1) / MM_BK;
    // what this thread copies per slab: one 16-byte piece of A, two of each B
    const int a_r = tid >> 2, a_c = (tid & 3) * 8;
    const int a_src = src_row[a_r];
    auto load = [&](int stage, int kt) {
        bf16* base = sm + (size_t)stage * STAGE_ELEMS;
        const int k = kt * MM_BK + a_c;
        {
            const bool ok = a_src >= 0 && k < K;
            mm_cp16(mm_smem(base + a_r * MM_LD + a_c), ok ? (const void*)(x + (size_t)a_src * K + k) : (const void*)x, ok ? 16 : 0);
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int r = a_r + i * 64, n = n0 + r;
            const bool ok = n < N && k < K;
#pragma unroll
            for (int b = 0; b < NB; b++)
                mm_cp16(mm_smem(base + A_ELEMS + b * B_ELEMS + r * MM_LD + a_c), ok ? (const void*)(wg + ((size_t)b * N + n) * K + k) : (const void*)w,
                        ok ? 16 : 0);
        }
    };
    float acc[NB][2][4][4];
#pragma unroll
    for (int b = 0; b < NB; b++)
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int c = 0; c < 4; c++) acc[b][i][j][c] = 0.f;
    for (int s = 0; s < MM_STAGES - 1; s++) {
        if (s < KT) load(s, s);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    const bool busy = wm * 32 < rows;      // a warp whose 32 rows lie beyond the expert's rows only helps to copy
    for (int kt = 0; kt < KT; kt++) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(MM_STAGES - 2));
        __syncthreads();
        if (kt + MM_STAGES - 1 < KT) load((kt + MM_STAGES - 1) % MM_STAGES, kt + MM_STAGES - 1);
        asm volatile("cp.async.commit_group;\n" ::);
        if (!busy) continue;
        const bf16* base = sm + (size_t)(kt % MM_STAGES) * STAGE_ELEMS;
#pragma unroll
        for (int ks = 0; ks < MM_BK; ks += 16) {
            unsigned a[2][4];
#pragma unroll
            for (int i = 0; i < 2; i++)
                mm_ldsm4(a[i][0], a[i][1], a[i][2], a[i][3], mm_smem(base + (wm * 32 + i * 16 + (lane & 15)) * MM_LD + ks + (lane >> 4) * 8));
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const bf16* bb = base + A_ELEMS + b * B_ELEMS;
#pragma unroll
                for (int jj = 0; jj < 2; jj++) {
                    unsigned r0, r1, r2, r3;
                    mm_ldsm4(r0, r1, r2, r3, mm_smem(bb + (wn * 32 + jj * 16 + (lane & 7) + ((lane >> 4) << 3)) * MM_LD + ks + ((lane >> 3) & 1) * 8));
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        mm_mma(acc[b][i][jj * 2], a[i], r0, r1);
                        mm_mma(acc[b][i][jj * 2 + 1], a[i], r2, r3);
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    if (!busy) return;
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int c = 0; c < 4; c += GATED ? 2 : 1) {
                const int m = wm * 32 + i * 16 + (lane >> 2) + (c >> 1) * 8;
                const int n = n0 + wn * 32 + j * 8 + (lane & 3) * 2 + (c & 1);
                if (m >= rows) continue;
                if (GATED) {          // columns n, n + 1 are gate and up of output n / 2
                    if (n + 1 < N) y[(size_t)(row0 + m) * (N / 2) + n / 2] = from_f32<TY>(moe_gated(acc[0][i][j][c], acc[0][i][j][c + 1], act, act_limit));
                } else if (n < N) {
                    y[(size_t)(row0 + m) * N + n] = from_f32<TY>(acc[0][i][j][c]);
                }
            }
}

// plus: float32 [T, D] added to the experts' sum (a shared expert's output), or nullptr
__global__ void moe_combine_kernel(const float* __restrict__ rows, const int* __restrict__ row_of_pair, const float* __restrict__ weight,
                                   const float* __restrict__ plus, float* __restrict__ out, int D, int top, long long n) {
    pdl_grid_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / D;
    const int c = (int)(i - t * D);
    float acc = 0.f;
    for (int k = 0; k < top; k++) acc = fmaf(weight[t * top + k], rows[(size_t)row_of_pair[t * top + k] * D + c], acc);
    out[i] = plus ? acc + plus[i] : acc;
}

extern "C" int illm_moe_max_tiles(int T, int top, int E, int bm) { return (int)(((long long)T * top + bm - 1) / bm) + E; }
// rows per tile: the tensor-core kernel takes 64; the plain one 16 for steps of few tokens, else 64
extern "C" int illm_moe_row_tile(int T, int top, int tensor_cores) { return tensor_cores || (long long)T * top > 1024 ? 64 : 16; }

// xs[row, :] = x[pair_of_row[row] / top, :], 16 bytes at a time (K a multiple of 8): the rows in the experts' order
__global__ void moe_gather_rows_kernel(const bf16* __restrict__ x, bf16* __restrict__ xs, const int* __restrict__ pair_of_row, int K, int top) {
    pdl_grid_sync();
    const int row = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(pair_of_row[row] / top) * K);
    uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)row * K);
    for (int c = threadIdx.x; c < K / 8; c += blockDim.x) dst[c] = src[c];
}
extern "C" int illm_moe_gather_rows(const void* x, void* xs, const int* pair_of_row, int P, int K, int top, void* stream) {
    if (P <= 0) return 0;
    if (K & 7) return ILLM_ERR_BAD_ARG;
    illm_launch(moe_gather_rows_kernel, dim3(P), dim3(128), 0, (cudaStream_t)stream, (const bf16*)x, (bf16*)xs, pair_of_row, K, top);
    return illm_launch_status();
}

extern "C" int illm_moe_route_ex(const float* logits, const float* bias, int T, int E, int top, int bm, int scoring, int groups, int keep, int renorm,
                                 int* expert, float* weight, int* row_of_pair, int* pair_of_row, int* tile_expert, int* tile_row0, int* tile_rows,
                                 void* stream);
// logits [T, E] float32 (without the bias); expert, weight [T, top]; row_of_pair, pair_of_row [T * top];
// tile_* [illm_moe_max_tiles(T, top, E, bm)], bm = illm_moe_row_tile(..)
extern "C" int illm_moe_route(const float* logits, const float* bias, int T, int E, int top, int bm, int* expert, float* weight, int* row_of_pair,
                              int* pair_of_row, int* tile_expert, int* tile_row0, int* tile_rows, void* stream) {
    return illm_moe_route_ex(logits, bias, T, E, top, bm, 0, 1, 1, 1, expert, weight, row_of_pair, pair_of_row, tile_expert, tile_row0, tile_rows, stream);
}

extern "C" int illm_moe_route_ex2(const float* logits, const float* bias, int T, int E, int top, int bm, int scoring, int groups, int keep, int renorm,
                                  int group_top, float sum_eps, float weight_scale, int* expert, float* weight, int* row_of_pair, int* pair_of_row,
                                  int* tile_expert, int* tile_row0, int* tile_rows, void* stream);
extern "C" int illm_moe_route_ex(const float* logits, const float* bias, int T, int E, int top, int bm, int scoring, int groups, int keep, int renorm,
                                 int* expert, float* weight, int* row_of_pair, int* pair_of_row, int* tile_expert, int* tile_row0, int* tile_rows,
                                 void* stream) {
    return illm_moe_route_ex2(logits, bias, T, E, top, bm, scoring, groups, keep, renorm, 1, 0.f, 1.f, expert, weight, row_of_pair, pair_of_row, tile_expert,
                              tile_row0, tile_rows, stream);
}
// scoring 0: the `top` largest logits + bias, weights the softmax over the chosen; scoring 1: scores are the softmax
// over all experts, 2: the sigmoid of every logit; with 1 and 2 the bias enters the choice only, `keep` of `groups` groups
// (scored by the sum of their group_top largest) may be chosen from, weights divided by their sum + sum_eps if renorm and
// multiplied by weight_scale (moe_route_scored_kernel)
extern "C" int illm_moe_route_ex2(const float* logits, const float* bias, int T, int E, int top, int bm, int scoring, int groups, int keep, int renorm,
                                  int group_top, float sum_eps, float weight_scale, int* expert, float* weight, int* row_of_pair, int* pair_of_row,
                                  int* tile_expert, int* tile_row0, int* tile_rows, void* stream) {
    if (T <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || (bm != 16 && bm != 64 && bm != 128) || (size_t)(3 * E + 1) * sizeof(int) > 160 * 1024) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (scoring == 1 || scoring == 2) {
        if (groups < 1 || groups > 32 || E % groups || keep < 1 || keep > groups || (long long)keep * (E / groups) < top || group_top < 1 || group_top > 4)
            return ILLM_ERR_BAD_ARG;
        illm_launch(moe_route_scored_kernel, dim3((T + 3) / 4), dim3(128), 0, s, logits, bias, T, E, top, groups, keep, renorm, scoring == 2 ? 1 : 0,
                    group_top, sum_eps, weight_scale, expert, weight);
    } else if (scoring == 0) {
        illm_launch(moe_route_kernel, dim3((T + 3) / 4), dim3(128), 0, s, logits, bias, T, E, top, expert, weight);
    } else {
        return ILLM_ERR_BAD_ARG;
    }
    const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
    static bool raised = false;
    if (!raised) {
        cudaFuncSetAttribute(moe_layout_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        raised = true;
    }
    illm_launch(moe_layout_kernel, dim3(1), dim3(1024), smem, s, (const int*)expert, T * top, E, bm, row_of_pair, pair_of_row, tile_expert,
                tile_row0, tile_rows, illm_moe_max_tiles(T, top, E, bm));
    return illm_launch_status();
}

// w [E, N, K].  gated != 0: x [T, K] (x_dtype), the matrix's rows 2i, 2i + 1 gate and up of output i, y [T * top, N / 2] in
// the dtype of x; else x [T * top, K], y [T * top, N] float32.
// tensor_cores != 0 (bfloat16, K % 8 == 0, tiles of 64 rows): the mma kernel.
extern "C" int illm_moe_gemm_ex(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int T, int top, int E, int N, int K, int gated,
                                int act, float act_limit, int bm, int tensor_cores, const int* pair_of_row, const int* tile_expert,
                                const int* tile_row0, const int* tile_rows, void* stream);
extern "C" int illm_moe_gemm(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int T, int top, int E, int N, int K, int gated,
                             int act, int bm, int tensor_cores, const int* pair_of_row, const int* tile_expert, const int* tile_row0,
                             const int* tile_rows, void* stream) {
    return illm_moe_gemm_ex(x, x_dtype, w, w_dtype, y, T, top, E, N, K, gated, act, 0.f, bm, tensor_cores, pair_of_row, tile_expert, tile_row0, tile_rows,
                            stream);
}
// act_limit: the limit of the clamped activation (act 4)
extern "C" int illm_moe_gemm_ex(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int T, int top, int E, int N, int K, int gated,
                                int act, float act_limit, int bm, int tensor_cores, const int* pair_of_row, const int* tile_expert,
                                const int* tile_row0, const int* tile_rows, void* stream) {
    if (T <= 0) return 0;
    if (N <= 0 || K <= 0 || x_dtype != w_dtype || (bm != 16 && bm != 64) || (gated && (N & 1))) return ILLM_ERR_BAD_ARG;
    const int tiles = illm_moe_max_tiles(T, top, E, bm);
    if (tiles > 65535) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (tensor_cores) {
        if (x_dtype != ILLM_BF16 || (K & 7) || bm != MM_BM || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return ILLM_ERR_BAD_ARG;
        dim3 mgrid((N + MM_BN - 1) / MM_BN, tiles);
        const size_t smem = (size_t)MM_STAGES * (MM_BM + MM_BN) * MM_LD * sizeof(bf16);
        static bool raised = false;
        if (!raised) {
            cudaFuncSetAttribute(moe_gemm_mma_kernel<bf16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            cudaFuncSetAttribute(moe_gemm_mma_kernel<float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            raised = true;
        }
        if (gated)
            illm_launch(moe_gemm_mma_kernel<bf16, true>, mgrid, dim3(256), smem, s, (const bf16*)x, (const bf16*)w, (bf16*)y, N, K, top, act, act_limit,
                        pair_of_row, tile_expert, tile_row0, tile_rows);
        else
            illm_launch(moe_gemm_mma_kernel<float, false>, mgrid, dim3(256), smem, s, (const bf16*)x, (const bf16*)w, (float*)y, N, K, top, act, act_limit,
                        pair_of_row, tile_expert, tile_row0, tile_rows);
        return illm_launch_status();
    }
    dim3 grid((N + MOE_BN - 1) / MOE_BN, tiles);
#define ILLM_MOE(TX, TY, BM, G)                                                                                                       \
    illm_launch(moe_gemm_kernel<TX, TX, TY, BM, G>, grid, dim3(256), 0, s, (const TX*)x, (const TX*)w, (TY*)y, N, K, top, act, act_limit, pair_of_row, \
                tile_expert, tile_row0, tile_rows)
    if (x_dtype == ILLM_BF16) {
        if (gated) { if (bm == 16) ILLM_MOE(bf16, bf16, 16, true); else ILLM_MOE(bf16, bf16, 64, true); }
        else { if (bm == 16) ILLM_MOE(bf16, float, 16, false); else ILLM_MOE(bf16, float, 64, false); }
    } else if (x_dtype == ILLM_F32) {
        if (gated) { if (bm == 16) ILLM_MOE(float, float, 16, true); else ILLM_MOE(float, float, 64, true); }
        else { if (bm == 16) ILLM_MOE(float, float, 16, false); else ILLM_MOE(float, float, 64, false); }
    } else {
        return ILLM_ERR_BAD_ARG;
    }
#undef ILLM_MOE
    return illm_launch_status();
}

extern "C" int illm_moe_combine_plus(const float* rows, const int* row_of_pair, const float* weight, const float* plus, float* out, int T, int D,
                                     int top, void* stream) {
    if (T <= 0) return 0;
    const long long n = (long long)T * D;
    illm_launch(moe_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, rows, row_of_pair, weight, plus, out, D, top, n);
    return illm_launch_status();
}
extern "C" int illm_moe_combine(const float* rows, const int* row_of_pair, const float* weight, float* out, int T, int D, int top,
                                void* stream) {
    return illm_moe_combine_plus(rows, row_of_pair, weight, nullptr, out, T, D, top, stream);
}
