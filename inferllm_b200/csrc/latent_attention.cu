// Pieces of attention through low-rank latents.
//
// latent_prep_kernel: from a token's packed float32 projection [query latent (Q), key/value latent (R)]:
//     c_q = rmsnorm(x[0:Q]) * w_q   -> a [T, Q] matrix of the activation dtype (what the query up-projection reads)
//     c   = rmsnorm(x[Q:Q+R]) * w_kv -> the token's row of the cache's key pages (one head of R channels)
// Only c is cached: keys and values of every head are linear maps of it, k_h = U_k,h c and v_h = U_v,h c, so
//     score_h = q_h . (U_k,h c) = (U_k,h^T q_h) . c        and        o_h = U_v,h (sum_j p_j c_j)
// and attention runs as one shared key/value head of R channels (the cached c is key and value at once) with
// queries U_k,h^T q_h, followed by U_v,h on its output.  Those two per-head maps are head_gemm_kernel:
//     y[t, h, :] = W_h x[t, h, :]      (W stored [heads * out, in], "NT")
//     y[t, h, :] = W_h^T x[t, h, :]    (W stored [heads * in, out], "NN")
// a 64 x 64 tile per block, float32 accumulation in one chain over the inner index per output, so a row's bits
// do not depend on what else is in the step.
#include "common.cuh"

template <typename TA>
__global__ void __launch_bounds__(256)
latent_prep_kernel(const float* __restrict__ x, int ld, int Q, int R, const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                   const int* __restrict__ token_pos, const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_pages,
                   int page_size, TA* __restrict__ cq_out, TA* __restrict__ kc, int* __restrict__ err) {
    pdl_grid_sync();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const float* row = x + (size_t)t * ld;
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < Q; c += blockDim.x) sq = fmaf(row[c], row[c], sq);
    for (int c = threadIdx.x; c < R; c += blockDim.x) sk = fmaf(row[Q + c], row[Q + c], sk);
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);
    const float iq = 1.0f / sqrtf(sq / (float)Q + eps), ik = 1.0f / sqrtf(sk / (float)R + eps);
    for (int c = threadIdx.x; c < Q; c += blockDim.x) cq_out[(size_t)t * Q + c] = from_f32<TA>((row[c] * iq) * wq[c]);
    if (!kc) return;
    const int pos = token_pos[t];
    const int page = block_table[(size_t)token_seq[t] * max_pages + pos / page_size];
    if (page < 0) {
        if (threadIdx.x == 0) atomicExch(err, 2);
        return;
    }
    TA* dst = kc + ((size_t)page * page_size + pos % page_size) * R;
    for (int c = threadIdx.x; c < R; c += blockDim.x) dst[c] = from_f32<TA>((row[Q + c] * ik) * wkv[c]);
}

extern "C" int illm_latent_prep(const float* x, int ld, int Q, int R, const float* wq, const float* wkv, float eps, const int* token_pos,
                                const int* token_seq, const int* block_table, int max_pages, int page_size, void* cq_out, void* kc,
                                int act_dtype, int T, int* err, void* stream) {
    if (T <= 0) return 0;
    if (Q <= 0 || R <= 0 || !x || !cq_out || !wq || !wkv) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == ILLM_BF16)
        illm_launch(latent_prep_kernel<bf16>, dim3(T), dim3(256), 0, s, x, ld, Q, R, wq, wkv, eps, token_pos, token_seq, block_table, max_pages,
                    page_size, (bf16*)cq_out, (bf16*)kc, err);
    else if (act_dtype == ILLM_F32)
        illm_launch(latent_prep_kernel<float>, dim3(T), dim3(256), 0, s, x, ld, Q, R, wq, wkv, eps, token_pos, token_seq, block_table,
                    max_pages, page_size, (float*)cq_out, (float*)kc, err);
    else
        return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

// latent_rope_prep_kernel: the same step for a layer whose heads have, beside the d channels that go through the latent,
// dr channels that are rotated by the position and compared with ONE rotated key part shared by all heads.  From a token's
// packed float32 projection [.., q (heads x (d + dr)) at q_off, .., latent (R) and raw key part (dr) at c_off, ..]:
//     c  = rmsnorm(x[c_off : c_off + R]) * w_kv;   kr = rotate(x[c_off + R : c_off + R + dr], p)
//     the cache row of the token (one head of R + dr channels) = [c, kr]
//     q_nope[t, h, :] = q[h, 0:d]                      -> [T, heads * d] (what U_k^T reads)
//     qa[t, h, R : R + dr] = rotate(q[h, d : d + dr], p) -> the tail of the absorbed queries [T, heads * (R + dr)], whose
//                                                          first R channels per head U_k^T q fills afterwards
// so that score = qa . [c, kr].  The rotation turns the first `rot` channels of the dr (interleaved pairs or rotate-half,
// as in qk_prep.cu) by angles from a float32 (cos, sin) table; the rest pass unchanged.  Everything is float32 until the stores.
template <typename TQ, typename TA>
__global__ void __launch_bounds__(256)
latent_rope_prep_kernel(const float* __restrict__ x, int ld, int q_off, int H, int d, int dr, int c_off, int R, const float* __restrict__ wkv, float eps,
                        const float* __restrict__ cos_sin, int rot, int pairs, int n_pos, const int* __restrict__ token_pos,
                        const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_pages, int page_size,
                        TQ* __restrict__ q_nope, TA* __restrict__ qa, TA* __restrict__ kc, int* __restrict__ err) {
    pdl_grid_sync();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const float* row = x + (size_t)t * ld;
    int p = token_pos[t];
    if (rot && (p < 0 || p >= n_pos)) {
        if (threadIdx.x == 0) atomicExch(err, 3);
        p = 0;
    }
    const float* cs = rot ? cos_sin + (size_t)p * rot : nullptr;      // rot / 2 pairs of (cos, sin)
    auto turned = [&](const float* v, int e) {       // channel e of the dr-vector v after the rotation
        if (e >= rot) return v[e];
        int j, partner;
        bool first;
        if (pairs) {
            j = e >> 1;
            first = !(e & 1);
            partner = e ^ 1;
        } else {
            const int half = rot >> 1;
            first = e < half;
            j = first ? e : e - half;
            partner = first ? e + half : e - half;
        }
        const float c = cs[2 * j], s = cs[2 * j + 1];
        return first ? v[e] * c - v[partner] * s : v[e] * c + v[partner] * s;
    };
    for (int i = threadIdx.x; i < H * d; i += blockDim.x) {
        const int h = i / d, c = i - h * d;
        q_nope[(size_t)t * H * d + i] = from_f32<TQ>(row[q_off + h * (d + dr) + c]);
    }
    for (int i = threadIdx.x; i < H * dr; i += blockDim.x) {
        const int h = i / dr, e = i - h * dr;
        qa[((size_t)t * H + h) * (R + dr) + R + e] = from_f32<TA>(turned(row + q_off + h * (d + dr) + d, e));
    }
    if (!kc) return;
    float sk = 0.f;
    for (int c = threadIdx.x; c < R; c += blockDim.x) sk = fmaf(row[c_off + c], row[c_off + c], sk);
    sk = block_sum(sk, scratch);
    const float ik = 1.0f / sqrtf(sk / (float)R + eps);
    const int pos = token_pos[t];
    const int page = block_table[(size_t)token_seq[t] * max_pages + pos / page_size];
    if (page < 0) {
        if (threadIdx.x == 0) atomicExch(err, 2);
        return;
    }
    TA* dst = kc + ((size_t)page * page_size + pos % page_size) * (R + dr);
    for (int c = threadIdx.x; c < R; c += blockDim.x) dst[c] = from_f32<TA>((row[c_off + c] * ik) * wkv[c]);
    for (int e = threadIdx.x; e < dr; e += blockDim.x) dst[R + e] = from_f32<TA>(turned(row + c_off + R, e));
}

// q_nope in float32 (q_f32 != 0) or in the activation dtype; qa and the cache row in the activation dtype.
extern "C" int illm_latent_rope_prep(const float* x, int ld, int q_off, int H, int d, int dr, int c_off, int R, const float* wkv, float eps,
                                     const float* cos_sin, int rot, int pairs, int n_pos, const int* token_pos, const int* token_seq,
                                     const int* block_table, int max_pages, int page_size, void* q_nope, int q_f32, void* qa, void* kc,
                                     int act_dtype, int T, int* err, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || d <= 0 || dr < 0 || R <= 0 || rot < 0 || rot > dr || (rot & 1) || (rot && !cos_sin) || !x || !q_nope || !qa || !wkv) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
#define ILLM_LRP(TQ, TA)                                                                                                                 \
    illm_launch(latent_rope_prep_kernel<TQ, TA>, dim3(T), dim3(256), 0, s, x, ld, q_off, H, d, dr, c_off, R, wkv, eps, cos_sin, rot, pairs, n_pos, \
                token_pos, token_seq, block_table, max_pages, page_size, (TQ*)q_nope, (TA*)qa, (TA*)kc, err)
    if (act_dtype == ILLM_BF16 && q_f32) ILLM_LRP(float, bf16);
    else if (act_dtype == ILLM_BF16) ILLM_LRP(bf16, bf16);
    else if (act_dtype == ILLM_F32) ILLM_LRP(float, float);
    else return ILLM_ERR_BAD_ARG;
#undef ILLM_LRP
    return illm_launch_status();
}

#define HG_BM 64
#define HG_BN 64
#define HG_BK 16

// grid (ceil(N / 64), ceil(T / 64), heads); 256 threads, a 4 x 4 patch of outputs each
template <typename TX, typename TW, typename TY, bool NN>
__global__ void __launch_bounds__(256)
head_gemm_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y, int T, int N, int K, int x_ld, int x_hs, int y_ld,
                 int y_hs) {
    pdl_grid_sync();
    __shared__ float xs[HG_BK][HG_BM + 4];
    __shared__ float ws[HG_BK][HG_BN + 4];
    const int h = blockIdx.z, n0 = blockIdx.x * HG_BN, t0 = blockIdx.y * HG_BM;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HG_BK) {
        for (int e = threadIdx.x; e < HG_BM * HG_BK; e += 256) {
            const int m = e / HG_BK, k = e % HG_BK;
            const int t = t0 + m;
            xs[k][m] = (t < T && k0 + k < K) ? to_f32(x[(size_t)t * x_ld + (size_t)h * x_hs + k0 + k]) : 0.f;
        }
        for (int e = threadIdx.x; e < HG_BN * HG_BK; e += 256) {
            int n, k;
            if (NN) { n = e % HG_BN; k = e / HG_BN; } else { k = e % HG_BK; n = e / HG_BK; }
            float v = 0.f;
            if (n0 + n < N && k0 + k < K)
                v = NN ? to_f32(w[((size_t)h * K + k0 + k) * N + n0 + n]) : to_f32(w[((size_t)h * N + n0 + n) * K + k0 + k]);
            ws[k][n] = v;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HG_BK; k++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < N) y[(size_t)t * y_ld + (size_t)h * y_hs + n] = from_f32<TY>(acc[i][j]);
        }
    }
}

// The same maps for the few rows of a single-token step (bfloat16 matrices, at most 16 rows): a block per (head, 32
// outputs), the rows' inputs in shared memory, the matrix read once, 16 bytes per thread where its rows are contiguous
// in the inner index.  NN: 8 slices of the inner index per output, added in order through shared memory; NT: 8 lanes per
// output, added by shuffles.
#define HV_ROWS 16

template <typename TX, typename TY>
__global__ void __launch_bounds__(256)
head_gemv_nn_kernel(const TX* __restrict__ x, const bf16* __restrict__ w, TY* __restrict__ y, int T, int N, int K, int x_ld, int x_hs, int y_ld,
                    int y_hs) {
    pdl_grid_sync();
    extern __shared__ float hv_sm[];               // x [T, K], then the partial sums [8, T, 32]
    const int h = blockIdx.y, n = blockIdx.x * 32 + (threadIdx.x & 31), ks = threadIdx.x >> 5;
    float* xs = hv_sm;
    float* red = hv_sm + T * K;
    for (int e = threadIdx.x; e < T * K; e += 256) xs[e] = to_f32(x[(size_t)(e / K) * x_ld + (size_t)h * x_hs + e % K]);
    __syncthreads();
    float acc[HV_ROWS];
#pragma unroll
    for (int t = 0; t < HV_ROWS; t++) acc[t] = 0.f;
    if (n < N) {
        const bf16* wp = w + (size_t)h * K * N + n;
#pragma unroll 4
        for (int k = ks; k < K; k += 8) {
            const float wv = to_f32(wp[(size_t)k * N]);
#pragma unroll
            for (int t = 0; t < HV_ROWS; t++)
                if (t < T) acc[t] = fmaf(xs[t * K + k], wv, acc[t]);
        }
    }
#pragma unroll
    for (int t = 0; t < HV_ROWS; t++)
        if (t < T) red[(ks * T + t) * 32 + (threadIdx.x & 31)] = acc[t];
    __syncthreads();
    for (int e = threadIdx.x; e < T * 32; e += 256) {
        const int t = e >> 5, nl = e & 31, nn = blockIdx.x * 32 + nl;
        if (nn >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int q = 0; q < 8; q++) v += red[(q * T + t) * 32 + nl];
        y[(size_t)t * y_ld + (size_t)h * y_hs + nn] = from_f32<TY>(v);
    }
}

template <typename TX, typename TY>
__global__ void __launch_bounds__(256)
head_gemv_nt_kernel(const TX* __restrict__ x, const bf16* __restrict__ w, TY* __restrict__ y, int T, int N, int K, int x_ld, int x_hs, int y_ld,
                    int y_hs) {
    pdl_grid_sync();
    extern __shared__ float hv_sm[];               // x [T, K]
    const int h = blockIdx.y, n = blockIdx.x * 32 + (threadIdx.x >> 3), kl = threadIdx.x & 7;
    for (int e = threadIdx.x; e < T * K; e += 256) hv_sm[e] = to_f32(x[(size_t)(e / K) * x_ld + (size_t)h * x_hs + e % K]);
    __syncthreads();
    float acc[HV_ROWS];
#pragma unroll
    for (int t = 0; t < HV_ROWS; t++) acc[t] = 0.f;
    if (n < N) {
        const bf16* wp = w + ((size_t)h * N + n) * K;
        for (int k = kl * 8; k < K; k += 64) {
            float wv[8];
            load8(wp + k, wv);
#pragma unroll
            for (int t = 0; t < HV_ROWS; t++)
                if (t < T) {
#pragma unroll
                    for (int j = 0; j < 8; j++) acc[t] = fmaf(hv_sm[t * K + k + j], wv[j], acc[t]);
                }
        }
    }
#pragma unroll
    for (int t = 0; t < HV_ROWS; t++)
        if (t < T) {
            float v = acc[t];
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            if (kl == 0 && n < N) y[(size_t)t * y_ld + (size_t)h * y_hs + n] = from_f32<TY>(v);
        }
}

// x [T, heads * K] -> y [T, heads * N]; w [heads * N, K] (nn = 0) or [heads * K, N] (nn = 1).  dtype codes for x, w, y.
extern "C" int illm_head_gemm_ex(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype, int T, int heads, int N, int K, int nn,
                                 int x_ld, int x_hs, int y_ld, int y_hs, void* stream);
extern "C" int illm_head_gemm(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype, int T, int heads, int N, int K,
                              int nn, void* stream) {
    return illm_head_gemm_ex(x, x_dtype, w, w_dtype, y, y_dtype, T, heads, N, K, nn, heads * K, K, heads * N, N, stream);
}
// The same where a head's input and output are pieces of wider rows: head h of row t reads x[t * x_ld + h * x_hs + 0..K)
// and writes y[t * y_ld + h * y_hs + 0..N) (elements).
extern "C" int illm_head_gemm_ex(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype, int T, int heads, int N, int K, int nn,
                                 int x_ld, int x_hs, int y_ld, int y_hs, void* stream) {
    if (T <= 0) return 0;
    if (heads <= 0 || heads > 65535 || N <= 0 || K <= 0 || x_hs < K || y_hs < N || x_ld < (heads - 1) * x_hs + K || y_ld < (heads - 1) * y_hs + N)
        return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t hv_smem = ((size_t)T * K + (nn ? (size_t)8 * T * 32 : 0)) * sizeof(float);
    if (T <= HV_ROWS && w_dtype == ILLM_BF16 && y_dtype == ILLM_BF16 && hv_smem <= 48 * 1024 && (nn || ((K & 7) == 0 && !((uintptr_t)w & 15)))) {
        dim3 grid((N + 31) / 32, heads);
#define ILLM_HV(TX)                                                                                                              \
    do {                                                                                                                         \
        if (nn) illm_launch(head_gemv_nn_kernel<TX, bf16>, grid, dim3(256), hv_smem, s, (const TX*)x, (const bf16*)w, (bf16*)y, T, N, K, x_ld, x_hs, y_ld, y_hs); \
        else illm_launch(head_gemv_nt_kernel<TX, bf16>, grid, dim3(256), hv_smem, s, (const TX*)x, (const bf16*)w, (bf16*)y, T, N, K, x_ld, x_hs, y_ld, y_hs);    \
    } while (0)
        if (x_dtype == ILLM_F32) ILLM_HV(float);
        else if (x_dtype == ILLM_BF16) ILLM_HV(bf16);
        else return ILLM_ERR_BAD_ARG;
#undef ILLM_HV
        return illm_launch_status();
    }
    for (int t0 = 0; t0 < T; t0 += 65535 * HG_BM) {
        const int n = min(T - t0, 65535 * HG_BM);
        dim3 grid((N + HG_BN - 1) / HG_BN, (n + HG_BM - 1) / HG_BM, heads);
        const size_t xo = (size_t)t0 * x_ld, yo = (size_t)t0 * y_ld;
#define ILLM_HG(TX, TW, TY)                                                                                                             \
    do {                                                                                                                                \
        if (nn) illm_launch(head_gemm_kernel<TX, TW, TY, true>, grid, dim3(256), 0, s, (const TX*)x + xo, (const TW*)w, (TY*)y + yo, n, N, K, x_ld, x_hs, y_ld, y_hs); \
        else illm_launch(head_gemm_kernel<TX, TW, TY, false>, grid, dim3(256), 0, s, (const TX*)x + xo, (const TW*)w, (TY*)y + yo, n, N, K, x_ld, x_hs, y_ld, y_hs); \
    } while (0)
        if (x_dtype == ILLM_F32 && w_dtype == ILLM_F32 && y_dtype == ILLM_F32) ILLM_HG(float, float, float);
        else if (x_dtype == ILLM_F32 && w_dtype == ILLM_BF16 && y_dtype == ILLM_BF16) ILLM_HG(float, bf16, bf16);
        else if (x_dtype == ILLM_BF16 && w_dtype == ILLM_BF16 && y_dtype == ILLM_BF16) ILLM_HG(bf16, bf16, bf16);
        else if (x_dtype == ILLM_BF16 && w_dtype == ILLM_BF16 && y_dtype == ILLM_F32) ILLM_HG(bf16, bf16, float);
        else return ILLM_ERR_BAD_ARG;
#undef ILLM_HG
    }
    return illm_launch_status();
}

// Attention of every token over ONE shared key/value head of any width (the cached latent is key and value): the form
// for widths that the framework's attention kernels do not take (not a multiple of 8, or beyond 256 channels).  A block
// per (token, head), four warps that take the visible keys in turn (key j by warp (j - lo) mod 4, which depends on the
// token's position alone), a lane holding every 32nd channel; float32 scores, an online softmax per warp, and the four
// warps merged in a fixed order.  Positions p - window + 1 .. p are visible (window 0: all up to p).
template <typename TA, int NR>
__global__ void __launch_bounds__(128)
latent_attention_any_kernel(const TA* __restrict__ q, const TA* __restrict__ kc, const int* __restrict__ block_table, int max_pages,
                            const int* __restrict__ token_pos, const int* __restrict__ token_seq, TA* __restrict__ out, int H, int R,
                            int page_size, int window, float scale, const float* __restrict__ gate, int gate_stride) {
    pdl_grid_sync();
    extern __shared__ float la_sm[];               // per warp: R partial outputs, then the warps' (max, sum)
    const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = token_pos[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int* table = block_table + (size_t)token_seq[t] * max_pages;
    float qv[NR], acc[NR];
#pragma unroll
    for (int i = 0; i < NR; i++) {
        const int r = lane + 32 * i;
        qv[i] = r < R ? to_f32(q[((size_t)t * H + h) * R + r]) * scale : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int j = lo + warp; j <= p; j += 4) {
        const int page = table[j / page_size];
        const TA* c = kc + ((size_t)page * page_size + j % page_size) * R;
        float cv[NR], dot = 0.f;
#pragma unroll
        for (int i = 0; i < NR; i++) {
            const int r = lane + 32 * i;
            cv[i] = (page >= 0 && r < R) ? to_f32(c[r]) : 0.f;
            dot = fmaf(qv[i], cv[i], dot);
        }
        dot = warp_sum(dot);
        const float m_new = fmaxf(m, dot), corr = expf(m - m_new), w = expf(dot - m_new);
        l = l * corr + w;
#pragma unroll
        for (int i = 0; i < NR; i++) acc[i] = fmaf(w, cv[i], acc[i] * corr);
        m = m_new;
    }
    float* part = la_sm + (size_t)warp * R;
    float* ml = la_sm + (size_t)4 * R;
#pragma unroll
    for (int i = 0; i < NR; i++) {
        const int r = lane + 32 * i;
        if (r < R) part[r] = acc[i];
    }
    if (lane == 0) {
        ml[2 * warp] = m;
        ml[2 * warp + 1] = l;
    }
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < 4; w++) M = fmaxf(M, ml[2 * w]);
    float f[4], L = 0.f;
    for (int w = 0; w < 4; w++) {
        f[w] = ml[2 * w + 1] > 0.f ? expf(ml[2 * w] - M) : 0.f;
        L += ml[2 * w + 1] * f[w];
    }
    if (gate) L *= 1.0f + expf(-gate[(size_t)t * gate_stride + h]);       // the head's output times sigmoid(gate)
    for (int r = threadIdx.x; r < R; r += 128) {
        float v = 0.f;
        for (int w = 0; w < 4; w++) v = fmaf(la_sm[(size_t)w * R + r], f[w], v);
        out[((size_t)t * H + h) * R + r] = from_f32<TA>(v / L);
    }
}

extern "C" int illm_latent_attention_any_gated(const void* q, const void* kc, const int* block_table, int max_pages, const int* token_pos,
                                               const int* token_seq, void* out, int act_dtype, int T, int H, int R, int page_size, int window,
                                               float scale, const float* gate, int gate_stride, void* stream);
extern "C" int illm_latent_attention_any(const void* q, const void* kc, const int* block_table, int max_pages, const int* token_pos,
                                         const int* token_seq, void* out, int act_dtype, int T, int H, int R, int page_size, int window,
                                         float scale, void* stream) {
    return illm_latent_attention_any_gated(q, kc, block_table, max_pages, token_pos, token_seq, out, act_dtype, T, H, R, page_size, window, scale, nullptr, 0,
                                           stream);
}
// gate: float32 [T, gate_stride] or nullptr; head h of token t is multiplied by sigmoid(gate[t * gate_stride + h])
extern "C" int illm_latent_attention_any_gated(const void* q, const void* kc, const int* block_table, int max_pages, const int* token_pos,
                                               const int* token_seq, void* out, int act_dtype, int T, int H, int R, int page_size, int window,
                                               float scale, const float* gate, int gate_stride, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || H > 65535 || R <= 0 || R > 1024 || page_size <= 0 || window < 0) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = ((size_t)4 * R + 8) * sizeof(float);
    const int nr = (R + 31) / 32;
#define ILLM_LA(TA, NR)                                                                                                               \
    illm_launch(latent_attention_any_kernel<TA, NR>, dim3(T, H), dim3(128), smem, s, (const TA*)q, (const TA*)kc, block_table, max_pages, \
                token_pos, token_seq, (TA*)out, H, R, page_size, window, scale, gate, gate_stride)
#define ILLM_LA_NR(TA)                                  \
    do {                                                \
        if (nr <= 1) ILLM_LA(TA, 1);                    \
        else if (nr <= 2) ILLM_LA(TA, 2);               \
        else if (nr <= 4) ILLM_LA(TA, 4);               \
        else if (nr <= 8) ILLM_LA(TA, 8);               \
        else if (nr <= 16) ILLM_LA(TA, 16);             \
        else ILLM_LA(TA, 32);                           \
    } while (0)
    if (act_dtype == ILLM_BF16) ILLM_LA_NR(bf16);
    else if (act_dtype == ILLM_F32) ILLM_LA_NR(float);
    else return ILLM_ERR_BAD_ARG;
#undef ILLM_LA_NR
#undef ILLM_LA
    return illm_launch_status();
}
