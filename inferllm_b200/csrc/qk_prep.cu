// What happens to the packed projection [T, ld] (float32, or the activation dtype) of an attention layer between the matrix
// product and the attention kernel, for mixers that do more there than rotate (rope_kv.cu):
//
//   q = x[q_off : q_off + nh d] + bq;   k = x[k_off : ...] + bk;   v = x[v_off : ...] + bv     (biases optional)
//   q = q / sqrt(mean(q^2) + eps) * wq,  the mean over the WHOLE projection of the token, all heads
//       together; likewise k with wk                                                            (optional)
//   the first `rot` channels of every q and k head are rotated by the token's position, either in the
//       interleaved layout (channel 2j with 2j + 1) or the rotate-half one (j with j + rot / 2), with
//       (cos, sin) from a float32 table [positions, rot / 2, 2] that may carry a magnitude factor
//   q goes to q_out [T, nh d] in the activation dtype; k and v go into the token's place in the pages
//       (k: [pages, nkv, page_size, d], v: [pages, nkv, page_size, dv]) if there are pages to write.
//
// A layer that attends to another layer's keys and values passes k_off < 0: only q is made.  A layer whose keys are
// also its values passes v_off < 0: k alone is stored.
// Everything is float32 until the stores.  One block per token; the sums have a fixed order.
#include "common.cuh"

struct QkPrepArgs {
    const void* x;
    int ld, q_off, k_off, v_off;
    int nh, nkv, d, dv;
    const float *bq, *bk, *bv, *wq, *wk;
    float eps;
    const float* cos_sin;
    int rot, pairs, n_pos;
    const int *token_pos, *token_seq, *block_table;
    int max_pages, page_size;
    void *q_out, *kc, *vc;
    int* err;
    float qt_coef;      // query temperature: q *= 1 + qt_coef * ln((p + 1) / qt_every + 1), the division whole-numbered
    int qt_every;       // 0: none
};

__device__ __forceinline__ float rotated(const float* buf, int e, int rot, int pairs, const float* cs) {
    // buf: one head; e < rot: the channel asked for
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
    const float a = buf[e], b = buf[partner];
    return first ? a * c - b * s : a * c + b * s;
}

template <typename TI, typename TA>
__global__ void __launch_bounds__(256) qk_prep_kernel(QkPrepArgs a) {
    pdl_grid_sync();
    extern __shared__ float buf[];      // [nh d] q, then [nkv d] k
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int nq = a.nh * a.d, nk = a.k_off >= 0 ? a.nkv * a.d : 0;
    const TI* x = (const TI*)a.x + (size_t)t * a.ld;
    int p = a.token_pos[t];
    if (a.rot && (p < 0 || p >= a.n_pos)) {
        if (threadIdx.x == 0) atomicExch(a.err, 3);
        p = 0;
    }
    float ssq = 0.f, ssk = 0.f;
    const float q_temp = a.qt_every > 0 ? 1.0f + a.qt_coef * logf((float)((a.token_pos[t] + 1) / a.qt_every + 1)) : 1.0f;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) {
        float v = to_f32(x[a.q_off + c]);
        if (a.bq) v += a.bq[c];
        if (a.qt_every > 0) v *= q_temp;
        buf[c] = v;
        ssq += v * v;
    }
    for (int c = threadIdx.x; c < nk; c += blockDim.x) {
        float v = to_f32(x[a.k_off + c]);
        if (a.bk) v += a.bk[c];
        buf[nq + c] = v;
        ssk += v * v;
    }
    if (a.wq) {
        ssq = block_sum(ssq, scratch);
        const float inv = 1.0f / sqrtf(ssq / (float)nq + a.eps);
        for (int c = threadIdx.x; c < nq; c += blockDim.x) buf[c] = (buf[c] * inv) * a.wq[c];
    }
    if (a.wk && nk) {
        ssk = block_sum(ssk, scratch);
        const float inv = 1.0f / sqrtf(ssk / (float)nk + a.eps);
        for (int c = threadIdx.x; c < nk; c += blockDim.x) buf[nq + c] = (buf[nq + c] * inv) * a.wk[c];
    }
    __syncthreads();
    const float* cs = a.rot ? a.cos_sin + (size_t)p * a.rot : nullptr;      // rot / 2 pairs of (cos, sin)
    TA* qo = (TA*)a.q_out + (size_t)t * nq;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) {
        const int e = c % a.d;
        qo[c] = from_f32<TA>(e < a.rot ? rotated(buf + (c - e), e, a.rot, a.pairs, cs) : buf[c]);
    }
    if (nk == 0 || a.kc == nullptr) return;
    const int pos = a.token_pos[t];
    const int page = a.block_table[(size_t)a.token_seq[t] * a.max_pages + pos / a.page_size];
    if (page < 0) {
        if (threadIdx.x == 0) atomicExch(a.err, 2);
        return;
    }
    const int slot = pos % a.page_size;
    for (int c = threadIdx.x; c < nk; c += blockDim.x) {
        const int hk = c / a.d, e = c - hk * a.d;
        const float v = e < a.rot ? rotated(buf + nq + (c - e), e, a.rot, a.pairs, cs) : buf[nq + c];
        ((TA*)a.kc)[(((size_t)page * a.nkv + hk) * a.page_size + slot) * a.d + e] = from_f32<TA>(v);
    }
    if (a.v_off < 0) return;        // the keys are also the values: nothing else to store
    const int nv = a.nkv * a.dv;
    for (int c = threadIdx.x; c < nv; c += blockDim.x) {
        const int hk = c / a.dv, e = c - hk * a.dv;
        float v = to_f32(x[a.v_off + c]);
        if (a.bv) v += a.bv[c];
        ((TA*)a.vc)[(((size_t)page * a.nkv + hk) * a.page_size + slot) * a.dv + e] = from_f32<TA>(v);
    }
}

// the same with a temperature on the queries that grows with the position (qt_every 0: none), applied behind the bias
extern "C" int illm_qk_prep_ex(const void* x, int x_dtype, int ld, int q_off, int k_off, int v_off, int nh, int nkv, int d, int dv, const float* bq,
                               const float* bk, const float* bv, const float* wq, const float* wk, float eps, const float* cos_sin, int rot,
                               int pairs, int n_pos, const int* token_pos, const int* token_seq, const int* block_table, int max_pages,
                               int page_size, void* q_out, void* kc, void* vc, int act_dtype, int T, int* err, float qt_coef, int qt_every,
                               void* stream);
extern "C" int illm_qk_prep(const void* x, int x_dtype, int ld, int q_off, int k_off, int v_off, int nh, int nkv, int d, int dv, const float* bq,
                            const float* bk, const float* bv, const float* wq, const float* wk, float eps, const float* cos_sin, int rot,
                            int pairs, int n_pos, const int* token_pos, const int* token_seq, const int* block_table, int max_pages,
                            int page_size, void* q_out, void* kc, void* vc, int act_dtype, int T, int* err, void* stream) {
    return illm_qk_prep_ex(x, x_dtype, ld, q_off, k_off, v_off, nh, nkv, d, dv, bq, bk, bv, wq, wk, eps, cos_sin, rot, pairs, n_pos, token_pos, token_seq,
                           block_table, max_pages, page_size, q_out, kc, vc, act_dtype, T, err, 0.f, 0, stream);
}
extern "C" int illm_qk_prep_ex(const void* x, int x_dtype, int ld, int q_off, int k_off, int v_off, int nh, int nkv, int d, int dv, const float* bq,
                               const float* bk, const float* bv, const float* wq, const float* wk, float eps, const float* cos_sin, int rot,
                               int pairs, int n_pos, const int* token_pos, const int* token_seq, const int* block_table, int max_pages,
                               int page_size, void* q_out, void* kc, void* vc, int act_dtype, int T, int* err, float qt_coef, int qt_every,
                               void* stream) {
    if (T <= 0) return 0;
    if (qt_every < 0) return ILLM_ERR_BAD_ARG;
    if (nh <= 0 || d <= 0 || rot < 0 || rot > d || (rot & 1) || (rot && !cos_sin) || !x || !q_out) return ILLM_ERR_BAD_ARG;
    if (k_off >= 0 && (nkv <= 0 || dv <= 0)) return ILLM_ERR_BAD_ARG;      // v_off < 0 with k_off >= 0: keys alone are stored
    QkPrepArgs a{x, ld, q_off, k_off, v_off, nh, nkv, d, dv, bq, bk, bv, wq, wk, eps, cos_sin, rot, pairs, n_pos,
                 token_pos, token_seq, block_table, max_pages, page_size, q_out, kc, vc, err, qt_coef, qt_every};
    const size_t smem = (size_t)(nh * d + (k_off >= 0 ? nkv * d : 0)) * sizeof(float);
    if (smem > 200 * 1024) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
#define ILLM_QKP(TI, TA)                                                                                                    \
    do {                                                                                                                    \
        if (smem > 48 * 1024) cudaFuncSetAttribute(qk_prep_kernel<TI, TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        illm_launch(qk_prep_kernel<TI, TA>, dim3(T), dim3(256), smem, s, a);                                                \
    } while (0)
    if (x_dtype == ILLM_F32 && act_dtype == ILLM_BF16) ILLM_QKP(float, bf16);
    else if (x_dtype == ILLM_F32 && act_dtype == ILLM_F32) ILLM_QKP(float, float);
    else if (x_dtype == ILLM_BF16 && act_dtype == ILLM_BF16) ILLM_QKP(bf16, bf16);
    else return ILLM_ERR_BAD_ARG;
#undef ILLM_QKP
    return illm_launch_status();
}
