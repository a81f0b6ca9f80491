// Differential attention over the paged cache: every head has TWO score maps over the same values,
//
//     a_m = softmax_j((q_m . k_m,j) * scale) V      m = 1, 2, causal (optionally the last `window` positions)
//     o   = a_1 - lambda a_2;   o <- o / sqrt(mean(o^2) + eps) * out_scale      (the mean over the head's dv values)
//
// A query head's row holds [q_1, q_2] (2 d channels), a key head's row in the pages [k_1, k_2]; query head h reads
// key/value head h / (heads / kv heads).  Pages: k [pages, kv heads, page_size, 2 d], v [pages, kv heads, page_size, dv].
//
// attention_diff_kernel: any sizes (d, dv up to 256), float32 or bfloat16 storage, prompts and single tokens alike,
// all arithmetic in float32.  One block owns one (token, head): its sixteen warps walk the keys lo..p in blocks of 32
// (a key per lane for both scores, a channel per lane for the values, which are read once for both maps) with a running
// maximum and sum per map, and are merged in a fixed order.  The split of the keys depends only on the token's own
// position and window, so a row's bits do not depend on the step it is part of.
//
// attention_diff_mma_kernel (below): the same for prompts in bfloat16 on warp-level MMA.
#include <math.h>

#include "common.cuh"

#define AD_WARPS 16
#define AD_MAX_D 256

template <typename TA>
__global__ void __launch_bounds__(AD_WARPS * 32)
attention_diff_kernel(const TA* __restrict__ q, int q_stride, const TA* __restrict__ kc, const TA* __restrict__ vc,
                      const int* __restrict__ block_table, int max_pages, const int* __restrict__ token_pos,
                      const int* __restrict__ token_seq, TA* __restrict__ out, int nh, int nkv, int d, int dv, int page_size,
                      int window, float scale, float lambda, float eps, float out_scale) {
    pdl_grid_sync();
    extern __shared__ float smem[];
    float* qs = smem;                     // [2 d]
    float* acc_s = smem + 2 * d;          // [2][AD_WARPS][dv]
    __shared__ float m_s[2][AD_WARPS], l_s[2][AD_WARPS], scratch[32];

    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hk = h / (nh / nkv);
    const int p = token_pos[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int* bt = block_table + (size_t)token_seq[t] * max_pages;

    const TA* qrow = q + (size_t)t * q_stride + (size_t)h * 2 * d;
    for (int c = threadIdx.x; c < 2 * d; c += blockDim.x) qs[c] = to_f32(qrow[c]);
    __syncthreads();

    float m1 = -INFINITY, l1 = 0.f, m2 = -INFINITY, l2 = 0.f;
    float acc1[AD_MAX_D / 32], acc2[AD_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < AD_MAX_D / 32; i++) acc1[i] = acc2[i] = 0.f;

    const bool vec = (d & 7) == 0;
    for (int kb = lo + warp * 32; kb <= p; kb += AD_WARPS * 32) {
        const int key = kb + lane;
        const bool valid = key <= p;
        float s1 = -INFINITY, s2 = -INFINITY;
        long long off = 0;
        if (valid) {
            const int page = bt[key / page_size];
            off = ((long long)page * nkv + hk) * page_size + (key % page_size);      // in rows
            const TA* kr = kc + off * 2 * d;
            float dot1 = 0.f, dot2 = 0.f;
            if (vec) {
#pragma unroll 2
                for (int c = 0; c < d; c += 8) {
                    float f[8], g[8];
                    load8(kr + c, f);
                    load8(kr + d + c, g);
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        dot1 = fmaf(qs[c + i], f[i], dot1);
                        dot2 = fmaf(qs[d + c + i], g[i], dot2);
                    }
                }
            } else {
                for (int c = 0; c < d; c++) {
                    dot1 = fmaf(qs[c], to_f32(kr[c]), dot1);
                    dot2 = fmaf(qs[d + c], to_f32(kr[d + c]), dot2);
                }
            }
            s1 = dot1 * scale;
            s2 = dot2 * scale;
        }
        const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
        const float p1 = valid ? expf(s1 - n1) : 0.f, p2 = valid ? expf(s2 - n2) : 0.f;
        const float c1 = (m1 == -INFINITY) ? 0.f : expf(m1 - n1), c2 = (m2 == -INFINITY) ? 0.f : expf(m2 - n2);
        l1 = l1 * c1 + warp_sum(p1);
        l2 = l2 * c2 + warp_sum(p2);
#pragma unroll
        for (int i = 0; i < AD_MAX_D / 32; i++) {
            acc1[i] *= c1;
            acc2[i] *= c2;
        }
        const int nk = (p - kb + 1 < 32) ? p - kb + 1 : 32;
#pragma unroll 2
        for (int j = 0; j < nk; j++) {
            const float w1 = __shfl_sync(0xffffffffu, p1, j), w2 = __shfl_sync(0xffffffffu, p2, j);
            const long long oj = __shfl_sync(0xffffffffu, off, j);
            const TA* vr = vc + oj * dv;
#pragma unroll
            for (int i = 0; i < AD_MAX_D / 32; i++) {
                const int c = lane + 32 * i;
                if (c < dv) {
                    const float v = to_f32(vr[c]);
                    acc1[i] = fmaf(w1, v, acc1[i]);
                    acc2[i] = fmaf(w2, v, acc2[i]);
                }
            }
        }
        m1 = n1;
        m2 = n2;
    }

    if (lane == 0) {
        m_s[0][warp] = m1;
        l_s[0][warp] = l1;
        m_s[1][warp] = m2;
        l_s[1][warp] = l2;
    }
#pragma unroll
    for (int i = 0; i < AD_MAX_D / 32; i++) {
        const int c = lane + 32 * i;
        if (c < dv) {
            acc_s[(size_t)warp * dv + c] = acc1[i];
            acc_s[(size_t)(AD_WARPS + warp) * dv + c] = acc2[i];
        }
    }
    __syncthreads();
    // every thread merges the warps of both maps for its channel, in the order of the warps
    float o = 0.f;
    const int c = threadIdx.x;
    if (c < dv) {
        float a[2];
#pragma unroll
        for (int mp = 0; mp < 2; mp++) {
            float M = m_s[mp][0];
#pragma unroll
            for (int w = 1; w < AD_WARPS; w++) M = fmaxf(M, m_s[mp][w]);
            float den = 0.f, num = 0.f;
#pragma unroll
            for (int w = 0; w < AD_WARPS; w++) {
                const float wg = (m_s[mp][w] == -INFINITY) ? 0.f : expf(m_s[mp][w] - M);
                den += l_s[mp][w] * wg;
                num += acc_s[(size_t)(mp * AD_WARPS + w) * dv + c] * wg;
            }
            a[mp] = num / den;
        }
        o = a[0] - lambda * a[1];
    }
    const float ss = block_sum(o * o, scratch);
    if (c < dv) out[((size_t)t * nh + h) * dv + c] = from_f32<TA>(o * (1.0f / sqrtf(ss / (float)dv + eps)) * out_scale);
}

extern "C" int illm_attention_diff(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages,
                                   const int* token_pos, const int* token_seq, void* out, int act_dtype, int T, int nh, int nkv, int d, int dv,
                                   int page_size, int window, float scale, float lambda, float eps, float out_scale, void* stream) {
    if (T <= 0) return 0;
    if (d <= 0 || dv <= 0 || 2 * d > 2 * AD_MAX_D || d > AD_MAX_D || dv > AD_MAX_D || nkv <= 0 || nh % nkv || nh > 65535) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, nh);
    const size_t smem = ((size_t)2 * d + (size_t)2 * AD_WARPS * dv) * sizeof(float);
    if (act_dtype == ILLM_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_diff_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        illm_launch(attention_diff_kernel<bf16>, grid, dim3(AD_WARPS * 32), smem, s, (const bf16*)q, q_stride, (const bf16*)kc, (const bf16*)vc,
                    block_table, max_pages, token_pos, token_seq, (bf16*)out, nh, nkv, d, dv, page_size, window, scale, lambda, eps, out_scale);
    } else if (act_dtype == ILLM_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_diff_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        illm_launch(attention_diff_kernel<float>, grid, dim3(AD_WARPS * 32), smem, s, (const float*)q, q_stride, (const float*)kc, (const float*)vc,
                    block_table, max_pages, token_pos, token_seq, (float*)out, nh, nkv, d, dv, page_size, window, scale, lambda, eps, out_scale);
    } else {
        return ILLM_ERR_BAD_ARG;
    }
    return illm_launch_status();
}
