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
// position and window, so a row's bits do not depend on the step it is part of.  For steps of few tokens over long
// sequences the keys of a (token, head) can be dealt to several blocks, whose shares a second kernel puts together
// (attention_diff_merge_kernel).
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
                      int window, float scale, float lambda, float eps, float out_scale, float* __restrict__ part) {
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
    // with several blocks per (token, head) (gridDim.z > 1) block z takes every gridDim.z-th group of sixteen key blocks
    for (int kb = lo + (blockIdx.z * AD_WARPS + warp) * 32; kb <= p; kb += gridDim.z * AD_WARPS * 32) {
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
            if (part) {       // this block's share: (maximum, sum, weighted values) per map, merged by attention_diff_merge_kernel
                float* dst = part + ((((size_t)t * nh + h) * gridDim.z + blockIdx.z) * 2 + mp) * (dv + 2);
                if (c == 0) {
                    dst[0] = M;
                    dst[1] = den;
                }
                dst[2 + c] = num;
            }
            a[mp] = num / den;
        }
        o = a[0] - lambda * a[1];
    }
    if (part) return;
    const float ss = block_sum(o * o, scratch);
    if (c < dv) out[((size_t)t * nh + h) * dv + c] = from_f32<TA>(o * (1.0f / sqrtf(ss / (float)dv + eps)) * out_scale);
}

// The shares of `splits` blocks of a (token, head) put together in the order of the blocks, then o = a_1 - lambda a_2,
// the head's unit norm and the factor.  A block per (token, head), a thread per value channel.
template <typename TA>
__global__ void __launch_bounds__(AD_MAX_D)
attention_diff_merge_kernel(const float* __restrict__ part, TA* __restrict__ out, int nh, int dv, int splits, float lambda, float eps, float out_scale) {
    pdl_grid_sync();
    __shared__ float scratch[32];
    const int t = blockIdx.x, h = blockIdx.y, c = threadIdx.x;
    const float* base = part + ((size_t)t * nh + h) * splits * 2 * (dv + 2);
    float o = 0.f;
    if (c < dv) {
        float a[2];
#pragma unroll
        for (int mp = 0; mp < 2; mp++) {
            float M = -INFINITY;
            for (int s = 0; s < splits; s++) M = fmaxf(M, base[(size_t)(s * 2 + mp) * (dv + 2)]);
            float den = 0.f, num = 0.f;
            for (int s = 0; s < splits; s++) {
                const float* ps = base + (size_t)(s * 2 + mp) * (dv + 2);
                const float wg = (ps[0] == -INFINITY) ? 0.f : expf(ps[0] - M);
                den += ps[1] * wg;
                num += ps[2 + c] * wg;
            }
            a[mp] = num / den;
        }
        o = a[0] - lambda * a[1];
    }
    const float ss = block_sum(o * o, scratch);
    if (c < dv) out[((size_t)t * nh + h) * dv + c] = from_f32<TA>(o * (1.0f / sqrtf(ss / (float)dv + eps)) * out_scale);
}

// floats of scratch that `splits` blocks per (token, head) need
extern "C" long long illm_attention_diff_scratch(int T, int nh, int dv, int splits) { return (long long)T * nh * splits * 2 * (dv + 2); }

// splits > 1: that many blocks per (token, head), each with a share of the keys, and a second kernel that puts the
// shares together; scratch: illm_attention_diff_scratch floats.
extern "C" int illm_attention_diff(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages,
                                   const int* token_pos, const int* token_seq, void* out, int act_dtype, int T, int nh, int nkv, int d, int dv,
                                   int page_size, int window, float scale, float lambda, float eps, float out_scale, int splits, float* scratch,
                                   void* stream) {
    if (T <= 0) return 0;
    if (d <= 0 || dv <= 0 || d > AD_MAX_D || dv > AD_MAX_D || nkv <= 0 || nh % nkv || nh > 65535 || splits < 1 || splits > 65535 || (splits > 1 && !scratch))
        return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, nh, splits);
    float* part = splits > 1 ? scratch : nullptr;
    const size_t smem = ((size_t)2 * d + (size_t)2 * AD_WARPS * dv) * sizeof(float);
    if (act_dtype == ILLM_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_diff_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        illm_launch(attention_diff_kernel<bf16>, grid, dim3(AD_WARPS * 32), smem, s, (const bf16*)q, q_stride, (const bf16*)kc, (const bf16*)vc,
                    block_table, max_pages, token_pos, token_seq, (bf16*)out, nh, nkv, d, dv, page_size, window, scale, lambda, eps, out_scale, part);
        if (part) illm_launch(attention_diff_merge_kernel<bf16>, dim3(T, nh), dim3(AD_MAX_D), 0, s, (const float*)part, (bf16*)out, nh, dv, splits, lambda, eps, out_scale);
    } else if (act_dtype == ILLM_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_diff_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        illm_launch(attention_diff_kernel<float>, grid, dim3(AD_WARPS * 32), smem, s, (const float*)q, q_stride, (const float*)kc, (const float*)vc,
                    block_table, max_pages, token_pos, token_seq, (float*)out, nh, nkv, d, dv, page_size, window, scale, lambda, eps, out_scale, part);
        if (part) illm_launch(attention_diff_merge_kernel<float>, dim3(T, nh), dim3(AD_MAX_D), 0, s, (const float*)part, (float*)out, nh, dv, splits, lambda, eps, out_scale);
    } else {
        return ILLM_ERR_BAD_ARG;
    }
    return illm_launch_status();
}

// ---------------------------------------------------------------------------------------------------------------------
// attention_diff_decode_kernel: single tokens in bfloat16.  A block owns (token, up to HB query heads of one key/value
// head, a share of the keys) and works through its share in rounds of 256 keys: (1) a thread per key reads the key row
// once, 16 bytes at a time, for the scores of all its heads and both maps (float32), and notes where the key's value
// row lies; (2) a warp per (head, map) takes the round's maximum, moves the running maximum and sum, and turns the
// scores into weights; (3) a thread per VEC value channels (16 or 8 bytes) and slice of the keys adds the weighted value
// rows for all heads and maps, every row read once, the loads independent of one another.  The slices are added in a fixed
// order and the block's share goes to attention_diff_merge_kernel.  Blocks whose share holds no visible key leave an
// empty share.  The grid depends on the longest sequence the cache allows, not on the step.
#define DD_THREADS 256

template <int HB, int VEC>
__global__ void __launch_bounds__(DD_THREADS)
attention_diff_decode_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                             const int* __restrict__ block_table, int max_pages, const int* __restrict__ token_pos,
                             const int* __restrict__ token_seq, float* __restrict__ part, int nh, int nkv, int d, int dv, int page_size,
                             int window, float scale, int keys_per_block) {
    pdl_grid_sync();
    extern __shared__ __align__(16) unsigned char dd_raw[];
    const int group = nh / nkv, subs = (group + HB - 1) / HB;
    const int t = blockIdx.x, hk = blockIdx.y / subs, sub = blockIdx.y - hk * subs, z = blockIdx.z, splits = gridDim.z;
    const int g0 = sub * HB, nhb = (group - g0 < HB) ? group - g0 : HB;
    const int h0 = hk * group + g0;
    const int tv = dv / VEC, KS = DD_THREADS / tv;        // threads per value row, slices of the keys
    long long* rowoff = reinterpret_cast<long long*>(dd_raw);                 // [256] row of the key in the pages
    float* qs = reinterpret_cast<float*>(rowoff + DD_THREADS);                // [HB][2 d]
    float* S = qs + HB * 2 * d;                                               // [256][HB * 2] scores, then weights (a key's rows side by side)
    float* red = S + HB * 2 * DD_THREADS;                                     // [KS][HB * 2][dv]
    __shared__ float run_m[HB * 2], run_l[HB * 2], fac[HB * 2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int p = token_pos[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    int k_begin = z * keys_per_block, k_end = k_begin + keys_per_block;      // this block's share [k_begin, k_end)
    if (k_begin < lo) k_begin = lo;
    if (k_end > p + 1) k_end = p + 1;
    const int* bt = block_table + (size_t)token_seq[t] * max_pages;
    if (k_begin >= k_end) {          // no visible key in this block's share: an empty share, at once
        for (int i = tid; i < nhb * 2 * dv; i += DD_THREADS) {
            const int row = i / dv, c = i - row * dv;
            float* dst = part + ((((size_t)t * nh + h0 + (row >> 1)) * splits + z) * 2 + (row & 1)) * (dv + 2);
            dst[2 + c] = 0.f;
            if (c == 0) {
                dst[0] = -INFINITY;
                dst[1] = 0.f;
            }
        }
        return;
    }

    for (int i = tid; i < nhb * 2 * d; i += DD_THREADS) qs[i] = to_f32(q[(size_t)t * q_stride + (size_t)h0 * 2 * d + i]);
    if (tid < HB * 2) {
        run_m[tid] = -INFINITY;
        run_l[tid] = 0.f;
    }
    const int cpair = tid % tv, ks = tid / tv;
    float acc[HB][2][VEC];
#pragma unroll
    for (int g = 0; g < HB; g++)
#pragma unroll
        for (int i = 0; i < VEC; i++) acc[g][0][i] = acc[g][1][i] = 0.f;
    __syncthreads();

    for (int r0 = k_begin; r0 < k_end; r0 += DD_THREADS) {
        const int nkeys = (k_end - r0 < DD_THREADS) ? k_end - r0 : DD_THREADS;
        // (1) scores of this thread's key
        {
            float dot[HB][2];
#pragma unroll
            for (int g = 0; g < HB; g++) dot[g][0] = dot[g][1] = 0.f;
            const bool valid = tid < nkeys;
            if (valid) {
                const int key = r0 + tid;
                const int page = bt[key / page_size];
                const long long row = ((long long)page * nkv + hk) * page_size + (key % page_size);
                rowoff[tid] = row;
                const bf16* kr = kc + row * 2 * d;
#pragma unroll 8
                for (int c = 0; c < d; c += 8) {
                    float f1[8], f2[8];
                    load8(kr + c, f1);
                    load8(kr + d + c, f2);
#pragma unroll
                    for (int g = 0; g < HB; g++) {
                        if (g < nhb) {
                            const float4* qa = reinterpret_cast<const float4*>(qs + g * 2 * d + c);        // d % 8 == 0: 16-byte reads, the same for all lanes
                            const float4* qb = reinterpret_cast<const float4*>(qs + g * 2 * d + d + c);
                            const float4 a0 = qa[0], a1 = qa[1], b0 = qb[0], b1 = qb[1];
                            dot[g][0] = fmaf(a0.x, f1[0], dot[g][0]); dot[g][0] = fmaf(a0.y, f1[1], dot[g][0]);
                            dot[g][0] = fmaf(a0.z, f1[2], dot[g][0]); dot[g][0] = fmaf(a0.w, f1[3], dot[g][0]);
                            dot[g][0] = fmaf(a1.x, f1[4], dot[g][0]); dot[g][0] = fmaf(a1.y, f1[5], dot[g][0]);
                            dot[g][0] = fmaf(a1.z, f1[6], dot[g][0]); dot[g][0] = fmaf(a1.w, f1[7], dot[g][0]);
                            dot[g][1] = fmaf(b0.x, f2[0], dot[g][1]); dot[g][1] = fmaf(b0.y, f2[1], dot[g][1]);
                            dot[g][1] = fmaf(b0.z, f2[2], dot[g][1]); dot[g][1] = fmaf(b0.w, f2[3], dot[g][1]);
                            dot[g][1] = fmaf(b1.x, f2[4], dot[g][1]); dot[g][1] = fmaf(b1.y, f2[5], dot[g][1]);
                            dot[g][1] = fmaf(b1.z, f2[6], dot[g][1]); dot[g][1] = fmaf(b1.w, f2[7], dot[g][1]);
                        }
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < HB; g++) {
                S[tid * (HB * 2) + g * 2] = valid ? dot[g][0] * scale : -INFINITY;
                S[tid * (HB * 2) + g * 2 + 1] = valid ? dot[g][1] * scale : -INFINITY;
            }
        }
        __syncthreads();
        // (2) the round's maximum, the running maximum and sum, the weights
        for (int row = warp; row < nhb * 2; row += DD_THREADS / 32) {
            float* sr = S + row;
            float mx = -INFINITY;
            for (int k = lane; k < DD_THREADS; k += 32) mx = fmaxf(mx, sr[k * (HB * 2)]);
            mx = warp_max(mx);
            const float m_old = run_m[row], m_new = fmaxf(m_old, mx);
            float sum = 0.f;
            for (int k = lane; k < DD_THREADS; k += 32) {
                const float w = (k < nkeys) ? expf(sr[k * (HB * 2)] - m_new) : 0.f;
                sr[k * (HB * 2)] = w;
                sum += w;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float f = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
                fac[row] = f;
                run_m[row] = m_new;
                run_l[row] = run_l[row] * f + sum;
            }
        }
        __syncthreads();
        // (3) weighted value rows: this thread's VEC channels, every KS-th key
        if (ks < KS) {
#pragma unroll
            for (int g = 0; g < HB; g++) {
                if (g < nhb) {
                    const float f0 = fac[g * 2], f1 = fac[g * 2 + 1];
#pragma unroll
                    for (int i = 0; i < VEC; i++) {
                        acc[g][0][i] *= f0;
                        acc[g][1][i] *= f1;
                    }
                }
            }
            // eight value rows at a time: all their loads are issued before the first is used, so that a block keeps tens of
            // kilobytes on their way (few warps run on an SM in a step of few tokens, and nothing else hides the latency)
            constexpr int KU = 8;
            for (int kb = ks; kb < nkeys; kb += KS * KU) {
                unsigned raw[KU][VEC / 2];
#pragma unroll
                for (int j = 0; j < KU; j++) {
                    const int k = kb + j * KS;
                    if (k < nkeys) {
                        const bf16* vr = vc + rowoff[k] * dv + VEC * cpair;
                        if (VEC == 8) {
                            const uint4 u = *reinterpret_cast<const uint4*>(vr);
                            raw[j][0] = u.x; raw[j][1] = u.y; raw[j][VEC / 2 - 2] = u.z; raw[j][VEC / 2 - 1] = u.w;
                        } else {
                            const uint2 u = *reinterpret_cast<const uint2*>(vr);
                            raw[j][0] = u.x; raw[j][1] = u.y;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < VEC / 2; i++) raw[j][i] = 0u;
                    }
                }
#pragma unroll
                for (int j = 0; j < KU; j++) {
                    const int k = kb + j * KS;
                    if (k >= nkeys) break;
                    float v[VEC];
#pragma unroll
                    for (int i = 0; i < VEC / 2; i++) {
                        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[j][i]));
                        v[2 * i] = f.x;
                        v[2 * i + 1] = f.y;
                    }
#pragma unroll
                    for (int g = 0; g < HB; g++) {
                        if (g < nhb) {
                            const float2 w01 = *reinterpret_cast<const float2*>(S + k * (HB * 2) + g * 2);
                            const float w0 = w01.x, w1 = w01.y;
#pragma unroll
                            for (int i = 0; i < VEC; i++) {
                                acc[g][0][i] = fmaf(w0, v[i], acc[g][0][i]);
                                acc[g][1][i] = fmaf(w1, v[i], acc[g][1][i]);
                            }
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
    // the slices' sums, in the order of the slices, and the block's share
    if (ks < KS) {
#pragma unroll
        for (int g = 0; g < HB; g++) {
            if (g < nhb) {
#pragma unroll
                for (int mp = 0; mp < 2; mp++)
#pragma unroll
                    for (int i = 0; i < VEC; i++) red[((size_t)ks * HB * 2 + g * 2 + mp) * dv + VEC * cpair + i] = acc[g][mp][i];
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < nhb * 2 * dv; i += DD_THREADS) {
        const int row = i / dv, c = i - row * dv;          // row = g * 2 + mp
        float v = 0.f;
        for (int sl = 0; sl < KS; sl++) v += red[((size_t)sl * HB * 2 + row) * dv + c];
        float* dst = part + ((((size_t)t * nh + h0 + (row >> 1)) * splits + z) * 2 + (row & 1)) * (dv + 2);
        dst[2 + c] = v;
        if (c == 0) {
            dst[0] = run_m[row];
            dst[1] = run_l[row];
        }
    }
}

// keys per block of the decode kernel for `splits` blocks over sequences of up to max_len keys: whole rounds of 256
extern "C" int illm_attention_diff_decode_keys(long long max_len, int splits) {
    const long long per = (max_len + splits - 1) / splits;
    return (int)((per + DD_THREADS - 1) / DD_THREADS * DD_THREADS);
}
extern "C" int illm_attention_diff_decode_supported(int nh, int nkv, int d, int dv) {
    return nkv > 0 && nh % nkv == 0 && d > 0 && d <= AD_MAX_D && d % 8 == 0 && dv >= 8 && dv <= AD_MAX_D && dv % 8 == 0 && dv / 4 <= DD_THREADS;
}

// q [T, q_stride] bfloat16, one token per sequence; scratch: illm_attention_diff_scratch(T, nh, dv, splits) floats (also for
// splits == 1); out [T, nh * dv] bfloat16
extern "C" int illm_attention_diff_decode(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages,
                                          const int* token_pos, const int* token_seq, void* out, int T, int nh, int nkv, int d, int dv, int page_size,
                                          int window, float scale, float lambda, float eps, float out_scale, long long max_len, int splits,
                                          float* scratch, void* stream) {
    if (T <= 0) return 0;
    if (!illm_attention_diff_decode_supported(nh, nkv, d, dv) || splits < 1 || splits > 65535 || !scratch || max_len <= 0 || nh > 65535) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int group = nh / nkv;
    const int hb = group >= 8 ? 8 : group > 2 ? 4 : group;
    const int subs = (group + hb - 1) / hb;
    if ((long long)nkv * subs > 65535) return ILLM_ERR_BAD_ARG;
    const int keys = illm_attention_diff_decode_keys(max_len, splits);
    const int vec = hb == 8 ? 4 : 8;          // channels per thread: sixteen heads-and-maps times eight channels would not fit the registers
    const int ksl = DD_THREADS / (dv / vec);
    const size_t smem = (size_t)DD_THREADS * sizeof(long long) + ((size_t)hb * 2 * d + (size_t)hb * 2 * DD_THREADS + (size_t)ksl * hb * 2 * dv) * sizeof(float);
    dim3 grid(T, nkv * subs, splits);
#define ILLM_DD(HB, VEC)                                                                                                                   \
    do {                                                                                                                                   \
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_diff_decode_kernel<HB, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        illm_launch(attention_diff_decode_kernel<HB, VEC>, grid, dim3(DD_THREADS), smem, s, (const bf16*)q, q_stride, (const bf16*)kc, (const bf16*)vc, \
                    block_table, max_pages, token_pos, token_seq, scratch, nh, nkv, d, dv, page_size, window, scale, keys);                \
    } while (0)
    if (smem > 200 * 1024) return ILLM_ERR_BAD_ARG;
    if (hb == 8) ILLM_DD(8, 4);
    else if (hb == 4) ILLM_DD(4, 8);
    else if (hb == 2) ILLM_DD(2, 8);
    else ILLM_DD(1, 8);
#undef ILLM_DD
    illm_launch(attention_diff_merge_kernel<bf16>, dim3(T, nh), dim3(AD_MAX_D), 0, s, (const float*)scratch, (bf16*)out, nh, dv, splits, lambda, eps, out_scale);
    return illm_launch_status();
}

// ---------------------------------------------------------------------------------------------------------------------
// attention_diff_mma_kernel: prompts (and further pieces of a sequence) in bfloat16 on warp-level MMA, flash-attention
// style.  A block owns 64 consecutive query tokens of one (sequence, head) and walks the sequence's keys in blocks of
// 64, K rows ([k_1, k_2], 2 d channels) and V rows (dv) from the cache pages into shared memory (cp.async, double
// buffered, rows padded by 16 bytes so that ldmatrix is conflict-free for every d and dv that are multiples of 16).
// Each of its 4 warps holds 16 query rows and takes the two maps in turn over the same staged tile: S_m = Q_m K_m^T
// (m16n8k16, float32 accumulators), scale, mask, running maximum and sum in float32, and O_m += P_m V with the weights
// as TWO bfloat16 terms (p = hi + lo, sixteen bits of mantissa), so the values are staged once for both maps.  The
// epilogue makes o = O_1 / l_1 - lambda O_2 / l_2, the head's unit norm and the factor, all in float32.
// d is a run-time size (a multiple of 16 up to 192); dv a template parameter (a multiple of 16 up to 128).

#define DM_BN 64
#define DM_BM 64
#define DM_THREADS 128

__device__ __forceinline__ unsigned dm_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void dm_cp16(unsigned dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void dm_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void dm_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void dm_ldsm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dm_ldsm4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dm_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// p0, p1 as two packed bfloat16 pairs: hi the rounded values, lo what the rounding left
__device__ __forceinline__ void dm_split(float p0, float p1, unsigned& hi, unsigned& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(p0 - hf.x, p1 - hf.y);
    hi = *reinterpret_cast<const unsigned*>(&h);
    lo = *reinterpret_cast<const unsigned*>(&l);
}

template <int DV>
__global__ void __launch_bounds__(DM_THREADS)
attention_diff_mma_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                          const int* __restrict__ block_table, int max_pages, const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
                          bf16* __restrict__ out, int nh, int nkv, int d, int page_size, int window, float scale_log2e, float lambda, float eps,
                          float out_scale) {
    pdl_grid_sync();
    constexpr int NT_V = DV / 8;          // n-tiles of the output
    const int KW = 2 * d;                 // channels of a query or key row (both maps)
    const int LDK = KW + 8, LDV = DV + 8; // padded rows (elements)
    const int CHK = KW / 8, CHV = DV / 8; // 16-byte chunks per row
    extern __shared__ __align__(128) unsigned char dm_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(dm_raw);          // [DM_BM][LDK]
    bf16* Ks = Qs + DM_BM * LDK;                         // [2][DM_BN][LDK]
    bf16* Vs = Ks + 2 * DM_BN * LDK;                     // [2][DM_BN][LDV]

    // the last tiles of a prompt see the most keys: they are started first
    const int b = blockIdx.z, h = blockIdx.y, tile = gridDim.x - 1 - blockIdx.x;
    const int q0 = cu_q[b], qlen = cu_q[b + 1] - q0;
    const int row0 = tile * DM_BM;
    if (row0 >= qlen) return;
    const int total = seq_lens[b], past = total - qlen;
    const int hk = h / (nh / nkv);
    const int rows_here = (qlen - row0 < DM_BM) ? qlen - row0 : DM_BM;
    const int first_pos = past + row0, last_pos = first_pos + rows_here - 1;
    const int lo_key = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
    const int jb0 = lo_key / DM_BN, jb1 = last_pos / DM_BN;
    const int* bt = block_table + (size_t)b * max_pages;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int mtx = lane >> 3;          // which 8x8 matrix of an ldmatrix.x4 this lane addresses
    const int wrow0 = warp * 16;        // first row of this warp inside the tile

    for (int i = tid; i < DM_BM * CHK; i += DM_THREADS) {
        const int r = i / CHK, c = i - r * CHK;
        const bool ok = r < rows_here;
        const bf16* src = ok ? q + (size_t)(q0 + row0 + r) * q_stride + (size_t)h * KW + c * 8 : q;
        dm_cp16(dm_smem(Qs + r * LDK + c * 8), src, ok ? 16 : 0);
    }
    auto load_kv = [&](int jb, int buf) {
        bf16* kd = Ks + buf * DM_BN * LDK;
        bf16* vd = Vs + buf * DM_BN * LDV;
        // rows that no query of the tile sees (beyond its last position, or below the window of its first, whose pages may
        // have gone back to the pool) are zero-filled instead of read
        for (int i = tid; i < DM_BN * (CHK + CHV); i += DM_THREADS) {
            const int r = i / (CHK + CHV), c = i - r * (CHK + CHV);
            const int key = jb * DM_BN + r;
            bool ok = key <= last_pos && key >= lo_key;
            size_t rowi = 0;
            if (ok) {
                const int page = bt[key / page_size];
                ok = page >= 0;
                if (ok) rowi = ((size_t)page * nkv + hk) * page_size + (key % page_size);
            }
            if (c < CHK) dm_cp16(dm_smem(kd + r * LDK + c * 8), kc + rowi * KW + c * 8, ok ? 16 : 0);
            else dm_cp16(dm_smem(vd + r * LDV + (c - CHK) * 8), vc + rowi * DV + (c - CHK) * 8, ok ? 16 : 0);
        }
    };
    load_kv(jb0, 0);
    dm_commit();

    // this thread owns rows g and g + 8 of the warp's 16
    float o[2][NT_V][4];
    float m_run[2][2], l_run[2][2];
    int pos_r[2];
#pragma unroll
    for (int mp = 0; mp < 2; mp++) {
#pragma unroll
        for (int i = 0; i < NT_V; i++) o[mp][i][0] = o[mp][i][1] = o[mp][i][2] = o[mp][i][3] = 0.f;
        m_run[mp][0] = m_run[mp][1] = -INFINITY;
        l_run[mp][0] = l_run[mp][1] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int r = wrow0 + g + e * 8;
        pos_r[e] = (r < rows_here) ? first_pos + r : last_pos;
    }
    const bool warp_active = wrow0 < rows_here;
    const int warp_last_pos = (wrow0 + 15 < rows_here) ? first_pos + wrow0 + 15 : last_pos;
    const int ksteps = d / 16;

    for (int jb = jb0; jb <= jb1; jb++) {
        const int buf = (jb - jb0) & 1;
        if (jb < jb1) load_kv(jb + 1, buf ^ 1);
        dm_commit();
        dm_wait<1>();
        __syncthreads();
        const bf16* kb = Ks + buf * DM_BN * LDK;
        const bf16* vb = Vs + buf * DM_BN * LDV;
        const int key0 = jb * DM_BN;
        if (warp_active && key0 <= warp_last_pos) {
            const bool need_mask = (key0 + DM_BN - 1 > first_pos + wrow0) || (window > 0);
#pragma unroll
            for (int mp = 0; mp < 2; mp++) {
                float s[DM_BN / 8][4];
#pragma unroll
                for (int i = 0; i < DM_BN / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
                for (int ks = 0; ks < ksteps; ks++) {
                    const int col = mp * d + ks * 16;
                    unsigned qf[4];
                    dm_ldsm4(qf[0], qf[1], qf[2], qf[3], dm_smem(Qs + (wrow0 + (mtx & 1) * 8 + (lane & 7)) * LDK + col + (mtx >> 1) * 8));
#pragma unroll
                    for (int np = 0; np < DM_BN / 16; np++) {
                        unsigned b0, b1, b2, b3;
                        dm_ldsm4(b0, b1, b2, b3, dm_smem(kb + (np * 16 + (mtx >> 1) * 8 + (lane & 7)) * LDK + col + (mtx & 1) * 8));
                        dm_mma(s[np * 2], qf, b0, b1);
                        dm_mma(s[np * 2 + 1], qf, b2, b3);
                    }
                }
                float m_new[2] = {m_run[mp][0], m_run[mp][1]};
#pragma unroll
                for (int nt = 0; nt < DM_BN / 8; nt++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        float v = s[nt][e] * scale_log2e;
                        if (need_mask) {
                            const int key = key0 + nt * 8 + t4 * 2 + (e & 1);
                            const int pr = pos_r[e >> 1];
                            if (key > pr || (window > 0 && key < pr - window + 1)) v = -INFINITY;
                        }
                        s[nt][e] = v;
                        m_new[e >> 1] = fmaxf(m_new[e >> 1], v);
                    }
                }
                float corr[2], m_use[2], psum[2] = {0.f, 0.f};
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 1));
                    m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 2));
                    m_use[e] = (m_new[e] == -INFINITY) ? 0.f : m_new[e];
                    corr[e] = (m_run[mp][e] == -INFINITY) ? 0.f : fast_exp2(m_run[mp][e] - m_use[e]);
                    m_run[mp][e] = m_new[e];
                }
                unsigned ph[DM_BN / 16][4], pl[DM_BN / 16][4];
#pragma unroll
                for (int nt = 0; nt < DM_BN / 8; nt++) {
                    const float p0 = fast_exp2(s[nt][0] - m_use[0]), p1 = fast_exp2(s[nt][1] - m_use[0]);
                    const float p2 = fast_exp2(s[nt][2] - m_use[1]), p3 = fast_exp2(s[nt][3] - m_use[1]);
                    psum[0] += p0 + p1;
                    psum[1] += p2 + p3;
                    dm_split(p0, p1, ph[nt >> 1][(nt & 1) * 2], pl[nt >> 1][(nt & 1) * 2]);
                    dm_split(p2, p3, ph[nt >> 1][(nt & 1) * 2 + 1], pl[nt >> 1][(nt & 1) * 2 + 1]);
                }
#pragma unroll
                for (int e = 0; e < 2; e++) l_run[mp][e] = l_run[mp][e] * corr[e] + psum[e];
#pragma unroll
                for (int i = 0; i < NT_V; i++) {
                    o[mp][i][0] *= corr[0];
                    o[mp][i][1] *= corr[0];
                    o[mp][i][2] *= corr[1];
                    o[mp][i][3] *= corr[1];
                }
                // the two terms of the weights in two passes over the staged values: an accumulator's two MMAs of a key
                // step then lie a whole pass apart instead of back to back (the second waits for the first's result)
#pragma unroll
                for (int ks = 0; ks < DM_BN / 16; ks++) {
#pragma unroll
                    for (int term = 0; term < 2; term++) {
#pragma unroll
                        for (int np = 0; np < NT_V / 2; np++) {
                            unsigned b0, b1, b2, b3;
                            dm_ldsm4_trans(b0, b1, b2, b3, dm_smem(vb + (ks * 16 + (mtx & 1) * 8 + (lane & 7)) * LDV + (np * 2 + (mtx >> 1)) * 8));
                            dm_mma(o[mp][np * 2], term ? pl[ks] : ph[ks], b0, b1);
                            dm_mma(o[mp][np * 2 + 1], term ? pl[ks] : ph[ks], b2, b3);
                        }
                    }
                }
            }
        }
        __syncthreads();   // everyone is done with this buffer before the next load overwrites it
    }
    dm_wait<0>();

    // ---- o = a_1 - lambda a_2, the head's unit norm, the factor; rows g and g + 8
#pragma unroll
    for (int e = 0; e < 2; e++) {
        float inv[2];
#pragma unroll
        for (int mp = 0; mp < 2; mp++) {
            float lsum = l_run[mp][e];
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
            inv[mp] = 1.0f / lsum;
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NT_V; i++) {
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const float v = o[0][i][e * 2 + c] * inv[0] - lambda * (o[1][i][e * 2 + c] * inv[1]);
                o[0][i][e * 2 + c] = v;
                ss = fmaf(v, v, ss);
            }
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        const int r = wrow0 + g + e * 8;
        if (r >= rows_here) continue;
        const float f = (1.0f / sqrtf(ss / (float)DV + eps)) * out_scale;
        bf16* dst = out + ((size_t)(q0 + row0 + r) * nh + h) * DV;
#pragma unroll
        for (int i = 0; i < NT_V; i++)
            *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + t4 * 2) = __floats2bfloat162_rn(o[0][i][e * 2] * f, o[0][i][e * 2 + 1] * f);
    }
}

template <int DV>
static int dm_launch(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* cu_q,
                     const int* seq_lens, void* out, int B, int max_q, int nh, int nkv, int d, int page_size, int window, float scale, float lambda,
                     float eps, float out_scale, cudaStream_t s) {
    const size_t smem = ((size_t)(DM_BM + 2 * DM_BN) * (2 * d + 8) + (size_t)2 * DM_BN * (DV + 8)) * sizeof(bf16);
    auto kern = attention_diff_mma_kernel<DV>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid((max_q + DM_BM - 1) / DM_BM, nh, B);
    illm_launch(kern, grid, dim3(DM_THREADS), smem, s, (const bf16*)q, q_stride, (const bf16*)kc, (const bf16*)vc, block_table, max_pages, cu_q,
                seq_lens, (bf16*)out, nh, nkv, d, page_size, window, scale * 1.4426950408889634f, lambda, eps, out_scale);
    return illm_launch_status();
}

// sizes the tensor-core kernel takes: d and dv multiples of 16, d up to 192 (what shared memory holds), dv up to 128
extern "C" int illm_attention_diff_mma_supported(int d, int dv) { return d > 0 && d <= 192 && d % 16 == 0 && dv > 0 && dv <= 128 && dv % 16 == 0; }

// q [T, q_stride] bfloat16 with head h's [q_1, q_2] at column h * 2 d; the step's sequences by cu_q [B + 1] and seq_lens [B]
extern "C" int illm_attention_diff_mma(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages,
                                       const int* cu_q, const int* seq_lens, void* out, int B, int max_q, int nh, int nkv, int d, int dv, int page_size,
                                       int window, float scale, float lambda, float eps, float out_scale, void* stream) {
    if (B <= 0 || max_q <= 0) return 0;
    if (!illm_attention_diff_mma_supported(d, dv) || nkv <= 0 || nh % nkv || nh > 65535 || B > 65535 || (q_stride & 7)) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
#define ILLM_DM(DV) \
    case DV: return dm_launch<DV>(q, q_stride, kc, vc, block_table, max_pages, cu_q, seq_lens, out, B, max_q, nh, nkv, d, page_size, window, scale, lambda, eps, out_scale, s)
    switch (dv) {
        ILLM_DM(16);
        ILLM_DM(32);
        ILLM_DM(48);
        ILLM_DM(64);
        ILLM_DM(80);
        ILLM_DM(96);
        ILLM_DM(112);
        ILLM_DM(128);
    }
#undef ILLM_DM
    return ILLM_ERR_BAD_ARG;
}
