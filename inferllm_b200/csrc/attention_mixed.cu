// Softmax attention whose heads see one another's scores before the softmax, over keys that are also the values:
//
//   raw_g(i, j)   = (q_g(i) . k_kv(g)(j)) * scale - r1_g * ln(1 + r2_g * (i - j))          (the distance term optional)
//   score_h(i, j) = sum_g mix[h, g] * raw_g(i, j)                                            (the mix optional)
//   o_h(i)        = sum_j softmax_j(score_h(i, .)) k_kv(h)(j),   j from max(0, i - window + 1) (window 0: 0) to i
//   out           = o * sigmoid(gate)                                                        (element by element, optional)
//
// Because a head's softmax needs every head's raw score of the same (i, j), one block owns a token with ALL its
// heads: it walks the keys in tiles that it stages in shared memory once for all heads (all key/value heads of the
// tile's positions, read from the paged cache: [pages, kv heads, page_size, d]), takes the raw scores of the tile
// (a thread per (head, key)), mixes them, updates each head's running maximum and sum (a warp per head) and adds the
// weighted keys to the outputs (a thread per output channel).  All arithmetic is float32; the cache and q are the
// activation dtype.  The walk depends only on the token's own position and the window, never on the step.
#include <math.h>

#include "common.cuh"

#define AM_THREADS 256
#define AM_MAX_ACC 32          // outputs per thread: heads * d <= 8192

struct AttnMixedArgs {
    const void* q;
    int q_stride;
    const void* kc;
    const int *block_table, *token_pos, *token_seq;
    int max_pages, page_size, window;
    int nh, nkv, d, kt, row_elems;      // kt keys per tile; a staged key row has row_elems elements (all kv heads + padding)
    float scale;
    const float *r1, *r2, *mix, *gate;
    int gate_stride;
    void* out;
    int splits;         // > 1: block (t, s) takes the s-th part of the token's keys and leaves (acc, m, l) in `part`
    float* part;        // [T, splits, nh * d + 2 * nh]
};

template <typename TA>
__global__ void __launch_bounds__(AM_THREADS) attention_mixed_kernel(AttnMixedArgs a) {
    pdl_grid_sync();
    extern __shared__ __align__(16) unsigned char am_raw[];
    const int nh = a.nh, nkv = a.nkv, d = a.d, KT = a.kt, nq = nh * d, grp = nh / nkv;
    float* qs = reinterpret_cast<float*>(am_raw);            // [nh * d]
    float* raw = qs + nq;                                      // [nh][KT]
    float* pr = raw + nh * KT;                                 // [nh][KT] mixed scores, then weights
    float* m_s = pr + nh * KT;                                 // [nh] running maximum
    float* l_s = m_s + nh;                                     // [nh] running sum
    float* c_s = l_s + nh;                                     // [nh] this tile's correction
    float* mix_s = c_s + nh;                                   // [nh * nh]
    const int n_floats = (nq + 2 * nh * KT + 3 * nh + (a.mix ? nh * nh : 0) + 3) & ~3;
    TA* kt_s = reinterpret_cast<TA*>(am_raw + (size_t)n_floats * sizeof(float));      // [KT][row_elems]
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int p = a.token_pos[t];
    const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
    const int* bt = a.block_table + (size_t)a.token_seq[t] * a.max_pages;
    const TA* qrow = (const TA*)a.q + (size_t)t * a.q_stride;
    for (int c = tid; c < nq; c += AM_THREADS) qs[c] = to_f32(qrow[c]);
    for (int h = tid; h < nh; h += AM_THREADS) {
        m_s[h] = -INFINITY;
        l_s[h] = 0.f;
    }
    if (a.mix)
        for (int i = tid; i < nh * nh; i += AM_THREADS) mix_s[i] = a.mix[i];
    float acc[AM_MAX_ACC];
#pragma unroll
    for (int i = 0; i < AM_MAX_ACC; i++) acc[i] = 0.f;
    const bool vec = (d & 7) == 0;
    const int kv_elems = nkv * d;
    int k_lo = lo, k_hi = p;
    if (a.splits > 1) {     // whole tiles per part, counted from the first visible key
        const int per = ((p - lo + a.splits) / a.splits + KT - 1) / KT * KT;
        k_lo = lo + (int)blockIdx.y * per;
        k_hi = k_lo + per - 1 < p ? k_lo + per - 1 : p;
    }
    for (int kb = k_lo; kb <= k_hi; kb += KT) {
        const int cnt = k_hi - kb + 1 < KT ? k_hi - kb + 1 : KT;
        __syncthreads();        // the tile before this one has been used up (and qs, m, l are written)
        // the tile's key rows, all kv heads of a position side by side
        if (vec) {
            const int per = kv_elems >> 3;
            for (int idx = tid; idx < cnt * per; idx += AM_THREADS) {
                const int j = idx / per, e = (idx - j * per) << 3, hk = e / d, c = e - hk * d, key = kb + j;
                const int page = bt[key / a.page_size];
                const TA* src = (const TA*)a.kc + ((((size_t)page * nkv + hk) * a.page_size + key % a.page_size) * d + c);
                *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(kt_s + (size_t)j * a.row_elems + e)) =
                    *reinterpret_cast<const uint4*>(src);
                if (sizeof(TA) == 4)
                    *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(kt_s + (size_t)j * a.row_elems + e + 4)) =
                        *reinterpret_cast<const uint4*>(src + 4);
            }
        } else {
            for (int idx = tid; idx < cnt * kv_elems; idx += AM_THREADS) {
                const int j = idx / kv_elems, e = idx - j * kv_elems, hk = e / d, c = e - hk * d, key = kb + j;
                const int page = bt[key / a.page_size];
                kt_s[(size_t)j * a.row_elems + e] = ((const TA*)a.kc)[(((size_t)page * nkv + hk) * a.page_size + key % a.page_size) * d + c];
            }
        }
        __syncthreads();
        // raw scores: a thread per (head, key)
        for (int idx = tid; idx < nh * KT; idx += AM_THREADS) {
            const int h = idx / KT, j = idx - h * KT;
            float s = 0.f;
            if (j < cnt) {
                const TA* kr = kt_s + (size_t)j * a.row_elems + (h / grp) * d;
                const float* qh = qs + h * d;
                float dot = 0.f;
                if (vec) {
                    for (int c = 0; c < d; c += 8) {
                        float f[8];
                        load8(kr + c, f);
#pragma unroll
                        for (int i = 0; i < 8; i++) dot = fmaf(qh[c + i], f[i], dot);
                    }
                } else {
                    for (int c = 0; c < d; c++) dot = fmaf(qh[c], to_f32(kr[c]), dot);
                }
                s = dot * a.scale;
                if (a.r1) s -= a.r1[h] * log1pf(a.r2[h] * (float)(p - (kb + j)));
            }
            raw[idx] = s;
        }
        __syncthreads();
        // the heads' scores mixed, then each head's running maximum and sum: a warp per head, a key per lane
        for (int h = warp; h < nh; h += AM_THREADS / 32) {
            float mx = -INFINITY;
            for (int j = lane; j < KT; j += 32) {
                float s = -INFINITY;
                if (j < cnt) {
                    if (a.mix) {
                        s = 0.f;
                        for (int g = 0; g < nh; g++) s = fmaf(mix_s[h * nh + g], raw[g * KT + j], s);
                    } else {
                        s = raw[h * KT + j];
                    }
                }
                pr[h * KT + j] = s;
                mx = fmaxf(mx, s);
            }
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, warp_max(mx));
            float sum = 0.f;
            for (int j = lane; j < KT; j += 32) {
                const float s = pr[h * KT + j];
                const float w = j < cnt ? expf(s - m_new) : 0.f;
                pr[h * KT + j] = w;
                sum += w;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float corr = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
                c_s[h] = corr;
                l_s[h] = l_s[h] * corr + sum;
                m_s[h] = m_new;
            }
        }
        __syncthreads();
        // the weighted keys: a thread per output channel
#pragma unroll
        for (int i = 0; i < AM_MAX_ACC; i++) {
            const int e = tid + i * AM_THREADS;
            if (e < nq) {
                const int h = e / d, c = e - h * d;
                const TA* col = kt_s + (h / grp) * d + c;
                const float* w = pr + h * KT;
                float s = acc[i] * c_s[h];
                for (int j = 0; j < cnt; j++) s = fmaf(w[j], to_f32(col[(size_t)j * a.row_elems]), s);
                acc[i] = s;
            }
        }
    }
    __syncthreads();
    if (a.splits > 1) {
        float* ps = a.part + ((size_t)t * a.splits + blockIdx.y) * (nq + 2 * nh);
#pragma unroll
        for (int i = 0; i < AM_MAX_ACC; i++) {
            const int e = tid + i * AM_THREADS;
            if (e < nq) ps[e] = acc[i];
        }
        for (int h = tid; h < nh; h += AM_THREADS) {
            ps[nq + h] = m_s[h];
            ps[nq + nh + h] = l_s[h];
        }
        return;
    }
    TA* o = (TA*)a.out + (size_t)t * nq;
#pragma unroll
    for (int i = 0; i < AM_MAX_ACC; i++) {
        const int e = tid + i * AM_THREADS;
        if (e < nq) {
            float v = acc[i] / l_s[e / d];
            if (a.gate) v *= 1.0f / (1.0f + expf(-a.gate[(size_t)t * a.gate_stride + e]));
            o[e] = from_f32<TA>(v);
        }
    }
}

// The parts of a token's keys put together: weights exp(m_s - max m), the parts in their order; then the gate.
template <typename TA>
__global__ void __launch_bounds__(AM_THREADS) attention_mixed_merge_kernel(AttnMixedArgs a) {
    pdl_grid_sync();
    const int t = blockIdx.x, nq = a.nh * a.d, stride = nq + 2 * a.nh;
    const float* ps = a.part + (size_t)t * a.splits * stride;
    for (int e = threadIdx.x; e < nq; e += AM_THREADS) {
        const int h = e / a.d;
        float mx = -INFINITY;
        for (int s = 0; s < a.splits; s++) mx = fmaxf(mx, ps[(size_t)s * stride + nq + h]);
        float l = 0.f, v = 0.f;
        for (int s = 0; s < a.splits; s++) {
            const float ms = ps[(size_t)s * stride + nq + h];
            if (ms == -INFINITY) continue;      // a part without keys
            const float w = expf(ms - mx);
            l = fmaf(ps[(size_t)s * stride + nq + a.nh + h], w, l);
            v = fmaf(ps[(size_t)s * stride + e], w, v);
        }
        v /= l;
        if (a.gate) v *= 1.0f / (1.0f + expf(-a.gate[(size_t)t * a.gate_stride + e]));
        ((TA*)a.out)[(size_t)t * nq + e] = from_f32<TA>(v);
    }
}

// keys per tile and the bytes of shared memory for a head count, kv head count, head size and element size
static int am_plan(int nh, int nkv, int d, int esize, int has_mix, size_t* smem, int* row_elems) {
    const int pad = 16 / esize;                                   // 16 bytes, so that rows shift by four banks
    *row_elems = nkv * d + pad;
    const size_t row_bytes = (size_t)*row_elems * esize;
    int kt = 32;
    for (;; kt >>= 1) {
        size_t floats = (size_t)nh * d + 2 * (size_t)nh * kt + 3 * (size_t)nh + (has_mix ? (size_t)nh * nh : 0);
        floats = (floats + 3) & ~(size_t)3;
        *smem = floats * sizeof(float) + (size_t)kt * row_bytes;
        if (*smem <= 160 * 1024 || kt == 1) break;
    }
    return kt;
}

extern "C" int illm_attention_mixed_supported(int nh, int nkv, int d, int esize) {
    if (nh <= 0 || nkv <= 0 || nh % nkv || d <= 0 || (long long)nh * d > AM_MAX_ACC * AM_THREADS) return 0;
    size_t smem;
    int re;
    am_plan(nh, nkv, d, esize, 1, &smem, &re);
    return smem <= 200 * 1024 ? 1 : 0;
}

// q [T, q_stride] and out [T, nh * d] in the activation dtype, kc the keys-only pages; r1, r2 [nh], mix [nh, nh],
// gate [T, gate_stride] float32, each nullptr to leave its term out.  splits > 1 (few tokens over many keys: the
// blocks of single-token steps would leave most of the GPU idle): every token's keys in that many parts, a block
// each, over `part` (float32 [T, splits, nh * d + 2 * nh]), and a second kernel that puts the parts together.  The
// sums then have another order than with one part.
extern "C" int illm_attention_mixed_keys_per_tile(int nh, int nkv, int d, int esize, int has_mix) {
    size_t smem;
    int re;
    return am_plan(nh, nkv, d, esize, has_mix, &smem, &re);
}

extern "C" int illm_attention_mixed(const void* q, int q_stride, const void* kc, const int* block_table, int max_pages, const int* token_pos,
                                    const int* token_seq, void* out, int act_dtype, int T, int nh, int nkv, int d, int page_size, int window,
                                    float scale, const float* r1, const float* r2, const float* mix, const float* gate, int gate_stride,
                                    int splits, float* part, void* stream) {
    if (T <= 0) return 0;
    const int esize = act_dtype == ILLM_F32 ? 4 : 2;
    if ((act_dtype != ILLM_F32 && act_dtype != ILLM_BF16) || !illm_attention_mixed_supported(nh, nkv, d, esize) || !q || !kc || !out ||
        ((r1 == nullptr) != (r2 == nullptr)) || page_size <= 0 || splits < 1 || splits > 65535 || (splits > 1 && !part))
        return ILLM_ERR_BAD_ARG;
    AttnMixedArgs a{q, q_stride, kc, block_table, token_pos, token_seq, max_pages, page_size, window, nh, nkv, d, 0, 0, scale, r1, r2, mix, gate,
                    gate_stride, out, splits, part};
    size_t smem;
    a.kt = am_plan(nh, nkv, d, esize, mix != nullptr, &smem, &a.row_elems);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == ILLM_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_mixed_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        illm_launch(attention_mixed_kernel<bf16>, dim3(T, splits), dim3(AM_THREADS), smem, s, a);
        if (splits > 1) illm_launch(attention_mixed_merge_kernel<bf16>, dim3(T), dim3(AM_THREADS), 0, s, a);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_mixed_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        illm_launch(attention_mixed_kernel<float>, dim3(T, splits), dim3(AM_THREADS), smem, s, a);
        if (splits > 1) illm_launch(attention_mixed_merge_kernel<float>, dim3(T), dim3(AM_THREADS), 0, s, a);
    }
    return illm_launch_status();
}
