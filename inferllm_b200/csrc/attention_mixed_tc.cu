// The prompts' form of the attention whose heads see one another's scores (attention_mixed.cu has the equations and
// the general kernel): bfloat16 q and keys, the two products on tensor cores (warp-level MMA, float32 accumulation),
// everything between them float32.
//
// A block owns 16 consecutive tokens of one sequence and HS of the heads' outputs.  A head's softmax needs EVERY
// head's raw score of the same (query, key), and the outputs of all heads of 16 tokens are more than an SM's
// registers hold, so each block takes the raw scores of all heads (q k^T of all heads, the cheap product: it is
// repeated by the heads / HS blocks of a token tile) and mixes, normalises and weighs only for its own HS heads.
// Per tile of AT_KT keys, staged once for all key heads:
//   1. raw_g(i, j) = q_g(i) . k(j) * scale - r1_g ln(1 + r2_g (p_i - j)), a head per warp in turn  -> shared memory
//      (the distance terms from a table of the tile's 31 distances per head)
//   2. two threads per (i, j), half of the block's heads each: s_h = sum_g mix[h, g] raw_g, g ascending, for the block's heads; hidden pairs get -inf
//   3. a thread per (head, query) row: the running maximum and sum, the tile's weights, the old sums' correction
//   4. o_h(i) <- o_h(i) corr + P_h K: the weights as two bfloat16 (upper and lower half of 16 bits of mantissa), the
//      keys read transposed from the staged tile; a warp owns some of the (head, 8 channels) tiles of the output.
#include <math.h>

#include "common.cuh"

#define AT_THREADS 512
#define AT_BQ 16
#define AT_KT 16
#define AT_ACC 8           // (head, 8 channels) output tiles per warp at most: HS * d <= 1024 over 16 warps
#define AT_ST 4           // pieces of 16 bytes of a key tile per thread whose places are kept in registers
#define AT_LD (AT_KT + 1)  // floats per (head, query) row of scores

struct AttnMixedTcArgs {
    const bf16* q;
    int q_stride;
    const bf16* kc;
    const int *block_table, *token_pos, *cu_q;
    int max_pages, page_size, page_shift, window;      // page_shift: log2 of the page size, -1 if it is no power of two
    int nh, nkv, d, hs, B;
    float scale;
    const float *r1, *r2, *mix, *gate;
    int gate_stride;
    bf16* out;
};

__device__ __forceinline__ void at_mma(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void at_ldmatrix_x2_trans(unsigned& r0, unsigned& r1, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}

// two weights as a pair of bfloat16 (the first in the low half), and what that rounding left of them as another pair
__device__ __forceinline__ void at_split(float x, float y, unsigned& hi, unsigned& lo) {
    const bf16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
    const bf16 xl = __float2bfloat16_rn(x - __bfloat162float(xh)), yl = __float2bfloat16_rn(y - __bfloat162float(yh));
    hi = (unsigned)__bfloat16_as_ushort(xh) | ((unsigned)__bfloat16_as_ushort(yh) << 16);
    lo = (unsigned)__bfloat16_as_ushort(xl) | ((unsigned)__bfloat16_as_ushort(yl) << 16);
}

struct AtPlan {
    int q_ld, k_ld;                                   // elements per staged q row and key row
    size_t q_off, k_off, raw_off, pr_off, corr_off, l_off, mix_off, pos_off, tab_off, total;
};

static __host__ __device__ inline AtPlan at_plan(int nh, int nkv, int d, int hs) {
    AtPlan p;
    p.q_ld = nh * d + 8;
    p.k_ld = nkv * d + 8;
    size_t at = 0;
    p.q_off = at, at += (size_t)AT_BQ * p.q_ld * 2;
    p.k_off = at, at += (size_t)AT_KT * p.k_ld * 2;
    p.raw_off = at, at += (size_t)nh * AT_BQ * AT_LD * 4;
    p.pr_off = at, at += (size_t)hs * AT_BQ * AT_LD * 4;
    p.corr_off = at, at += (size_t)hs * AT_BQ * 4;
    p.l_off = at, at += (size_t)hs * AT_BQ * 4;
    p.mix_off = at, at += (size_t)hs * nh * 4;
    p.pos_off = at, at += AT_BQ * 4;
    p.tab_off = at, at += (size_t)nh * 32 * 4;
    p.total = (at + 15) & ~(size_t)15;
    return p;
}

// HSM: a power of two that is at least the heads per block (the bound of the loops over a pair's heads)
template <int HSM>
__global__ void __launch_bounds__(AT_THREADS) attention_mixed_tc_kernel(AttnMixedTcArgs a) {
    pdl_grid_sync();
    extern __shared__ __align__(16) unsigned char at_raw[];
    const int nh = a.nh, nkv = a.nkv, d = a.d, HS = a.hs, grp = nh / nkv, nq = nh * d;
    const AtPlan pl = at_plan(nh, nkv, d, HS);
    bf16* q_s = reinterpret_cast<bf16*>(at_raw + pl.q_off);          // [16][q_ld]
    bf16* k_s = reinterpret_cast<bf16*>(at_raw + pl.k_off);          // [AT_KT][k_ld]
    float* raw = reinterpret_cast<float*>(at_raw + pl.raw_off);      // [nh][16][AT_LD]
    float* pr = reinterpret_cast<float*>(at_raw + pl.pr_off);        // [HS][16][AT_LD] mixed scores, then weights
    float* corr_s = reinterpret_cast<float*>(at_raw + pl.corr_off);  // [HS][16]
    float* l_s = reinterpret_cast<float*>(at_raw + pl.l_off);        // [HS][16]
    float* mix_s = reinterpret_cast<float*>(at_raw + pl.mix_off);    // [HS][nh]: the block's rows of the mix
    int* pos_s = reinterpret_cast<int*>(at_raw + pl.pos_off);        // [16], -1 beyond the sequence's tokens
    float* tab_s = reinterpret_cast<float*>(at_raw + pl.tab_off);    // [nh][32]: the tile's distance terms
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
    const int q_ld = pl.q_ld, k_ld = pl.k_ld;

    // which sequence, and which 16 of its tokens
    int b = 0, tile = blockIdx.x;
    for (; b < a.B; b++) {
        const int nt = (a.cu_q[b + 1] - a.cu_q[b] + AT_BQ - 1) / AT_BQ;
        if (tile < nt) break;
        tile -= nt;
    }
    if (b >= a.B) return;
    const int t0 = a.cu_q[b] + tile * AT_BQ;
    const int rows = a.cu_q[b + 1] - t0 < AT_BQ ? a.cu_q[b + 1] - t0 : AT_BQ;
    const int h0 = blockIdx.y * HS;
    const int* bt = a.block_table + (size_t)b * a.max_pages;

    if (tid < AT_BQ) pos_s[tid] = tid < rows ? a.token_pos[t0 + tid] : -1;
    {
        const int per8 = nq >> 3;
        for (int idx = tid; idx < AT_BQ * per8; idx += AT_THREADS) {
            const int i = idx / per8, e = (idx - i * per8) << 3;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (i < rows) v = *reinterpret_cast<const uint4*>(a.q + (size_t)(t0 + i) * a.q_stride + e);
            *reinterpret_cast<uint4*>(q_s + (size_t)i * q_ld + e) = v;
        }
    }
    if (a.mix)
        for (int i = tid; i < HS * nh; i += AT_THREADS) mix_s[i] = a.mix[(size_t)(h0 + i / nh) * nh + i % nh];
    __syncthreads();
    const int p_first = pos_s[0], p_last = pos_s[rows - 1];
    const int lo_first = (a.window > 0 && p_first - a.window + 1 > 0) ? p_first - a.window + 1 : 0;

    float m_run = -INFINITY, l_run = 0.f;          // of the row (head, query) = tid, for tid < HS * 16
    float acc[AT_ACC][4];
#pragma unroll
    for (int x = 0; x < AT_ACC; x++) acc[x][0] = acc[x][1] = acc[x][2] = acc[x][3] = 0.f;
    const int d8 = d >> 3, n_out = HS * d8, per = (n_out + AT_THREADS / 32 - 1) / (AT_THREADS / 32);     // output tiles, and how many a warp owns
    const int kper8 = (nkv * d) >> 3;
    // which pieces of a key tile this thread stages are the same for every tile: taken apart once (no division in the walk)
    const size_t page_elems = (size_t)nkv * a.page_size * d;
    int st_j[AT_ST], st_src[AT_ST], st_dst[AT_ST];
#pragma unroll
    for (int r = 0; r < AT_ST; r++) {
        const int idx = tid + r * AT_THREADS;
        st_j[r] = -1, st_src[r] = 0, st_dst[r] = 0;
        if (idx < AT_KT * kper8) {
            const int j = idx / kper8, e = (idx - j * kper8) << 3, hk = e / d, c = e - hk * d;
            st_j[r] = j;
            st_src[r] = hk * a.page_size * d + c;
            st_dst[r] = j * k_ld + e;
        }
    }
    // the first output tile of this warp; the others follow by counting
    const int u0 = warp * per, hh_first = u0 / d8, nt_first = u0 - hh_first * d8;

    for (int kb = lo_first; kb <= p_last; kb += AT_KT) {
        __syncthreads();        // the tile before this one has been used up
#pragma unroll
        for (int r = 0; r < AT_ST; r++) {
            if (st_j[r] >= 0) {
                const int key = kb + st_j[r];
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (key <= p_last) {
                    const int pg = a.page_shift >= 0 ? key >> a.page_shift : key / a.page_size;
                    const int in_pg = key - pg * a.page_size;
                    v = *reinterpret_cast<const uint4*>(a.kc + (size_t)bt[pg] * page_elems + st_src[r] + in_pg * d);
                }
                *reinterpret_cast<uint4*>(k_s + st_dst[r]) = v;
            }
        }
        for (int idx = tid + AT_ST * AT_THREADS; idx < AT_KT * kper8; idx += AT_THREADS) {      // key rows beyond AT_ST pieces per thread
            const int j = idx / kper8, e = (idx - j * kper8) << 3, hk = e / d, c = e - hk * d, key = kb + j;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (key <= p_last) {
                const int page = bt[key / a.page_size];
                v = *reinterpret_cast<const uint4*>(a.kc + ((((size_t)page * nkv + hk) * a.page_size + key % a.page_size) * d + c));
            }
            *reinterpret_cast<uint4*>(k_s + (size_t)j * k_ld + e) = v;
        }
        // the distance terms of the tile: a sequence's tokens have consecutive positions, so the pair (i, j) is
        // p_first + i - kb - j apart, one of 31 distances; entry [h][i - j + 15] (hidden pairs, whose distance is
        // negative, get the term of distance 0 and are masked later)
        if (a.r1)
            for (int idx = tid; idx < nh * 32; idx += AT_THREADS) {
                const int h = idx >> 5, dist = p_first - kb + (idx & 31) - 15;
                tab_s[idx] = a.r1[h] * __logf(1.0f + a.r2[h] * (float)(dist > 0 ? dist : 0));
            }
        __syncthreads();
        // 1. every head's raw scores of the 16 x 16 pairs
        for (int h = warp; h < nh; h += AT_THREADS / 32) {
            float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};      // keys 0..7 and 8..15 of the tile
            const bf16* qa = q_s + (size_t)gid * q_ld + h * d + 2 * tig;
            const bf16* ka = k_s + (size_t)gid * k_ld + (h / grp) * d + 2 * tig;
            for (int k0 = 0; k0 < d; k0 += 16) {
                const unsigned a0 = *reinterpret_cast<const unsigned*>(qa + k0), a1 = *reinterpret_cast<const unsigned*>(qa + 8 * q_ld + k0);
                const unsigned a2 = *reinterpret_cast<const unsigned*>(qa + k0 + 8), a3 = *reinterpret_cast<const unsigned*>(qa + 8 * q_ld + k0 + 8);
                at_mma(c0, a0, a1, a2, a3, *reinterpret_cast<const unsigned*>(ka + k0), *reinterpret_cast<const unsigned*>(ka + k0 + 8));
                at_mma(c1, a0, a1, a2, a3, *reinterpret_cast<const unsigned*>(ka + 8 * k_ld + k0), *reinterpret_cast<const unsigned*>(ka + 8 * k_ld + k0 + 8));
            }
#pragma unroll
            for (int v = 0; v < 8; v++) {
                const int i = gid + ((v & 2) ? 8 : 0), j = 2 * tig + (v & 1) + ((v & 4) ? 8 : 0);
                float s = ((v & 4) ? c1[v & 3] : c0[v & 3]) * a.scale;
                if (a.r1) s -= tab_s[h * 32 + i - j + 15];
                raw[(h * AT_BQ + i) * AT_LD + j] = s;
            }
        }
        __syncthreads();
        // 2. the block's heads' mixed scores: a pair and half of the block's heads per thread
        {
            constexpr int HH = HSM > 1 ? HSM / 2 : 1;
            const int pair = tid & 255, hb = (tid >> 8) * HH;
            const int i = pair >> 4, j = pair & 15, key = kb + j, pi = pos_s[i];
            const int lo_i = (a.window > 0 && pi - a.window + 1 > 0) ? pi - a.window + 1 : 0;
            const bool visible = pi >= 0 && key <= pi && key >= lo_i;
            const int at = i * AT_LD + j;
            if (a.mix) {
                float s[HH];
#pragma unroll
                for (int x = 0; x < HH; x++) s[x] = 0.f;
                for (int g = 0; g < nh; g++) {
                    const float r = raw[g * AT_BQ * AT_LD + at];
#pragma unroll
                    for (int x = 0; x < HH; x++)
                        if (hb + x < HS) s[x] = fmaf(mix_s[(hb + x) * nh + g], r, s[x]);
                }
#pragma unroll
                for (int x = 0; x < HH; x++)
                    if (hb + x < HS) pr[(hb + x) * AT_BQ * AT_LD + at] = visible ? s[x] : -INFINITY;
            } else {
#pragma unroll
                for (int x = 0; x < HH; x++)
                    if (hb + x < HS) pr[(hb + x) * AT_BQ * AT_LD + at] = visible ? raw[(h0 + hb + x) * AT_BQ * AT_LD + at] : -INFINITY;
            }
        }
        __syncthreads();
        // 3. a (head, query) row per thread: maximum, weights, sum
        if (tid < HS * AT_BQ) {
            float* row = pr + tid * AT_LD;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < AT_KT; j++) mx = fmaxf(mx, row[j]);
            const float m_new = fmaxf(m_run, mx);
            float sum = 0.f, corr = 1.f;
            if (m_new == -INFINITY) {           // nothing visible yet
#pragma unroll
                for (int j = 0; j < AT_KT; j++) row[j] = 0.f;
            } else {
                corr = __expf(m_run - m_new);
#pragma unroll
                for (int j = 0; j < AT_KT; j++) {
                    const float w = __expf(row[j] - m_new);
                    row[j] = w;
                    sum += w;
                }
            }
            l_run = l_run * corr + sum;
            m_run = m_new;
            corr_s[tid] = corr;
        }
        __syncthreads();
        // 4. the weighted keys
        {
            int cur = -1;
            unsigned ah[4] = {0u, 0u, 0u, 0u}, al[4] = {0u, 0u, 0u, 0u};
            float cg = 1.f, cg8 = 1.f;
            int hh = hh_first, nt = nt_first;
#pragma unroll
            for (int x = 0; x < AT_ACC; x++) {
                if (x < per && u0 + x < n_out) {
                    if (hh != cur) {
                        cur = hh;
                        const float* pw = pr + hh * AT_BQ * AT_LD;
                        at_split(pw[gid * AT_LD + 2 * tig], pw[gid * AT_LD + 2 * tig + 1], ah[0], al[0]);
                        at_split(pw[(gid + 8) * AT_LD + 2 * tig], pw[(gid + 8) * AT_LD + 2 * tig + 1], ah[1], al[1]);
                        at_split(pw[gid * AT_LD + 2 * tig + 8], pw[gid * AT_LD + 2 * tig + 9], ah[2], al[2]);
                        at_split(pw[(gid + 8) * AT_LD + 2 * tig + 8], pw[(gid + 8) * AT_LD + 2 * tig + 9], ah[3], al[3]);
                        cg = corr_s[hh * AT_BQ + gid];
                        cg8 = corr_s[hh * AT_BQ + gid + 8];
                    }
                    acc[x][0] *= cg, acc[x][1] *= cg, acc[x][2] *= cg8, acc[x][3] *= cg8;
                    const bf16* vb = k_s + (size_t)(lane & 15) * k_ld + ((h0 + hh) / grp) * d + nt * 8;
                    unsigned b0, b1;
                    at_ldmatrix_x2_trans(b0, b1, (unsigned)__cvta_generic_to_shared(vb));
                    at_mma(acc[x], ah[0], ah[1], ah[2], ah[3], b0, b1);
                    at_mma(acc[x], al[0], al[1], al[2], al[3], b0, b1);
                    if (++nt == d8) nt = 0, hh++;
                }
            }
        }
    }
    if (tid < HS * AT_BQ) l_s[tid] = l_run;
    __syncthreads();
#pragma unroll
    for (int x = 0; x < AT_ACC; x++) {
        if (x < per && u0 + x < n_out) {
            const int hh = (u0 + x) / d8, nt = u0 + x - hh * d8;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int i = gid + 8 * half;
                if (i < rows) {
                    const int e = (h0 + hh) * d + nt * 8 + 2 * tig;
                    const float l = l_s[hh * AT_BQ + i];
                    float v0 = acc[x][2 * half] / l, v1 = acc[x][2 * half + 1] / l;
                    if (a.gate) {
                        const float* gt = a.gate + (size_t)(t0 + i) * a.gate_stride + e;
                        v0 *= 1.0f / (1.0f + expf(-gt[0]));
                        v1 *= 1.0f / (1.0f + expf(-gt[1]));
                    }
                    const unsigned pk = (unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(v0)) | ((unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(v1)) << 16);
                    *reinterpret_cast<unsigned*>(a.out + (size_t)(t0 + i) * nq + e) = pk;
                }
            }
        }
    }
}

// heads per block: the most that divide the head count with their outputs in a block's registers
static int at_heads_per_block(int nh, int d) {
    for (int hs = 16; hs >= 1; hs--)
        if (nh % hs == 0 && hs * d <= 1024) return hs;
    return 0;
}

template <int HSM>
static void at_launch(const AttnMixedTcArgs& a, dim3 grid, size_t smem, cudaStream_t s) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(attention_mixed_tc_kernel<HSM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    illm_launch(attention_mixed_tc_kernel<HSM>, grid, dim3(AT_THREADS), smem, s, a);
}

// bfloat16, head sizes that are multiples of 16 up to 1024, and a token tile's q with a key tile in shared memory
extern "C" int illm_attention_mixed_tc_supported(int nh, int nkv, int d) {
    if (nh <= 0 || nkv <= 0 || nh % nkv || d <= 0 || d % 16) return 0;
    const int hs = at_heads_per_block(nh, d);
    if (!hs) return 0;
    return at_plan(nh, nkv, d, hs).total <= 220 * 1024 ? 1 : 0;
}

// q [T, q_stride] and out [T, nh * d] bfloat16, kc the keys-only pages (bfloat16); cu_q [B + 1] the sequences' token
// offsets in the step, block_table [B, max_pages]; r1, r2, mix, gate as for illm_attention_mixed.
extern "C" int illm_attention_mixed_tc(const void* q, int q_stride, const void* kc, const int* block_table, int max_pages, const int* token_pos,
                                       const int* cu_q, int B, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale,
                                       const float* r1, const float* r2, const float* mix, const float* gate, int gate_stride, int n_sms,
                                       void* stream) {
    if (T <= 0 || B <= 0) return 0;
    if (!illm_attention_mixed_tc_supported(nh, nkv, d) || !q || !kc || !out || !cu_q || !token_pos || !block_table || q_stride % 8 ||
        ((r1 == nullptr) != (r2 == nullptr)) || page_size <= 0 || (gate && gate_stride % 2))
        return ILLM_ERR_BAD_ARG;
    // a short step would leave SMs without a block: fewer heads per block then, as long as the blocks still run all at
    // once (q k^T is repeated once more per halving)
    int hs = at_heads_per_block(nh, d);
    while (hs % 2 == 0 && 2LL * (T / AT_BQ + B) * (nh / hs) <= n_sms) hs /= 2;
    int page_shift = -1;
    for (int b = 0; b < 31; b++)
        if (page_size == (1 << b)) page_shift = b;
    AttnMixedTcArgs a{(const bf16*)q, q_stride, (const bf16*)kc, block_table, token_pos, cu_q, max_pages, page_size, page_shift, window, nh, nkv, d, hs, B,
                      scale, r1, r2, mix, gate, gate_stride, (bf16*)out};
    const size_t smem = at_plan(nh, nkv, d, hs).total;
    const dim3 grid((unsigned)(T / AT_BQ + B), (unsigned)(nh / hs));
    cudaStream_t s = (cudaStream_t)stream;
    if (hs <= 1) at_launch<1>(a, grid, smem, s);
    else if (hs <= 2) at_launch<2>(a, grid, smem, s);
    else if (hs <= 4) at_launch<4>(a, grid, smem, s);
    else if (hs <= 8) at_launch<8>(a, grid, smem, s);
    else at_launch<16>(a, grid, smem, s);
    return illm_launch_status();
}
