// Linear attention with a fixed decay per head, as a recurrence over a per-sequence state:
//
//   S_t = decay_h * S_{t-1} + k_t v_t^T          (S: [d, dv] float32 per sequence and head)
//   o_t = S_t^T q_t
//
// q, k (heads x d) and v (heads x dv) are columns of the packed float32 projection [T, ld]; on their
// way in they may pass an activation (silu), a rotate-half rotation of their first `rot` channels by
// the token's position (q and k only; table float32 [positions, rot / 2, 2]) and a constant factor
// on k, in that order.  The state lives in the cache's per-sequence storage, [slots, heads, d, dv]
// float32; a step loads it, runs its tokens in order and stores it, so prompts, portions of
// prompts and single tokens are the same code and carry the same bits from step to step.
//
// decay_prep_kernel: activation, rotation and factor, in place on the projection's q, k and v
// columns (one thread per rotated pair, so nothing is read after it was written).
//
// decay_scan_kernel: the columns of S evolve independently of one another (S[:, j] only ever meets
// v[j]), so a block owns one (sequence, head, group of columns) and a thread keeps its part of the
// state in registers for the whole step: R rows of C columns (16 rows of four columns up to head
// size 512, so that a token costs a thread few shared-memory reads per FMA), the rows of a column
// group dealt to LI neighbouring lanes (R LI >= d, rows beyond d are zeros).  The step's
// tokens come in tiles through two shared-memory buffers filled by cp.async, the next tile on its
// way while this one is used; every thread runs a tile's tokens one after the other without any
// synchronisation: 64 independent chains s = decay s + k v[j], its parts of o_t[j] = sum_i s q[i], and
// a fixed tree of shuffles over the LI lanes of the column group.  What bounds it is the float32 FMA rate
// and the latency of the chain, not memory; a prompt of one sequence fills heads x dv / (512 / LI)
// blocks (times its segments, see below).  The state is stored column by column ([slots, heads, dv, d]), so that a thread's rows are
// 16-byte pieces.
//
// The recurrence is float32 throughout, in the float32 mode and in the bfloat16 mode alike, because
// that is what such layers ask for (a state that is rounded to sixteen bits forgets).
//
// group_norm_gate_kernel: what follows the recurrence in such mixers: an RMS norm over groups of the
// concatenated heads (one group = all heads together, with a weight; or one group per head, without),
// times an activation of a gate projection (sigmoid or silu), rounded once to the activation dtype.
#include <type_traits>

#include "common.cuh"

#define DS_THREADS 128
#define DS_MAX_TILE 16
#define DS_U 4             // tokens whose reductions are interleaved

struct DecayScanArgs {
    float* x;
    int ld, q_off, k_off, v_off;
    int nh, d, dv;
    int qk_act, v_act;              // 0: none, 1: silu
    const float* cos_sin;
    int rot, n_pos;
    float k_scale;
    const float* decay;             // [nh]
    float* state;                   // [slots, nh, dv, d]
    const int *slots, *cu_q, *token_pos;
    float* out;                     // [T, nh * dv]
    int* err;
    int tile;                       // tokens staged at a time
    int vec;                        // 16-byte copies are possible
    int inline_prep;                // the scan prepares q, k, v itself while it stages them (steps of few tokens)
    int segments;                   // a sequence's tokens of this step in up to so many segments side by side (1: in order)
    float* seg_state;               // [B, segments, nh, dv, d]: what each segment's own tokens add to the state
    // per-token gates (decay_scan_kernel<.., GATED>): S_t = ga[t, h] S_(t-1) + gb[t, h] k_t v_t^T in place of the fixed decay
    const float *ga, *gb;           // [T, nh]
    int qk_div;                     // value head h reads query/key head h / qk_div (1: a head of its own)
    long long state_stride;         // floats from one slot's state to the next (nh * d * dv unless more is kept beside S)
    float* seg_gate;                // [B, segments, nh]: the product of a segment's gates a_t (GATED with segments)
};

__device__ __forceinline__ float act_of(float v, int act) {
    if (act == 1) return v / (1.0f + expf(-v));
    if (act == 2) return 1.0f / (1.0f + expf(-v));
    return v;
}

// One channel of a rotated pair: own * cos -+ other * sin, each operation rounded by itself, so that the
// preparation kernel and the scan's own staging give the same bits.
__device__ __forceinline__ float rot_val(float own, float other, float cs, float sn, bool lower) {
    return lower ? __fsub_rn(__fmul_rn(own, cs), __fmul_rn(other, sn)) : __fadd_rn(__fmul_rn(own, cs), __fmul_rn(other, sn));
}

__global__ void __launch_bounds__(128) decay_prep_kernel(DecayScanArgs a) {
    pdl_grid_sync();
    const int t = blockIdx.x, h = blockIdx.y;
    float* row = a.x + (size_t)t * a.ld;
    float* q = row + a.q_off + h * a.d;
    float* k = row + a.k_off + h * a.d;
    const int half = a.rot >> 1;
    int p = a.rot ? a.token_pos[t] : 0;
    if (a.rot && (p < 0 || p >= a.n_pos)) {
        if (threadIdx.x == 0) atomicExch(a.err, 3);
        p = 0;
    }
    for (int c = threadIdx.x; c < a.d; c += blockDim.x) {
        if (c < half) {
            const float cs = a.cos_sin[((size_t)p * half + c) * 2], sn = a.cos_sin[((size_t)p * half + c) * 2 + 1];
            const float q1 = act_of(q[c], a.qk_act), q2 = act_of(q[c + half], a.qk_act);
            const float k1 = act_of(k[c], a.qk_act), k2 = act_of(k[c + half], a.qk_act);
            q[c] = rot_val(q1, q2, cs, sn, true);
            q[c + half] = rot_val(q2, q1, cs, sn, false);
            k[c] = rot_val(k1, k2, cs, sn, true) * a.k_scale;
            k[c + half] = rot_val(k2, k1, cs, sn, false) * a.k_scale;
        } else if (c >= a.rot) {
            q[c] = act_of(q[c], a.qk_act);
            k[c] = act_of(k[c], a.qk_act) * a.k_scale;
        }
    }
    if (a.v_act) {
        float* v = row + a.v_off + h * a.dv;
        for (int c = threadIdx.x; c < a.dv; c += blockDim.x) v[c] = act_of(v[c], a.v_act);
    }
}

__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

// R rows x C columns of the state per thread, the rows of a column group over LI lanes.
//
// Segments: a long prompt of few sequences leaves most of the GPU idle, because a sequence's tokens
// are a chain.  With a.segments = P > 1 the chain is cut: pass 0 runs every segment of 16 k tokens on
// its own, the first from the sequence's state, the others from zero, and leaves each segment's final
// state in seg_state; pass 1 gives every later segment what it missed: the state at its start,
// S_in = sum over earlier segments r of decay^(tokens between) S_r, enters its tokens' outputs as
// o_t += decay^(t - t0 + 1) S_in^T q_t (no chain: the tokens are independent), and the last segment
// writes the sequence's state.  The sums then have another order than token by token, so the float32
// mode, which promises the same bits however a prompt is cut, never asks for segments.
//
// GATED: the decay is not one number per head but a gate per token and head, a_t, and the token's outer product
// enters with a second one, b_t: S_t = a_t S_(t-1) + b_t k_t v_t^T.  The two gates of a token travel with its staged
// row.  Value head h may share the queries and keys of head h / qk_div.  With segments, pass 0 also leaves the product
// of each segment's gates in seg_gate; pass 1 folds the earlier segments' states with these products
// (S_in = (..(S_0 G_1 + S_1) G_2 + ..) + S_(seg-1)) and gives token t the product of the gates from its segment's
// start up to itself in place of a power of the decay.
template <int R, int C, int LI, int PASS, bool GATED>
__global__ void __launch_bounds__(DS_THREADS) decay_scan_kernel(DecayScanArgs a) {
    pdl_grid_sync();
    extern __shared__ __align__(16) float sm[];
    constexpr int M = R / 4;                        // 16-byte pieces of q and k per thread
    constexpr int JW = C * (32 / LI);               // columns per warp
    constexpr int JB = JW * (DS_THREADS / 32);      // columns per block
    constexpr int DP = R * LI;                      // rows with padding
    constexpr int ROW = 2 * DP + JB + (GATED ? 4 : 0);      // floats of one staged token: q, k, v (and the two gates)
    constexpr int GATE_AT = 2 * DP + JB;
    const int P = a.segments;
    const int b = blockIdx.x / P, seg = blockIdx.x % P, h = blockIdx.y, j0 = blockIdx.z * JB;
    const int d = a.d, dv = a.dv;
    const int q0 = a.cu_q[b], q1 = a.cu_q[b + 1];
    const int seg_len = P > 1 ? (((q1 - q0 + P - 1) / P + 15) & ~15) : q1 - q0;      // whole tiles
    const int t0 = q0 + seg * seg_len, t1 = t0 + seg_len < q1 ? t0 + seg_len : q1;
    if (t0 >= t1) return;                                                           // a short sequence fills fewer segments
    const bool last_seg = t1 == q1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane % LI;
    const int jl = (warp * (32 / LI) + lane / LI) * C;      // first of this thread's columns within the block
    const int jn = dv - j0 < JB ? dv - j0 : JB;     // columns of this block that exist
    const float dec = GATED ? 1.f : a.decay[h];
    const int hq = h / a.qk_div;                    // the head whose queries and keys this head reads
    float* Sg = a.state + (size_t)a.slots[b] * a.state_stride + (size_t)h * d * dv;       // [dv][d]
    // row of register (m, r): m * 4 LI + 4 g + r, so that the LI lanes of a column group read 16-byte
    // pieces of q, k and the state that lie side by side
    float s[C][M][4];
    // one thread's elements of a state [dv][d] at `src`, times `mul`, plus `add` (what it holds already) if asked
    auto load_state = [&](const float* src, float mul, bool accumulate) {
#pragma unroll
        for (int c = 0; c < C; c++) {
            const int j = j0 + jl + c;
#pragma unroll
            for (int m = 0; m < M; m++) {
                const int i = m * 4 * LI + 4 * g;
                float v[4];
                if (a.vec && j < dv && i < d) {
                    const float4 v4 = *reinterpret_cast<const float4*>(src + (size_t)j * d + i);
                    v[0] = v4.x; v[1] = v4.y; v[2] = v4.z; v[3] = v4.w;
                } else {
#pragma unroll
                    for (int r = 0; r < 4; r++) v[r] = (j < dv && i + r < d) ? src[(size_t)j * d + i + r] : 0.f;
                }
#pragma unroll
                for (int r = 0; r < 4; r++) s[c][m][r] = accumulate ? fmaf(s[c][m][r], mul, v[r]) : v[r];
            }
        }
    };
    auto store_state = [&](float* dst) {
#pragma unroll
        for (int c = 0; c < C; c++) {
            const int j = j0 + jl + c;
#pragma unroll
            for (int m = 0; m < M; m++) {
                const int i = m * 4 * LI + 4 * g;
                if (a.vec && j < dv && i < d) {
                    *reinterpret_cast<float4*>(dst + (size_t)j * d + i) = make_float4(s[c][m][0], s[c][m][1], s[c][m][2], s[c][m][3]);
                } else {
#pragma unroll
                    for (int r = 0; r < 4; r++)
                        if (j < dv && i + r < d) dst[(size_t)j * d + i + r] = s[c][m][r];
                }
            }
        }
    };
    auto power = [&](int n) {       // decay^n by n multiplications (n is a segment's length at most)
        float f = 1.f;
        for (int i = 0; i < n; i++) f *= dec;
        return f;
    };
    float* seg_base = a.seg_state + ((size_t)b * P * a.nh + h) * (size_t)d * dv;      // + seg * nh * d * dv per segment
    const size_t seg_stride = (size_t)a.nh * d * dv;
    float factor = dec;             // pass 1: decay^(t - t0 + 1) of the token at hand (GATED: the product of the gates up to it)
    float* seg_gate = GATED && P > 1 ? a.seg_gate + (size_t)b * P * a.nh + h : nullptr;      // + seg * nh per segment
    if (PASS == 0) {
        if (seg == 0) {
            load_state(Sg, 0.f, false);
        } else {
#pragma unroll
            for (int c = 0; c < C; c++)
#pragma unroll
                for (int m = 0; m < M; m++)
#pragma unroll
                    for (int r = 0; r < 4; r++) s[c][m][r] = 0.f;
        }
    } else {
        if (seg == 0) {             // nothing to correct; a sequence of one segment still has to get its state
            if (last_seg) {
                load_state(seg_base, 0.f, false);
                store_state(Sg);
            }
            return;
        }
        const float dec_len = GATED ? 1.f : power(seg_len);
        load_state(seg_base, 0.f, false);
        for (int r = 1; r < seg; r++) load_state(seg_base + r * seg_stride, GATED ? seg_gate[(size_t)r * a.nh] : dec_len, true);
    }
    // rows beyond d and columns beyond dv stay zero in both buffers
    for (int idx = threadIdx.x; idx < 2 * a.tile * ROW; idx += DS_THREADS) sm[idx] = 0.f;
    __syncthreads();
    auto stage = [&](int buf, int tb) {
        const int n = t1 - tb < a.tile ? t1 - tb : a.tile;
        float* base = sm + buf * a.tile * ROW;
        if (a.inline_prep) {
            const int per = 2 * d + jn, half = a.rot >> 1;
            for (int idx = threadIdx.x; idx < n * per; idx += DS_THREADS) {
                const int tt = idx / per, c = idx - tt * per;
                const float* row = a.x + (size_t)(tb + tt) * a.ld;
                float* dst = base + tt * ROW;
                if (c < 2 * d) {
                    const bool is_k = c >= d;
                    const int e = is_k ? c - d : c;
                    const float* src = row + (is_k ? a.k_off : a.q_off) + hq * d;
                    float val = act_of(src[e], a.qk_act);
                    if (e < a.rot) {
                        int p = a.token_pos[tb + tt];
                        if (p < 0 || p >= a.n_pos) {
                            atomicExch(a.err, 3);
                            p = 0;
                        }
                        const bool lower = e < half;
                        const int jp = lower ? e : e - half;
                        const float cs = a.cos_sin[((size_t)p * half + jp) * 2], sn = a.cos_sin[((size_t)p * half + jp) * 2 + 1];
                        const float other = act_of(src[lower ? e + half : e - half], a.qk_act);
                        val = rot_val(val, other, cs, sn, lower);
                    }
                    dst[(is_k ? DP : 0) + e] = is_k ? val * a.k_scale : val;
                } else {
                    dst[2 * DP + c - 2 * d] = act_of(row[a.v_off + h * dv + j0 + c - 2 * d], a.v_act);
                }
            }
        } else if (a.vec) {
            const int cq = d >> 2, cv = jn >> 2, per = 2 * cq + cv;
            for (int idx = threadIdx.x; idx < n * per; idx += DS_THREADS) {
                const int tt = idx / per, c = idx - tt * per;
                const float* row = a.x + (size_t)(tb + tt) * a.ld;
                float* dst = base + tt * ROW;
                if (c < cq) cp_async16(dst + 4 * c, row + a.q_off + hq * d + 4 * c);
                else if (c < 2 * cq) cp_async16(dst + DP + 4 * (c - cq), row + a.k_off + hq * d + 4 * (c - cq));
                else cp_async16(dst + 2 * DP + 4 * (c - 2 * cq), row + a.v_off + h * dv + j0 + 4 * (c - 2 * cq));
            }
        } else {
            const int per = 2 * d + jn;
            for (int idx = threadIdx.x; idx < n * per; idx += DS_THREADS) {
                const int tt = idx / per, c = idx - tt * per;
                const float* row = a.x + (size_t)(tb + tt) * a.ld;
                float* dst = base + tt * ROW;
                if (c < d) dst[c] = row[a.q_off + hq * d + c];
                else if (c < 2 * d) dst[DP + c - d] = row[a.k_off + hq * d + c - d];
                else dst[2 * DP + c - 2 * d] = row[a.v_off + h * dv + j0 + c - 2 * d];
            }
        }
        if (GATED)
            for (int tt = threadIdx.x; tt < n; tt += DS_THREADS) {
                base[tt * ROW + GATE_AT] = a.ga[(size_t)(tb + tt) * a.nh + h];
                base[tt * ROW + GATE_AT + 1] = a.gb[(size_t)(tb + tt) * a.nh + h];
            }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto tokens = [&](auto group, const float* rowp, int t) {
        constexpr int U = decltype(group)::value;
        float p[U][C];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const float4* q4 = reinterpret_cast<const float4*>(rowp + u * ROW) + g;
            const float4* k4 = reinterpret_cast<const float4*>(rowp + u * ROW + DP) + g;
            const float* vp = rowp + u * ROW + 2 * DP + jl;
            float v[C];
            const float dec_t = GATED ? rowp[u * ROW + GATE_AT] : dec;
            const float put_t = GATED ? rowp[u * ROW + GATE_AT + 1] : 1.f;
            if (GATED && PASS == 0) factor *= dec_t;
#pragma unroll
            for (int c = 0; c < C; c++) {
                v[c] = GATED ? vp[c] * put_t : vp[c];
                p[u][c] = 0.f;
            }
#pragma unroll
            for (int m = 0; m < M; m++) {
                const float4 kk = k4[m * LI], qq = q4[m * LI];
#pragma unroll
                for (int c = 0; c < C; c++) {
                    if (PASS == 0) {
                        s[c][m][0] = fmaf(dec_t, s[c][m][0], kk.x * v[c]);
                        s[c][m][1] = fmaf(dec_t, s[c][m][1], kk.y * v[c]);
                        s[c][m][2] = fmaf(dec_t, s[c][m][2], kk.z * v[c]);
                        s[c][m][3] = fmaf(dec_t, s[c][m][3], kk.w * v[c]);
                    }
                    p[u][c] = fmaf(s[c][m][0], qq.x, p[u][c]);
                    p[u][c] = fmaf(s[c][m][1], qq.y, p[u][c]);
                    p[u][c] = fmaf(s[c][m][2], qq.z, p[u][c]);
                    p[u][c] = fmaf(s[c][m][3], qq.w, p[u][c]);
                }
            }
        }
        // the sums over the LI lanes of the column group, a fixed tree: while a lane holds several
        // columns, each step halves them (a lane keeps the lower half if its bit is clear and gets the
        // partner's part of that half); with one column left the steps are plain
        int first = 0;          // first column this lane still holds
        int nc = C, plain_bits = 0;
#pragma unroll
        for (int o = LI / 2; o >= 1; o >>= 1) {
            const bool up = (lane & o) != 0;
            if (nc > 1) {
                const int hf = nc / 2;
#pragma unroll
                for (int u = 0; u < U; u++)
#pragma unroll
                    for (int c = 0; c < C / 2; c++) {
                        if (c < hf) {
                            const float mine = up ? p[u][c + hf] : p[u][c];
                            const float theirs = up ? p[u][c] : p[u][c + hf];
                            p[u][c] = mine + __shfl_xor_sync(0xffffffffu, theirs, o);
                        }
                    }
                if (up) first += hf;
                nc = hf;
            } else {
#pragma unroll
                for (int u = 0; u < U; u++) p[u][0] += __shfl_xor_sync(0xffffffffu, p[u][0], o);
                plain_bits |= o;
            }
        }
        // lanes that differ only in the bits of the plain steps hold the same sum: one of them writes
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (GATED && PASS == 1) factor *= rowp[u * ROW + GATE_AT];
            if ((lane & plain_bits) == 0) {
                float* orow = a.out + (size_t)(t + u) * a.nh * dv + (size_t)h * dv + j0 + jl + first;
#pragma unroll
                for (int c = 0; c < C; c++)
                    if (c < nc && j0 + jl + first + c < dv) {
                        if (PASS == 0) orow[c] = p[u][c];
                        else orow[c] += factor * p[u][c];
                    }
            }
            if (PASS == 1 && !GATED) factor *= dec;
        }
    };
    if (t0 < t1) stage(0, t0);
    int buf = 0;
    for (int tb = t0; tb < t1; tb += a.tile, buf ^= 1) {
        const int n = t1 - tb < a.tile ? t1 - tb : a.tile;
        if (tb + a.tile < t1) {
            stage(buf ^ 1, tb + a.tile);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* base = sm + buf * a.tile * ROW;
        // tokens in groups of DS_U: the state chains run through the group's tokens in order, and the
        // group's reductions go level by level side by side, so that one token's shuffle latency is
        // spent on the others' shuffles
        int tt = 0;
        for (; tt + DS_U <= n; tt += DS_U) tokens(std::integral_constant<int, DS_U>(), base + tt * ROW, tb + tt);
        for (; tt < n; tt++) tokens(std::integral_constant<int, 1>(), base + tt * ROW, tb + tt);
        __syncthreads();        // the buffer is filled again by the tile after the next
    }
    if (PASS == 0) {
        store_state(P > 1 ? seg_base + seg * seg_stride : Sg);
        if (GATED && P > 1 && threadIdx.x == 0 && blockIdx.z == 0) seg_gate[(size_t)seg * a.nh] = factor;
    } else if (last_seg) {
        // the sequence's state: what came in, decayed over this segment, plus what the segment added
        load_state(seg_base + seg * seg_stride, GATED ? factor : power(t1 - t0), true);
        store_state(Sg);
    }
}

// head sizes up to 1024 (the rows of a column group over at most 32 lanes), any value size
extern "C" int illm_decay_scan_supported(int d, int dv) { return d > 0 && d <= 1024 && dv > 0 ? 1 : 0; }

template <int R, int C, int LI, bool GATED>
static void decay_launch(DecayScanArgs a, int B, cudaStream_t s) {
    constexpr int DP = R * LI, JB = C * (32 / LI) * (DS_THREADS / 32), ROW = 2 * DP + JB + (GATED ? 4 : 0);
    int tile = (int)(48 * 1024 / sizeof(float) / (2 * ROW));
    a.tile = tile > DS_MAX_TILE ? DS_MAX_TILE : (tile < 1 ? 1 : tile);
    const size_t smem = (size_t)2 * a.tile * ROW * sizeof(float);
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(decay_scan_kernel<R, C, LI, 0, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(decay_scan_kernel<R, C, LI, 1, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    const dim3 grid(B * a.segments, a.nh, (a.dv + JB - 1) / JB);
    illm_launch(decay_scan_kernel<R, C, LI, 0, GATED>, grid, dim3(DS_THREADS), smem, s, a);
    if (a.segments > 1) illm_launch(decay_scan_kernel<R, C, LI, 1, GATED>, grid, dim3(DS_THREADS), smem, s, a);
}

template <bool GATED>
static void decay_launch_for(DecayScanArgs a, int B, cudaStream_t s) {
    const int d = a.d;
    // 16 rows x 4 columns per thread (64 state elements in registers), the rows of a column group over d / 16 lanes:
    // a token costs a thread four 16-byte reads of q and of k, few enough to be on their way a token ahead,
    // and the lanes few shuffles.  (Measured against 4 x 4 over 32 lanes, 16 x 8 over 8 and 64 x 2 over 2 at
    // head size 128.)
    if (d <= 16) decay_launch<16, 4, 1, GATED>(a, B, s);
    else if (d <= 32) decay_launch<16, 4, 2, GATED>(a, B, s);
    else if (d <= 64) decay_launch<16, 4, 4, GATED>(a, B, s);
    else if (d <= 128) decay_launch<16, 4, 8, GATED>(a, B, s);
    else if (d <= 256) decay_launch<16, 4, 16, GATED>(a, B, s);
    else if (d <= 512) decay_launch<16, 4, 32, GATED>(a, B, s);
    else decay_launch<32, 2, 32, GATED>(a, B, s);
}

// x: the packed projection; its q, k and v columns are prepared in place (T rows).
extern "C" int illm_decay_scan(float* x, int T, int ld, int q_off, int k_off, int v_off, int nh, int d, int dv, int qk_act, int v_act,
                               const float* cos_sin, int rot, int n_pos, float k_scale, const float* decay, float* state, const int* slots,
                               const int* cu_q, const int* token_pos, float* out, int B, int* err, int segments, float* seg_state,
                               void* stream) {
    if (B <= 0 || T <= 0) return 0;
    if (segments < 1 || (segments > 1 && !seg_state) || (long long)B * segments > 0x7fffffff) return ILLM_ERR_BAD_ARG;
    if (nh <= 0 || d <= 0 || d > 1024 || dv <= 0 || nh > 65535 || rot < 0 || rot > d || (rot & 1) || (rot && !cos_sin) || !x || !state || !out)
        return ILLM_ERR_BAD_ARG;
    DecayScanArgs a{x, ld, q_off, k_off, v_off, nh, d, dv, qk_act, v_act, cos_sin, rot, n_pos, k_scale, decay, state, slots, cu_q, token_pos, out, err, 0, 0, 0, segments, seg_state,
                    nullptr, nullptr, 1, (long long)nh * d * dv, nullptr};
    a.vec = !((d | dv | ld | q_off | k_off | v_off) & 3) && !((uintptr_t)x & 15) && !((uintptr_t)state & 15);
    cudaStream_t s = (cudaStream_t)stream;
    // a step of few tokens (single tokens of a batch) is not worth a launch of its own for the preparation
    a.inline_prep = T <= 64 ? 1 : 0;
    if (!a.inline_prep && (qk_act || v_act || rot || k_scale != 1.0f)) illm_launch(decay_prep_kernel, dim3(T, nh), dim3(128), 0, s, a);
    decay_launch_for<false>(a, B, s);
    return illm_launch_status();
}

// The same recurrence with a gate pair per token and head (ga, gb: float32 [T, nh]) in place of the fixed decay, the
// q and k columns read as they are (nqk = nh / qk_div query/key heads).  state: the slots' S [nh, dv, d] blocks,
// `state_stride` floats apart.  segments > 1: seg_state [B, segments, nh, dv, d] and seg_gate [B, segments, nh] are scratch.
extern "C" int illm_gated_scan(const float* x, int T, int ld, int q_off, int k_off, int v_off, int nh, int qk_div, int d, int dv, const float* ga,
                               const float* gb, float* state, long long state_stride, const int* slots, const int* cu_q, float* out, int B,
                               int segments, float* seg_state, float* seg_gate, void* stream) {
    if (B <= 0 || T <= 0) return 0;
    if (segments < 1 || (segments > 1 && (!seg_state || !seg_gate)) || (long long)B * segments > 0x7fffffff) return ILLM_ERR_BAD_ARG;
    if (nh <= 0 || qk_div <= 0 || nh % qk_div || d <= 0 || d > 1024 || dv <= 0 || nh > 65535 || !x || !state || !out || !ga || !gb ||
        state_stride < (long long)nh * d * dv)
        return ILLM_ERR_BAD_ARG;
    DecayScanArgs a{const_cast<float*>(x), ld, q_off, k_off, v_off, nh, d, dv, 0, 0, nullptr, 0, 0, 1.f, nullptr, state, slots, cu_q, nullptr, out, nullptr,
                    0, 0, 0, segments, seg_state, ga, gb, qk_div, state_stride, seg_gate};
    a.vec = !((d | dv | ld | q_off | k_off | v_off) & 3) && !((uintptr_t)x & 15) && !((uintptr_t)state & 15) && !(state_stride & 3);
    a.inline_prep = 0;
    decay_launch_for<true>(a, B, (cudaStream_t)stream);
    return illm_launch_status();
}

// y[t, g, :] = u[t, g, :] / sqrt(mean_g(u^2) + eps) (* w) * act(gate[t, g, :]);  one block per (token, group);
// w covers the whole row or, shorter, repeats along it.  What is normed, u, is the recurrence's output o, optionally
// times a factor per token and head (row_scale [T, width / head]), plus a skip term skip_w[head] * skip_x[t, c]
// (skip_x: float32 rows skip_ld apart), and, with gate_first, already times the gate's activation (the gate then
// comes before the norm instead of after it).
struct GroupNormGateArgs {
    const float* o;
    int width, group;
    const float* w;
    int w_len;
    float eps;
    const float* gate;
    int gate_ld, gate_act, gate_first;
    const float* row_scale;
    int head;
    const float *skip_w, *skip_x;
    int skip_ld;
};

template <typename TA>
__global__ void __launch_bounds__(128) group_norm_gate_kernel(GroupNormGateArgs a, TA* __restrict__ y) {
    pdl_grid_sync();
    __shared__ float scratch[32];
    const int t = blockIdx.x, g0 = blockIdx.y * a.group;
    const float* row = a.o + (size_t)t * a.width + g0;
    const int n_heads = a.width / a.head;
    auto value = [&](int c) {
        float v = row[c];
        const int h = (g0 + c) / a.head;
        if (a.row_scale) v *= a.row_scale[(size_t)t * n_heads + h];
        if (a.skip_w) v = fmaf(a.skip_w[h], a.skip_x[(size_t)t * a.skip_ld + g0 + c], v);
        if (a.gate && a.gate_first) v *= act_of(a.gate[(size_t)t * a.gate_ld + g0 + c], a.gate_act);
        return v;
    };
    float ss = 0.f;
    for (int c = threadIdx.x; c < a.group; c += blockDim.x) {
        const float v = value(c);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)a.group + a.eps);
    for (int c = threadIdx.x; c < a.group; c += blockDim.x) {
        float v = value(c) * inv;
        if (a.w) v *= a.w[(g0 + c) % a.w_len];
        if (a.gate && !a.gate_first) v *= act_of(a.gate[(size_t)t * a.gate_ld + g0 + c], a.gate_act);
        y[(size_t)t * a.width + g0 + c] = from_f32<TA>(v);
    }
}

// w_len: the weight's length, the whole width or a divisor of it (a weight of one group's size is shared by the groups);
// head: columns per entry of row_scale and skip_w (0 when neither is given)
extern "C" int illm_group_norm_gate_ex(const float* o, int T, int width, int group, const float* w, int w_len, float eps, const float* gate,
                                       int gate_ld, int gate_act, int gate_first, const float* row_scale, int head, const float* skip_w,
                                       const float* skip_x, int skip_ld, void* y, int act_dtype, void* stream) {
    if (T <= 0) return 0;
    if (width <= 0 || group <= 0 || width % group || width / group > 65535 || !o || !y) return ILLM_ERR_BAD_ARG;
    if (w && (w_len <= 0 || width % w_len)) return ILLM_ERR_BAD_ARG;
    if ((row_scale || skip_w) && (head <= 0 || width % head)) return ILLM_ERR_BAD_ARG;
    if (skip_w && !skip_x) return ILLM_ERR_BAD_ARG;
    if (!w) w_len = width;
    if (head <= 0) head = width;
    GroupNormGateArgs a{o, width, group, w, w_len, eps, gate, gate_ld, gate_act, gate_first, row_scale, head, skip_w, skip_x, skip_ld};
    dim3 grid(T, width / group);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == ILLM_BF16) illm_launch(group_norm_gate_kernel<bf16>, grid, dim3(128), 0, s, a, (bf16*)y);
    else if (act_dtype == ILLM_F32) illm_launch(group_norm_gate_kernel<float>, grid, dim3(128), 0, s, a, (float*)y);
    else return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

extern "C" int illm_group_norm_gate(const float* o, int T, int width, int group, const float* w, int w_len, float eps, const float* gate,
                                    int gate_ld, int gate_act, void* y, int act_dtype, void* stream) {
    return illm_group_norm_gate_ex(o, T, width, group, w, w_len, eps, gate, gate_ld, gate_act, 0, nullptr, 0, nullptr, nullptr, 0, y, act_dtype, stream);
}
