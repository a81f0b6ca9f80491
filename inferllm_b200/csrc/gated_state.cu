// The per-token gates of two recurrences that share one form of state update,
//
//   S_t = a_t S_(t-1) + b_t k_t v_t^T,    o_t = S_t^T q_t          (per head; a_t, b_t scalars)
//
// which decay_state.cu runs with its per-token gates (decay_scan_kernel<.., GATED>).  Both kernels here turn a
// layer's raw projections into a_t and b_t, float32 [T, heads], in accurate float32 arithmetic.
//
// mlstm_gates_kernel: the matrix memory with exponential gating, stabilised by a running maximum m that starts at 0:
//   i_t = cap tanh((z_i + b_i) / cap),  f_t = logsigmoid(cap tanh((z_f + b_f) / cap))
//   m_t = max(f_t + m_(t-1), i_t),  a_t = exp(f_t + m_(t-1) - m_t),  b_t = exp(i_t - m_t)
//   n_t = a_t n_(t-1) + b_t k_t,  scale_t = q_scale / (max(|q_scale n_t . q_t|, exp(-m_t)) + 1e-6)
// so that the layer's output is scale_t * S_t^T q_t with the raw q.  m and n are a chain over the sequence's tokens:
// a block owns one (sequence, head), keeps n over its threads, and goes through the tokens in order; the two gates
// (the tanh, the logarithm) are made for 32 tokens at a time, a token per lane, outside the chain.  n [heads, d] and
// m [heads] live in the sequence's state at n_off and m_off.
//
// ssm_gates_kernel: the selective state space with a scalar decay per head:
//   dt = softplus(z + dt_bias),  a_t = exp(-exp(A_log) dt),  b_t = dt
#include "common.cuh"

struct MlstmGateArgs {
    const float* x;
    int ld, q_off, k_off, i_off, f_off;
    const float *i_bias, *f_bias;
    float cap, q_scale;
    int nh, d;
    float* state;
    long long state_stride, n_off, m_off;
    const int *slots, *cu_q;
    float *ga, *gb, *scale;
    int B;
};

__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// A block owns one (sequence, head); warp w owns channels [32 w, 32 w + 32) of n, a channel per lane, so a head of d
// channels takes ceil(d / 32) warps and every warp has G tokens' rows on their way at a time (nothing of them hangs
// on the chain: the chain itself is one multiply-add per token).  Every warp runs the chain of m by itself (the same
// bits in all of them).  Nothing in a link of the chain crosses lanes, so that the compiler can overlap the links of
// G tokens: the gates of a block of 32 tokens (the tanh, the logarithm; a token per lane) go through shared memory,
// and a token's n . q is summed afterwards, for 32 tokens at once: each lane leaves its product in shared memory,
// warp w adds its 32 channels of token `lane` in the order of the channels, and the first warp adds the warps' sums
// in the order of the warps.
template <int MAXT, int G>
__global__ void __launch_bounds__(MAXT) mlstm_gates_kernel(MlstmGateArgs a) {
    pdl_grid_sync();
    extern __shared__ float mg_prod[];   // [32 tokens][32 nw + 1]: a token's products, a channel each
    __shared__ float part[32][33];       // [token of the block of 32][warp]
    __shared__ float ig_s[MAXT / 32][32], fg_s[MAXT / 32][32];      // [warp][token]: every warp keeps the gates for itself
    __shared__ float ga_s[32], gb_s[32], em_s[32];
    const int unit = blockIdx.x, lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5, pld = 32 * nw + 1;
    const int b = unit / a.nh, h = unit - b * a.nh;
    const int t0 = a.cu_q[b], t1 = a.cu_q[b + 1];
    float* st = a.state + (size_t)a.slots[b] * a.state_stride;
    const int c = w * 32 + lane;
    const bool has = c < a.d;
    float n = has ? st[a.n_off + (size_t)h * a.d + c] : 0.f;
    float m = st[a.m_off + h];
    const float bi = a.i_bias ? a.i_bias[h] : 0.f, bf = a.f_bias ? a.f_bias[h] : 0.f;
    const float* kcol = a.x + a.k_off + h * a.d + (has ? c : 0);
    const float* qcol = a.x + a.q_off + h * a.d + (has ? c : 0);
    // The rows of G tokens are asked for one group ahead of their use, and a block's two gate logits one block
    // ahead; places beyond the step's last token read its last row again.
    float kA[G], qA[G], kB[G], qB[G];
    auto fetch = [&](int first, float* kk, float* qq) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            const size_t r = (size_t)(first + g < t1 ? first + g : t1 - 1) * a.ld;
            kk[g] = has ? kcol[r] : 0.f;
            qq[g] = has ? qcol[r] : 0.f;
        }
    };
    auto links = [&](int j0, const float* kk, const float* qq) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            const int j = j0 + g;
            const float ig = ig_s[w][j], fg = fg_s[w][j];
            const float m_new = fmaxf(fg + m, ig);
            const float ga = expf(fg + m - m_new), gb = expf(ig - m_new), em = expf(-m_new);
            n = fmaf(ga, n, gb * kk[g]);
            mg_prod[j * pld + c] = n * qq[g];
            m = m_new;
            if (threadIdx.x == 0) {
                ga_s[j] = ga;
                gb_s[j] = gb;
                em_s[j] = em;
            }
        }
    };
    if (t1 <= t0) return;
    fetch(t0, kA, qA);
    float zi, zf;
    {
        const float* row = a.x + (size_t)(t0 + lane < t1 ? t0 + lane : t1 - 1) * a.ld;
        zi = row[a.i_off + h], zf = row[a.f_off + h];
    }
    for (int tb = t0; tb < t1; tb += 32) {
        const int cnt = t1 - tb < 32 ? t1 - tb : 32;
        // places beyond the step's last token get gates that leave m and n as they are (f = 0, i = -inf: a = 1,
        // b = 0), so that the links of the chain need no branch
        float ig_l = -INFINITY, fg_l = 0.f;
        if (lane < cnt) {
            ig_l = a.cap * tanhf((zi + bi) / a.cap);
            fg_l = log_sigmoid_f(a.cap * tanhf((zf + bf) / a.cap));
        }
        {
            const float* row = a.x + (size_t)(tb + 32 + lane < t1 ? tb + 32 + lane : t1 - 1) * a.ld;
            zi = row[a.i_off + h], zf = row[a.f_off + h];
        }
        ig_s[w][lane] = ig_l;
        fg_s[w][lane] = fg_l;
        __syncwarp();
#pragma unroll
        for (int j0 = 0; j0 < 32; j0 += 2 * G) {
            fetch(tb + j0 + G, kB, qB);
            links(j0, kA, qA);
            fetch(tb + j0 + 2 * G, kA, qA);
            links(j0 + G, kB, qB);
        }
        __syncthreads();
        if (lane < cnt) {
            const float* pr = mg_prod + lane * pld + w * 32;
            float dot = 0.f;
#pragma unroll 8
            for (int i = 0; i < 32; i++) dot += pr[i];
            part[lane][w] = dot;
        }
        __syncthreads();
        if (w == 0 && lane < cnt) {
            float dot = 0.f;
            for (int i = 0; i < nw; i++) dot += part[lane][i];
            dot *= a.q_scale;
            const size_t o = (size_t)(tb + lane) * a.nh + h;
            a.ga[o] = ga_s[lane];
            a.gb[o] = gb_s[lane];
            a.scale[o] = a.q_scale / (fmaxf(fabsf(dot), em_s[lane]) + 1e-6f);
        }
        __syncthreads();        // the block's scratch is free again
    }
    if (has) st[a.n_off + (size_t)h * a.d + c] = n;
    if (threadIdx.x == 0) st[a.m_off + h] = m;
}

extern "C" int illm_mlstm_gates(const float* x, int T, int ld, int q_off, int k_off, int i_off, int f_off, const float* i_bias, const float* f_bias,
                                float cap, float q_scale, int nh, int d, float* state, long long state_stride, long long n_off, long long m_off,
                                const int* slots, const int* cu_q, float* ga, float* gb, float* scale, int B, void* stream) {
    if (T <= 0 || B <= 0) return 0;
    if (nh <= 0 || d <= 0 || d > 1024 || !(cap > 0.f) || !x || !state || !ga || !gb || !scale) return ILLM_ERR_BAD_ARG;
    MlstmGateArgs a{x, ld, q_off, k_off, i_off, f_off, i_bias, f_bias, cap, q_scale, nh, d, state, state_stride, n_off, m_off, slots, cu_q, ga, gb, scale, B};
    const int nw = (d + 31) / 32;
    const size_t smem = (size_t)32 * (32 * nw + 1) * sizeof(float);
    if (nw <= 8) {
        illm_launch((mlstm_gates_kernel<256, 16>), dim3((unsigned)B * nh), dim3(32 * nw), smem, (cudaStream_t)stream, a);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(mlstm_gates_kernel<1024, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        illm_launch((mlstm_gates_kernel<1024, 8>), dim3((unsigned)B * nh), dim3(32 * nw), smem, (cudaStream_t)stream, a);
    }
    return illm_launch_status();
}

__global__ void ssm_gates_kernel(const float* __restrict__ x, int ld, int dt_off, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                 int nh, float* __restrict__ ga, float* __restrict__ gb, long long n) {
    pdl_grid_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / nh;
    const int h = (int)(i - t * nh);
    const float z = x[(size_t)t * ld + dt_off + h] + (dt_bias ? dt_bias[h] : 0.f);
    const float dt = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
    ga[i] = expf(-expf(a_log[h]) * dt);
    gb[i] = dt;
}

extern "C" int illm_ssm_gates(const float* x, int T, int ld, int dt_off, const float* dt_bias, const float* a_log, int nh, float* ga, float* gb,
                              void* stream) {
    if (T <= 0) return 0;
    if (nh <= 0 || !x || !a_log || !ga || !gb) return ILLM_ERR_BAD_ARG;
    const long long n = (long long)T * nh;
    illm_launch(ssm_gates_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, x, ld, dt_off, dt_bias, a_log, nh, ga, gb, n);
    return illm_launch_status();
}
