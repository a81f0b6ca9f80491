// Small element-wise kernels between matrix products.
//
// gated_act:    out[t, i] = act(gu[t, 2i]) * gu[t, 2i + 1]  for the activations that the fused silu kernels do not
//               cover (act 1: silu, 2: relu, 3: tanh-form gelu); the packed projection holds gate and up of an
//               output next to each other, as in swiglu.cu.
// take_columns: y[t, :] = x[t, off : off + n] of a float32 matrix with row stride ld, as a contiguous matrix of
//               the activation dtype (what a second, low-rank product reads).
// join_rows:    y[t, :] = [a[t, :], b[t, :]] of two float32 matrices of equal width, in the activation dtype.
#include "common.cuh"

__device__ __forceinline__ float gate_act_of(float v, int act) {
    if (act == 1) return v / (1.0f + expf(-v));
    if (act == 2) return fmaxf(v, 0.f);
    if (act == 3) return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return v;
}

template <typename TA>
__global__ void gated_act_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int I, long long n, int act) {
    pdl_grid_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / I;
    const int c = (int)(i - t * I);
    const float g = to_f32(gu[t * 2 * I + 2 * c]), u = to_f32(gu[t * 2 * I + 2 * c + 1]);
    out[i] = from_f32<TA>(gate_act_of(g, act) * u);
}

extern "C" int illm_gated_act(const void* gu, void* out, int act_dtype, int T, int I, int act, void* stream) {
    if (T <= 0 || I <= 0) return 0;
    if (act < 1 || act > 3) return ILLM_ERR_BAD_ARG;
    const long long n = (long long)T * I;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == ILLM_BF16) illm_launch(gated_act_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)gu, (bf16*)out, I, n, act);
    else if (act_dtype == ILLM_F32) illm_launch(gated_act_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)gu, (float*)out, I, n, act);
    else return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

template <typename TA>
__global__ void take_columns_kernel(const float* __restrict__ x, int ld, int off, int n_cols, TA* __restrict__ y, long long n) {
    pdl_grid_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / n_cols;
    y[i] = from_f32<TA>(x[t * ld + off + (i - t * n_cols)]);
}

extern "C" int illm_take_columns(const float* x, int ld, int off, int n_cols, void* y, int act_dtype, int T, void* stream) {
    if (T <= 0 || n_cols <= 0) return 0;
    const long long n = (long long)T * n_cols;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == ILLM_BF16) illm_launch(take_columns_kernel<bf16>, dim3(blocks), dim3(256), 0, s, x, ld, off, n_cols, (bf16*)y, n);
    else if (act_dtype == ILLM_F32) illm_launch(take_columns_kernel<float>, dim3(blocks), dim3(256), 0, s, x, ld, off, n_cols, (float*)y, n);
    else return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

template <typename TA>
__global__ void join_rows_kernel(const float* __restrict__ a, const float* __restrict__ b, int H, TA* __restrict__ y, long long n) {
    pdl_grid_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / (2 * H);
    const int c = (int)(i - t * 2 * H);
    y[i] = from_f32<TA>(c < H ? a[t * H + c] : b[t * H + c - H]);
}

extern "C" int illm_join_rows(const float* a, const float* b, int H, void* y, int act_dtype, int T, void* stream) {
    if (T <= 0 || H <= 0) return 0;
    const long long n = (long long)T * 2 * H;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == ILLM_BF16) illm_launch(join_rows_kernel<bf16>, dim3(blocks), dim3(256), 0, s, a, b, H, (bf16*)y, n);
    else if (act_dtype == ILLM_F32) illm_launch(join_rows_kernel<float>, dim3(blocks), dim3(256), 0, s, a, b, H, (float*)y, n);
    else return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

// add2_rmsnorm: resid[t, :] += d1[t, :] (+ d2[t, :]), all float32, and y[t, :] = resid[t, :] / sqrt(mean(resid^2) + eps) * w
// in the activation dtype: the two sublayer outputs of a parallel block folded into the next layer's norm.  A block
// per row, the row kept in shared memory between the two passes; the sum is (x + d1) + d2, as two separate additions give.
template <typename TY>
__global__ void __launch_bounds__(1024)
add2_rmsnorm_kernel(float* __restrict__ resid, const float* __restrict__ d1, const float* __restrict__ d2, const float* __restrict__ w,
                    TY* __restrict__ y, int H, float eps, int vec) {
    pdl_grid_sync();
    extern __shared__ __align__(16) float row_sm[];
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.f;
    if (vec) {          // rows of whole 16-byte pieces: a thread's loads are all in flight before its first store
        const float4* r4 = reinterpret_cast<const float4*>(resid + base);
        const float4* a4 = reinterpret_cast<const float4*>(d1 + base);
        const float4* b4 = d2 ? reinterpret_cast<const float4*>(d2 + base) : nullptr;
        for (int c = threadIdx.x; c < H / 4; c += blockDim.x) {
            float4 v = r4[c];
            const float4 a = a4[c];
            v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            if (b4) {
                const float4 b = b4[c];
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            reinterpret_cast<float4*>(resid + base)[c] = v;
            reinterpret_cast<float4*>(row_sm)[c] = v;
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float v = resid[base + c] + d1[base + c];
            if (d2) v += d2[base + c];
            resid[base + c] = v;
            row_sm[c] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) y[base + c] = from_f32<TY>((row_sm[c] * inv) * w[c]);
}

extern "C" int illm_add2_rmsnorm(float* resid, const float* d1, const float* d2, const float* w, void* y, int act_dtype, int T, int H, float eps,
                                 void* stream) {
    if (T <= 0 || H <= 0) return 0;
    if (!d1 || (size_t)H * sizeof(float) > 200 * 1024) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)H * sizeof(float);
    static bool raised = false;
    if (!raised) {
        cudaFuncSetAttribute(add2_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(add2_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        raised = true;
    }
    const int vec = (H & 3) == 0 && !((uintptr_t)resid & 15) && !((uintptr_t)d1 & 15) && !((uintptr_t)d2 & 15) ? 1 : 0;
    // a thread per 16-byte piece up to 1,024 threads (the block size depends on the width alone)
    int threads = ((vec ? H / 4 : H) + 31) / 32 * 32;
    threads = threads < 128 ? 128 : (threads > 1024 ? 1024 : threads);
    if (act_dtype == ILLM_BF16) illm_launch(add2_rmsnorm_kernel<bf16>, dim3(T), dim3(threads), smem, s, resid, d1, d2, w, (bf16*)y, H, eps, vec);
    else if (act_dtype == ILLM_F32) illm_launch(add2_rmsnorm_kernel<float>, dim3(T), dim3(threads), smem, s, resid, d1, d2, w, (float*)y, H, eps, vec);
    else return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

// scaled_add_rmsnorm: resid[t, :] += delta[t, :] * ls   (a sublayer's output through a per-channel layer scale,
// all float32), and, if w is given, y[t, :] = resid[t, :] / sqrt(mean(resid^2) + eps) * w in the activation dtype: the
// layer scale folded into the next norm.  A block per row, the row kept in shared memory between the two passes.
template <typename TY>
__global__ void __launch_bounds__(1024)
scaled_add_rmsnorm_kernel(float* __restrict__ resid, const float* __restrict__ delta, const float* __restrict__ ls,
                          const float* __restrict__ w, TY* __restrict__ y, int H, float eps, int vec) {
    pdl_grid_sync();
    extern __shared__ __align__(16) float row_sm[];
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.f;
    if (vec) {          // rows of whole 16-byte pieces: a thread's loads are all in flight before its first store
        const float4* r4 = reinterpret_cast<const float4*>(resid + base);
        const float4* d4 = reinterpret_cast<const float4*>(delta + base);
        const float4* l4 = reinterpret_cast<const float4*>(ls);
        for (int c = threadIdx.x; c < H / 4; c += blockDim.x) {
            float4 v = r4[c];
            const float4 dl = d4[c], f = l4[c];
            v.x = fmaf(dl.x, f.x, v.x);
            v.y = fmaf(dl.y, f.y, v.y);
            v.z = fmaf(dl.z, f.z, v.z);
            v.w = fmaf(dl.w, f.w, v.w);
            reinterpret_cast<float4*>(resid + base)[c] = v;
            reinterpret_cast<float4*>(row_sm)[c] = v;
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float v = fmaf(delta[base + c], ls[c], resid[base + c]);
            resid[base + c] = v;
            row_sm[c] = v;
            ss = fmaf(v, v, ss);
        }
    }
    if (!w) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) y[base + c] = from_f32<TY>((row_sm[c] * inv) * w[c]);
}

extern "C" int illm_scaled_add_rmsnorm(float* resid, const float* delta, const float* ls, const float* w, void* y, int act_dtype,
                                       int T, int H, float eps, void* stream) {
    if (T <= 0 || H <= 0) return 0;
    if (!delta || !ls || (w && !y) || (size_t)H * sizeof(float) > 200 * 1024) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)H * sizeof(float);
    static bool raised = false;
    if (!raised) {
        cudaFuncSetAttribute(scaled_add_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(scaled_add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        raised = true;
    }
    const int vec = (H & 3) == 0 && !((uintptr_t)resid & 15) && !((uintptr_t)delta & 15) && !((uintptr_t)ls & 15) ? 1 : 0;
    int threads = ((vec ? H / 4 : H) + 31) / 32 * 32;       // the block size depends on the width alone
    threads = threads < 128 ? 128 : (threads > 1024 ? 1024 : threads);
    if (act_dtype == ILLM_BF16) illm_launch(scaled_add_rmsnorm_kernel<bf16>, dim3(T), dim3(threads), smem, s, resid, delta, ls, w, (bf16*)y, H, eps, vec);
    else if (act_dtype == ILLM_F32) illm_launch(scaled_add_rmsnorm_kernel<float>, dim3(T), dim3(threads), smem, s, resid, delta, ls, w, (float*)y, H, eps, vec);
    else return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

// add_bias: y[t, c] += b[c] (b float32), in place, for a projection with a bias whose product kernel has no bias epilogue
template <typename TA>
__global__ void add_bias_kernel(TA* __restrict__ y, const float* __restrict__ b, int H, long long n) {
    pdl_grid_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = from_f32<TA>(to_f32(y[i]) + b[i % H]);
}
extern "C" int illm_add_bias(void* y, int dtype, const float* b, int T, int H, void* stream) {
    if (T <= 0 || H <= 0) return 0;
    if (!y || !b) return ILLM_ERR_BAD_ARG;
    const long long n = (long long)T * H;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ILLM_BF16) illm_launch(add_bias_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (bf16*)y, b, H, n);
    else if (dtype == ILLM_F32) illm_launch(add_bias_kernel<float>, dim3(blocks), dim3(256), 0, s, (float*)y, b, H, n);
    else return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}
