// Layer norm with a weight and no bias, around the float32 residual stream of a block that norms a sublayer's
// input AND its output:
//
//   x[r] <- x[r] + ln(y[r]) * wb          (the sublayer's output y, normed, joins the stream; optional)
//   out[r] = ln(x[r]) * w                 (what the next sublayer reads; optional)
//   ln(v) = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps)
//
// in one kernel, because the second norm reads the row the first one has just made.  One block per row, the row in
// shared memory, every statistic in two passes (mean, then the mean squared deviation) with a fixed order of the
// sums, all float32.  `rows` (int32) gathers: only those rows are made, and x is then left as it is (the model's
// last norm, for the rows whose logits are wanted).
#include "common.cuh"

__device__ __forceinline__ void ln_store4(float* o, float a, float b, float c, float d) { *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d); }
__device__ __forceinline__ void ln_store4(bf16* o, float a, float b, float c, float d) {
    const unsigned lo = (unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(a)) | ((unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(b)) << 16);
    const unsigned hi = (unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(c)) | ((unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(d)) << 16);
    *reinterpret_cast<uint2*>(o) = make_uint2(lo, hi);
}

// V = 4: a thread takes four neighbouring channels at a time (the width a multiple of four); V = 1: any width.  A
// thread's part of a sum is taken in the order of its channels in both; which of the two runs follows from the
// width alone.
template <typename TO, int V>
__global__ void __launch_bounds__(1024)
ln_sandwich_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ wb, const float* __restrict__ w,
                   TO* __restrict__ out, const int* __restrict__ rows, int H, float eps, int write_x) {
    pdl_grid_sync();
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* xr = x + (size_t)r * H;
    const int first = threadIdx.x * V, step = blockDim.x * V;
    if (y) {
        const float* yr = y + (size_t)r * H;
        float s = 0.f;
        for (int c = first; c < H; c += step) {
            if (V == 4) {
                const float4 v = *reinterpret_cast<const float4*>(yr + c);
                *reinterpret_cast<float4*>(row + c) = v;
                s += v.x, s += v.y, s += v.z, s += v.w;
            } else {
                const float v = yr[c];
                row[c] = v;
                s += v;
            }
        }
        const float mean = block_sum(s, scratch) / (float)H;
        float q = 0.f;
        for (int c = first; c < H; c += step) {
#pragma unroll
            for (int i = 0; i < V; i++) {
                const float dlt = row[c + i] - mean;
                q = fmaf(dlt, dlt, q);
            }
        }
        const float inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)H + eps);
        for (int c = first; c < H; c += step) {
            if (V == 4) {
                const float4 xv = *reinterpret_cast<const float4*>(xr + c), wv = *reinterpret_cast<const float4*>(wb + c);
                float4 v;
                v.x = xv.x + ((row[c] - mean) * inv) * wv.x;
                v.y = xv.y + ((row[c + 1] - mean) * inv) * wv.y;
                v.z = xv.z + ((row[c + 2] - mean) * inv) * wv.z;
                v.w = xv.w + ((row[c + 3] - mean) * inv) * wv.w;
                *reinterpret_cast<float4*>(row + c) = v;
                if (write_x) *reinterpret_cast<float4*>(xr + c) = v;
            } else {
                const float v = xr[c] + ((row[c] - mean) * inv) * wb[c];
                row[c] = v;
                if (write_x) xr[c] = v;
            }
        }
    } else {
        for (int c = first; c < H; c += step) {
            if (V == 4) *reinterpret_cast<float4*>(row + c) = *reinterpret_cast<const float4*>(xr + c);
            else row[c] = xr[c];
        }
    }
    if (!out) return;
    float s = 0.f;
    for (int c = first; c < H; c += step) {
#pragma unroll
        for (int i = 0; i < V; i++) s += row[c + i];
    }
    const float mean = block_sum(s, scratch) / (float)H;
    float q = 0.f;
    for (int c = first; c < H; c += step) {
#pragma unroll
        for (int i = 0; i < V; i++) {
            const float dlt = row[c + i] - mean;
            q = fmaf(dlt, dlt, q);
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)H + eps);
    TO* o = out + (size_t)blockIdx.x * H;
    for (int c = first; c < H; c += step) {
        if (V == 4) {
            const float4 wv = *reinterpret_cast<const float4*>(w + c);
            ln_store4(o + c, ((row[c] - mean) * inv) * wv.x, ((row[c + 1] - mean) * inv) * wv.y, ((row[c + 2] - mean) * inv) * wv.z,
                      ((row[c + 3] - mean) * inv) * wv.w);
        } else {
            o[c] = from_f32<TO>(((row[c] - mean) * inv) * w[c]);
        }
    }
}

template <typename TO>
static void ln_launch(float* x, const float* y, const float* wb, const float* w, TO* out, const int* rows, int n_rows, int H, float eps, int write_x,
                      cudaStream_t s) {
    const size_t smem = (size_t)H * sizeof(float);
    // a thread per four channels up to 512 threads: a step of few rows is a few blocks, each bound by the latency of its
    // passes.  The block's size follows from the width alone, so a row's sums have one order in every step.
    if (H % 4 == 0) {
        const int threads = H >= 2048 ? 512 : H >= 1024 ? 256 : 128;
        if (smem > 48 * 1024) cudaFuncSetAttribute(ln_sandwich_kernel<TO, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        illm_launch((ln_sandwich_kernel<TO, 4>), dim3(n_rows), dim3(threads), smem, s, x, y, wb, w, out, rows, H, eps, write_x);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(ln_sandwich_kernel<TO, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        illm_launch((ln_sandwich_kernel<TO, 1>), dim3(n_rows), dim3(256), smem, s, x, y, wb, w, out, rows, H, eps, write_x);
    }
}

// y, wb: nullptr for no addition; w, out: nullptr for the addition alone; rows: nullptr for rows 0 .. n_rows - 1
extern "C" int illm_layernorm_sandwich(float* x, const float* y, const float* wb, const float* w, void* out, int out_dtype, const int* rows,
                                       int n_rows, int H, float eps, int write_x, void* stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || !x || (y && !wb) || ((out != nullptr) != (w != nullptr))) return ILLM_ERR_BAD_ARG;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == ILLM_BF16) ln_launch<bf16>(x, y, wb, w, (bf16*)out, rows, n_rows, H, eps, write_x, s);
    else if (out_dtype == ILLM_F32) ln_launch<float>(x, y, wb, w, (float*)out, rows, n_rows, H, eps, write_x, s);
    else return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}
