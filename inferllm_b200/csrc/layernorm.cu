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

template <typename TO>
__global__ void __launch_bounds__(1024)
ln_sandwich_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ wb, const float* __restrict__ w,
                   TO* __restrict__ out, const int* __restrict__ rows, int H, float eps, int write_x) {
    pdl_grid_sync();
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* xr = x + (size_t)r * H;
    if (y) {
        const float* yr = y + (size_t)r * H;
        float s = 0.f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float v = yr[c];
            row[c] = v;
            s += v;
        }
        const float mean = block_sum(s, scratch) / (float)H;
        float q = 0.f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float dlt = row[c] - mean;
            q = fmaf(dlt, dlt, q);
        }
        const float inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)H + eps);
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float v = xr[c] + ((row[c] - mean) * inv) * wb[c];
            row[c] = v;
            if (write_x) xr[c] = v;
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) row[c] = xr[c];
    }
    if (!out) return;
    float s = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) s += row[c];
    const float mean = block_sum(s, scratch) / (float)H;
    float q = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float dlt = row[c] - mean;
        q = fmaf(dlt, dlt, q);
    }
    const float inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)H + eps);
    TO* o = out + (size_t)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = from_f32<TO>(((row[c] - mean) * inv) * w[c]);
}

// y, wb: nullptr for no addition; w, out: nullptr for the addition alone; rows: nullptr for rows 0 .. n_rows - 1
extern "C" int illm_layernorm_sandwich(float* x, const float* y, const float* wb, const float* w, void* out, int out_dtype, const int* rows,
                                       int n_rows, int H, float eps, int write_x, void* stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || !x || (y && !wb) || ((out != nullptr) != (w != nullptr))) return ILLM_ERR_BAD_ARG;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    // four elements per thread and pass for wide rows: a step of few rows is a few blocks, each bound by the latency of
    // its passes.  The block's size follows from the width alone, so a row's sums have one order in every step.
    const dim3 block(H >= 4096 ? 1024 : H >= 2048 ? 512 : 256);
    if (out_dtype == ILLM_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(ln_sandwich_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        illm_launch(ln_sandwich_kernel<bf16>, dim3(n_rows), block, smem, s, x, y, wb, w, (bf16*)out, rows, H, eps, write_x);
    } else if (out_dtype == ILLM_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(ln_sandwich_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        illm_launch(ln_sandwich_kernel<float>, dim3(n_rows), block, smem, s, x, y, wb, w, (float*)out, rows, H, eps, write_x);
    } else {
        return ILLM_ERR_BAD_ARG;
    }
    return illm_launch_status();
}
