// A short causal convolution over time, one filter per channel, across the steps of a sequence:
//
//   y_t[c] = act( sum_j w[c, j] * x_(t - taps + 1 + j)[c] + bias[c] )  (+ x_t[c], the residual form)
//
// x are channels [x_off, x_off + C) of the float32 rows [T, ldx] of one step; the rows before the step's first one
// come from the sequence's state, the last taps - 1 input rows [taps - 1, C] (oldest first, zero for a new
// sequence) at `state_off` of the sequence's slot.  The taps are added oldest first whether a row comes from the
// step or from the state, so the result does not depend on how a prompt was cut.  short_conv_state_kernel renews
// the state from the step's rows afterwards (a launch of its own: the convolution reads the old one).
#include <stdint.h>

#include "common.cuh"

struct ShortConvArgs {
    const float* x;
    int ldx, x_off, C, taps;
    const float *w, *bias;
    int act, residual;
    float* state;
    long long state_stride, state_off;
    const int *slots, *cu_q, *token_seq;
    void* out;
    int ldo, o_off;
};

__device__ __forceinline__ void sc_store(float* o, const float* v, int n) {
    if (n == 4) *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
    else o[0] = v[0];
}
__device__ __forceinline__ void sc_store(bf16* o, const float* v, int n) {
    if (n == 4) {
        const unsigned lo = (unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(v[0])) | ((unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(v[1])) << 16);
        const unsigned hi = (unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(v[2])) | ((unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(v[3])) << 16);
        *reinterpret_cast<uint2*>(o) = make_uint2(lo, hi);
    } else {
        o[0] = __float2bfloat16_rn(v[0]);
    }
}

// V channels per thread (4 where the widths, offsets and addresses are multiples of four, else 1); a channel's
// arithmetic is the same in both.
template <typename TO, int V>
__global__ void __launch_bounds__(256) short_conv_kernel(ShortConvArgs a) {
    pdl_grid_sync();
    const int t = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    if (c >= a.C) return;
    const int b = a.token_seq[t], t0 = a.cu_q[b], i = t - t0, n_old = a.taps - 1;
    // one tap keeps no rows: such a call has no state and no slots
    const float* st = n_old > 0 ? a.state + (size_t)a.slots[b] * a.state_stride + a.state_off : nullptr;
    float acc[V];
#pragma unroll
    for (int k = 0; k < V; k++) acc[k] = 0.f;
    for (int j = 0; j < a.taps; j++) {
        const int s = i - n_old + j;
        const float* src = s >= 0 ? a.x + (size_t)(t0 + s) * a.ldx + a.x_off + c : st + (size_t)(n_old + s) * a.C + c;
        float v[V];
        if (V == 4) {
            const float4 f = *reinterpret_cast<const float4*>(src);
            v[0] = f.x, v[V > 1 ? 1 : 0] = f.y, v[V > 2 ? 2 : 0] = f.z, v[V > 3 ? 3 : 0] = f.w;
        } else {
            v[0] = src[0];
        }
#pragma unroll
        for (int k = 0; k < V; k++) acc[k] = fmaf(a.w[(size_t)(c + k) * a.taps + j], v[k], acc[k]);
    }
#pragma unroll
    for (int k = 0; k < V; k++) {
        if (a.bias) acc[k] += a.bias[c + k];
        if (a.act == 1) acc[k] = acc[k] / (1.0f + expf(-acc[k]));
        if (a.residual) acc[k] += a.x[(size_t)t * a.ldx + a.x_off + c + k];
    }
    sc_store((TO*)a.out + (size_t)t * a.ldo + a.o_off + c, acc, V);
}

// the last taps - 1 rows of (old state rows, then the step's rows), per sequence; a thread owns a channel and goes
// through the rows oldest first, so that it reads an old row before it overwrites it
__global__ void __launch_bounds__(256) short_conv_state_kernel(ShortConvArgs a) {
    pdl_grid_sync();
    const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const int t0 = a.cu_q[b], n = a.cu_q[b + 1] - t0, n_old = a.taps - 1;
    float* st = a.state + (size_t)a.slots[b] * a.state_stride + a.state_off;
    for (int r = 0; r < n_old; r++) {
        const int idx = n + r;      // place in (old rows, step rows)
        st[(size_t)r * a.C + c] = idx < n_old ? st[(size_t)idx * a.C + c] : a.x[(size_t)(t0 + idx - n_old) * a.ldx + a.x_off + c];
    }
}

// out_dtype: 0 float32, 1 bfloat16.  update_state != 0: the state is renewed after the convolution.
extern "C" int illm_short_conv(const float* x, int T, int ldx, int x_off, int C, int taps, const float* w, const float* bias, int act, int residual,
                               float* state, long long state_stride, long long state_off, const int* slots, const int* cu_q,
                               const int* token_seq, int B, void* out, int out_dtype, int ldo, int o_off, int update_state, void* stream) {
    if (T <= 0 || B <= 0) return 0;
    if (C <= 0 || taps < 1 || !x || !w || !out || (taps > 1 && (!state || !slots)) || T > 0x7fffffff / 2) return ILLM_ERR_BAD_ARG;
    ShortConvArgs a{x, ldx, x_off, C, taps, w, bias, act, residual, state, state_stride, state_off, slots, cu_q, token_seq, out, ldo, o_off};
    cudaStream_t s = (cudaStream_t)stream;
    const int by = (C + 255) / 256;
    if (by > 65535) return ILLM_ERR_BAD_ARG;
    if (out_dtype != ILLM_BF16 && out_dtype != ILLM_F32) return ILLM_ERR_BAD_ARG;
    const size_t osz = out_dtype == ILLM_BF16 ? 2 : 4;
    const bool by4 = C % 4 == 0 && ldx % 4 == 0 && x_off % 4 == 0 && ldo % 4 == 0 && o_off % 4 == 0 && (uintptr_t)x % 16 == 0 &&
                     (uintptr_t)out % (4 * osz) == 0 && (taps == 1 || (state_stride % 4 == 0 && state_off % 4 == 0 && (uintptr_t)state % 16 == 0));
    if (by4) {
        const dim3 grid(T, (C / 4 + 127) / 128);
        if (out_dtype == ILLM_BF16) illm_launch((short_conv_kernel<bf16, 4>), grid, dim3(128), 0, s, a);
        else illm_launch((short_conv_kernel<float, 4>), grid, dim3(128), 0, s, a);
    } else {
        if (out_dtype == ILLM_BF16) illm_launch((short_conv_kernel<bf16, 1>), dim3(T, by), dim3(256), 0, s, a);
        else illm_launch((short_conv_kernel<float, 1>), dim3(T, by), dim3(256), 0, s, a);
    }
    if (update_state && taps > 1) illm_launch(short_conv_state_kernel, dim3(B, by), dim3(256), 0, s, a);
    return illm_launch_status();
}
