// Short causal convolutions over time, one filter per channel, for steps that hold any
// mix of prompt portions and decoded tokens:
//
//   y_t[c] = (add_input ? u_t[c] : 0) + sum_{j < taps} w[c, j] * u_{t - taps + 1 + j}[c]
//
// with u = 0 before a sequence's start.  The taps - 1 inputs before an entry's first row
// are the request's state: 32-bit [taps - 1, C] per slot, oldest first (a fresh slot is
// all zeros, which is the sequence's start).  causal_conv reads the state, conv_state
// brings it up to date in a launch of its own once every row has read it.  Sums in
// 32-bit in tap order, one rounding at the store; a token's result does not depend on
// how its sequence was cut into steps.
#include "common.cuh"

using namespace ib;

#define IB_CONV_MAX_TAPS 16

template <typename T, typename TO>
__global__ void causal_conv_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ w,
                                   const float* __restrict__ state, long long state_stride,
                                   const int* __restrict__ row_entry, const int* __restrict__ cu_rows,
                                   const int* __restrict__ slot_ids, TO* __restrict__ out, int out_stride, int C,
                                   int taps, int add_input) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int e = row_entry[row];
    const int first = cu_rows[e];
    const int idx = row - first;  // place among the entry's rows
    const float* st = state + (long long)slot_ids[e] * state_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int src = idx - (taps - 1) + j;  // negative: in the state
            const float u = src >= 0 ? to_f32(x[(size_t)(first + src) * x_stride + c])
                                     : st[(size_t)(taps - 1 + src) * C + c];
            acc = fmaf(w[(size_t)c * taps + j], u, acc);
        }
        if (add_input) acc += to_f32(x[(size_t)row * x_stride + c]);
        out[(size_t)row * out_stride + c] = from_f32<TO>(acc);
    }
}

// The same for bfloat16 rows eight channels a thread (16-byte loads and stores), for channel counts and
// row strides that are multiples of 8 and 16-byte aligned rows; the same operations in the same order.
__global__ void causal_conv_vec8_kernel(const bf16* __restrict__ x, int x_stride, const float* __restrict__ w,
                                        const float* __restrict__ state, long long state_stride,
                                        const int* __restrict__ row_entry, const int* __restrict__ cu_rows,
                                        const int* __restrict__ slot_ids, bf16* __restrict__ out, int out_stride, int C,
                                        int taps, int add_input) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int e = row_entry[row];
    const int first = cu_rows[e];
    const int idx = row - first;
    const float* st = state + (long long)slot_ids[e] * state_stride;
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8; c < C; c += gridDim.y * blockDim.x * 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        float u[8];
        for (int j = 0; j < taps; ++j) {
            const int src = idx - (taps - 1) + j;
            if (src >= 0) {
                const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)(first + src) * x_stride + c);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(h[i]);
                    u[2 * i] = f.x;
                    u[2 * i + 1] = f.y;
                }
            } else {
                const float4 a = *reinterpret_cast<const float4*>(st + (size_t)(taps - 1 + src) * C + c);
                const float4 b = *reinterpret_cast<const float4*>(st + (size_t)(taps - 1 + src) * C + c + 4);
                u[0] = a.x; u[1] = a.y; u[2] = a.z; u[3] = a.w;
                u[4] = b.x; u[5] = b.y; u[6] = b.z; u[7] = b.w;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[(size_t)(c + i) * taps + j], u[i], acc[i]);
        }
        if (add_input) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)row * x_stride + c);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(h[i]);
                acc[2 * i] += f.x;
                acc[2 * i + 1] += f.y;
            }
        }
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        *reinterpret_cast<uint4*>(out + (size_t)row * out_stride + c) = o;
    }
}

// x: [n_rows, C] with row stride x_stride, of dtype `dtype` (0 = f32, 1 = bf16); out the same
// dtype; w: float32 [C, taps]; state: float32, slot s at state + s * state_stride.
IB_EXPORT int ib_causal_conv(const void* x, int x_stride, int dtype, const float* w, const float* state,
                             long long state_stride, const int* row_entry, const int* cu_rows, const int* slot_ids,
                             void* out, int out_stride, int n_rows, int C, int taps, int add_input, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x || !w || !row_entry || !cu_rows || !slot_ids || !out || C <= 0 || x_stride < C || out_stride < C)
        return IB_ERR_BAD_ARG;
    if (taps < 1 || taps > IB_CONV_MAX_TAPS) return IB_ERR_TOO_LARGE;
    if (taps > 1 && (!state || state_stride < (long long)(taps - 1) * C)) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 128;
    const dim3 grid(n_rows, min(64, (C + threads - 1) / threads));
    cudaError_t le;
    if (dtype == 0)
        le = launch_kernel(causal_conv_kernel<float, float>, grid, dim3(threads), 0, s, (const float*)x, x_stride, w,
                           state, state_stride, row_entry, cu_rows, slot_ids, (float*)out, out_stride, C, taps,
                           add_input);
    else if (dtype == 1 && C % 8 == 0 && x_stride % 8 == 0 && out_stride % 8 == 0 && ((uintptr_t)x & 15) == 0 &&
             ((uintptr_t)out & 15) == 0 && (taps == 1 || (((uintptr_t)state & 15) == 0 && state_stride % 4 == 0)))
        le = launch_kernel(causal_conv_vec8_kernel, dim3(n_rows, min(64, (C / 8 + threads - 1) / threads)), dim3(threads), 0,
                           s, (const bf16*)x, x_stride, w, state, state_stride, row_entry, cu_rows, slot_ids, (bf16*)out,
                           out_stride, C, taps, add_input);
    else if (dtype == 1)
        le = launch_kernel(causal_conv_kernel<bf16, bf16>, grid, dim3(threads), 0, s, (const bf16*)x, x_stride, w,
                           state, state_stride, row_entry, cu_rows, slot_ids, (bf16*)out, out_stride, C, taps,
                           add_input);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// The state after the step: the last taps - 1 inputs of (old state ++ the entry's rows).
// An entry without rows leaves its slot alone.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state,
                                         long long state_stride, const int* __restrict__ cu_rows,
                                         const int* __restrict__ slot_ids, int C, int taps) {
    pdl_trigger();
    pdl_wait();
    const int e = blockIdx.x;
    const int first = cu_rows[e], n = cu_rows[e + 1] - first;
    if (n <= 0) return;
    float* st = state + (long long)slot_ids[e] * state_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float nv[IB_CONV_MAX_TAPS];
        for (int k = 0; k < taps - 1; ++k) {
            const int idx = n - (taps - 1 - k);  // place among the entry's rows; negative: in the old state
            nv[k] = idx >= 0 ? to_f32(x[(size_t)(first + idx) * x_stride + c]) : st[(size_t)(taps - 1 + idx) * C + c];
        }
        for (int k = 0; k < taps - 1; ++k) st[(size_t)k * C + c] = nv[k];
    }
}

IB_EXPORT int ib_conv_state_update(const void* x, int x_stride, int dtype, float* state, long long state_stride,
                                   const int* cu_rows, const int* slot_ids, int n_entries, int C, int taps,
                                   void* stream) {
    if (n_entries <= 0 || taps <= 1) return IB_OK;
    if (!x || !state || !cu_rows || !slot_ids || C <= 0 || x_stride < C || state_stride < (long long)(taps - 1) * C)
        return IB_ERR_BAD_ARG;
    if (taps > IB_CONV_MAX_TAPS) return IB_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 128;
    const dim3 grid(n_entries, min(64, (C + threads - 1) / threads));
    cudaError_t le;
    if (dtype == 0)
        le = launch_kernel(conv_state_update_kernel<float>, grid, dim3(threads), 0, s, (const float*)x, x_stride, state,
                           state_stride, cu_rows, slot_ids, C, taps);
    else if (dtype == 1)
        le = launch_kernel(conv_state_update_kernel<bf16>, grid, dim3(threads), 0, s, (const bf16*)x, x_stride, state,
                           state_stride, cu_rows, slot_ids, C, taps);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
