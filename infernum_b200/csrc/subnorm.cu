// Layers that norm a sub-layer's result before adding it to the stream, with an
// RMS norm over equal consecutive parts of the vector, and whose stream between
// layers is a weighted sum of all layers' results so far.
//
//   part norm       n(y)[c] = y[c] / sqrt(mean_{c' in part(c)} y[c']^2 + eps) * w[c]
//   sub-layer add   X = x + n(y)
//   depth average   x' = sum_{j <= J} coef[j] R_j,  R_J = X (stored), R_0 the embedding output
//
// A part of a row is independent of the others in all three, so one CTA works on
// one (row, part): two passes over its share of the sub-layer's result (the second
// from L1), everything in 32-bit, the stream written in 32-bit and, rounded once,
// in the activation dtype for the products of the next sub-layer.
#include "common.cuh"

using namespace ib;

// Token embedding into the 32-bit stream and, when asked, its copy in the
// activation dtype (sub-layers of this arrangement read the stream itself).
template <typename TW, typename TA>
__global__ void embed_dual_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                  float* __restrict__ out, TA* __restrict__ act, int H, int V,
                                  unsigned* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int id = ids[row];
    float* o = out + (size_t)row * H;
    TA* a = act ? act + (size_t)row * H : nullptr;
    const bool bad = id < 0 || id >= V;
    if (bad && threadIdx.x == 0) atomicOr(err, IB_FLAG_BAD_TOKEN);
    const TW* src = table + (size_t)(bad ? 0 : id) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = bad ? 0.f : to_f32(src[i]);
        o[i] = v;
        if (a) a[i] = from_f32<TA>(v);
    }
}

IB_EXPORT int ib_embed_dual(const int* ids, const void* table, int table_dtype, float* out, void* act, int act_dtype,
                            int n_rows, int H, int V, unsigned* err, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!ids || !table || !out || !err || H <= 0 || V <= 0) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    cudaError_t le;
    if (table_dtype == 0 && (!act || act_dtype == 0))
        le = launch_kernel(embed_dual_kernel<float, float>, dim3(n_rows), dim3(threads), 0, s, ids, (const float*)table,
                           out, (float*)act, H, V, err);
    else if (table_dtype == 1 && (!act || act_dtype == 1))
        le = launch_kernel(embed_dual_kernel<bf16, bf16>, dim3(n_rows), dim3(threads), 0, s, ids, (const bf16*)table,
                           out, (bf16*)act, H, V, err);
    else if (table_dtype == 0 && act_dtype == 1)
        le = launch_kernel(embed_dual_kernel<float, bf16>, dim3(n_rows), dim3(threads), 0, s, ids, (const float*)table,
                           out, (bf16*)act, H, V, err);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// x_in, out_res: float32 [N, W] (they may be the same buffer); y: [N, W] of the
// activation dtype; w: float32 [W]; results: float32 [slots][N][W] or null; slot:
// where X is stored; coef: float32 [slot + 1]; out_act: [N, W] or null.
template <typename T>
__global__ void sub_norm_add_kernel(const float* __restrict__ x_in, const T* __restrict__ y,
                                    const float* __restrict__ w, float eps, float* __restrict__ results,
                                    int slot, const float* __restrict__ coef, float* __restrict__ out_res,
                                    T* __restrict__ out_act, int n_rows, int W, int part) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int row = blockIdx.x, c0 = blockIdx.y * part;
    const size_t base = (size_t)row * W + c0;
    const T* yp = y + base;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        const float v = to_f32(yp[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)part + eps);
    const size_t plane = (size_t)n_rows * W;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        const float X = x_in[base + i] + to_f32(yp[i]) * inv * w[c0 + i];
        float o = X;
        if (results) {
            results[(size_t)slot * plane + base + i] = X;
            float acc = 0.f;
            for (int j = 0; j < slot; ++j) acc = fmaf(coef[j], results[(size_t)j * plane + base + i], acc);
            o = fmaf(coef[slot], X, acc);
        }
        out_res[base + i] = o;
        if (out_act) out_act[base + i] = from_f32<T>(o);
    }
}

// The same four columns at a time: 16-byte loads and stores of the 32-bit planes (8-byte of a
// 16-bit activation), for parts whose length is a multiple of 4 and 16-byte aligned planes.
template <typename T>
struct Vec4 {
    static __device__ __forceinline__ float4 load(const T* p);
    static __device__ __forceinline__ void store(T* p, float4 v);
};
template <>
struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <>
struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
        const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
        return make_float4(fa.x, fa.y, fb.x, fb.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 r;
        r.x = *reinterpret_cast<const unsigned*>(&a);
        r.y = *reinterpret_cast<const unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = r;
    }
};

template <typename T>
__global__ void sub_norm_add_vec4_kernel(const float* __restrict__ x_in, const T* __restrict__ y,
                                         const float* __restrict__ w, float eps, float* __restrict__ results,
                                         int slot, const float* __restrict__ coef, float* __restrict__ out_res,
                                         T* __restrict__ out_act, int n_rows, int W, int part) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int row = blockIdx.x, c0 = blockIdx.y * part;
    const size_t base = (size_t)row * W + c0;
    const T* yp = y + base;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < part; i += blockDim.x * 4) {
        const float4 v = Vec4<T>::load(yp + i);
        ss = fmaf(v.x, v.x, ss);
        ss = fmaf(v.y, v.y, ss);
        ss = fmaf(v.z, v.z, ss);
        ss = fmaf(v.w, v.w, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)part + eps);
    const size_t plane = (size_t)n_rows * W;
    for (int i = threadIdx.x * 4; i < part; i += blockDim.x * 4) {
        const float4 yv = Vec4<T>::load(yp + i);
        const float4 xv = Vec4<float>::load(x_in + base + i);
        const float4 wv = Vec4<float>::load(w + c0 + i);
        // the same operations in the same order as the column-by-column kernel
        float4 X = make_float4(xv.x + yv.x * inv * wv.x, xv.y + yv.y * inv * wv.y, xv.z + yv.z * inv * wv.z,
                               xv.w + yv.w * inv * wv.w);
        float4 o = X;
        if (results) {
            Vec4<float>::store(results + (size_t)slot * plane + base + i, X);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < slot; ++j) {
                const float c = coef[j];
                const float4 r = Vec4<float>::load(results + (size_t)j * plane + base + i);
                acc.x = fmaf(c, r.x, acc.x);
                acc.y = fmaf(c, r.y, acc.y);
                acc.z = fmaf(c, r.z, acc.z);
                acc.w = fmaf(c, r.w, acc.w);
            }
            const float c = coef[slot];
            o = make_float4(fmaf(c, X.x, acc.x), fmaf(c, X.y, acc.y), fmaf(c, X.z, acc.z), fmaf(c, X.w, acc.w));
        }
        Vec4<float>::store(out_res + base + i, o);
        if (out_act) Vec4<T>::store(out_act + base + i, o);
    }
}

static int vec4_threads(int part) {
    const int v = part / 4;
    return v >= 256 ? 256 : (v >= 128 ? 128 : (v >= 64 ? 64 : 32));
}

static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

static int part_threads(int part) { return part >= 2048 ? 512 : (part >= 512 ? 256 : (part >= 128 ? 128 : 64)); }

IB_EXPORT int ib_sub_norm_add(const float* x_in, const void* y, int act_dtype, const float* w, float eps,
                              float* results, int slot, const float* coef, float* out_res, void* out_act,
                              int n_rows, int W, int parts, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x_in || !y || !w || !out_res || W <= 0 || parts <= 0 || W % parts || !(eps > 0.f)) return IB_ERR_BAD_ARG;
    if (results && (!coef || slot < 1)) return IB_ERR_BAD_ARG;
    if (parts > 65535) return IB_ERR_TOO_LARGE;
    const int part = W / parts;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_rows, parts), block(part_threads(part));
    cudaError_t le;
    const bool vec = part % 4 == 0 && aligned16(x_in) && aligned16(y) && aligned16(w) && aligned16(out_res) &&
                     (!results || aligned16(results)) && (!out_act || aligned16(out_act)) &&
                     (act_dtype == 0 || act_dtype == 1);
    if (vec && act_dtype == 0)
        le = launch_kernel(sub_norm_add_vec4_kernel<float>, grid, dim3(vec4_threads(part)), 0, s, x_in,
                           (const float*)y, w, eps, results, slot, coef, out_res, (float*)out_act, n_rows, W, part);
    else if (vec)
        le = launch_kernel(sub_norm_add_vec4_kernel<bf16>, grid, dim3(vec4_threads(part)), 0, s, x_in,
                           (const bf16*)y, w, eps, results, slot, coef, out_res, (bf16*)out_act, n_rows, W, part);
    else if (act_dtype == 0)
        le = launch_kernel(sub_norm_add_kernel<float>, grid, block, 0, s, x_in, (const float*)y, w, eps, results, slot,
                           coef, out_res, (float*)out_act, n_rows, W, part);
    else if (act_dtype == 1)
        le = launch_kernel(sub_norm_add_kernel<bf16>, grid, block, 0, s, x_in, (const bf16*)y, w, eps, results, slot,
                           coef, out_res, (bf16*)out_act, n_rows, W, part);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// The part norm of rows of the 32-bit stream (all rows, or those `row_idx` names),
// written compactly in the activation dtype.
template <typename T>
__global__ void part_rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ row_idx,
                                    const float* __restrict__ w, float eps, T* __restrict__ out, int W, int part) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x, c0 = blockIdx.y * part;
    const int row = row_idx ? row_idx[r] : r;
    const float* xp = x + (size_t)row * W + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) ss = fmaf(xp[i], xp[i], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)part + eps);
    T* op = out + (size_t)r * W + c0;
    for (int i = threadIdx.x; i < part; i += blockDim.x) op[i] = from_f32<T>(xp[i] * inv * w[c0 + i]);
}

IB_EXPORT int ib_part_rmsnorm(const float* x, const int* row_idx, const float* w, float eps, void* out,
                              int act_dtype, int n_out, int W, int parts, void* stream) {
    if (n_out <= 0) return IB_OK;
    if (!x || !w || !out || W <= 0 || parts <= 0 || W % parts || !(eps > 0.f)) return IB_ERR_BAD_ARG;
    if (parts > 65535) return IB_ERR_TOO_LARGE;
    const int part = W / parts;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_out, parts), block(part_threads(part));
    cudaError_t le;
    if (act_dtype == 0)
        le = launch_kernel(part_rmsnorm_kernel<float>, grid, block, 0, s, x, row_idx, w, eps, (float*)out, W, part);
    else if (act_dtype == 1)
        le = launch_kernel(part_rmsnorm_kernel<bf16>, grid, block, 0, s, x, row_idx, w, eps, (bf16*)out, W, part);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// Layers that norm both what a sub-layer reads and what it returns, with a gate on the
// result and a fixed factor on the addition:
//   X = x + mult * n(y * sigmoid(g + b))
// y: the sub-layer's result, g: the gate's projection (both of the activation dtype, g may
// lie in wider rows), b: the gate's bias (float32, may be null; g null: no gate).  One CTA
// per (row, part); the gated values are formed twice (sum of squares, then the store)
// rather than kept, 32-bit throughout.
template <typename T>
__global__ void gated_norm_add_kernel(const float* __restrict__ x_in, const T* __restrict__ y,
                                      const T* __restrict__ g, int g_stride, const float* __restrict__ gb,
                                      const float* __restrict__ w, float eps, float mult,
                                      float* __restrict__ out_res, T* __restrict__ out_act, int W, int part) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int row = blockIdx.x, c0 = blockIdx.y * part;
    const size_t base = (size_t)row * W + c0;
    const T* yp = y + base;
    const T* gp = g ? g + (size_t)row * g_stride + c0 : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        float v = to_f32(yp[i]);
        if (gp) v = v / (1.f + expf(-(to_f32(gp[i]) + (gb ? gb[c0 + i] : 0.f))));
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        float v = to_f32(yp[i]);
        if (gp) v = v / (1.f + expf(-(to_f32(gp[i]) + (gb ? gb[c0 + i] : 0.f))));
        const float X = fmaf(mult, v * inv * w[c0 + i], x_in[base + i]);
        out_res[base + i] = X;
        if (out_act) out_act[base + i] = from_f32<T>(X);
    }
}

IB_EXPORT int ib_gated_norm_add(const float* x_in, const void* y, const void* g, int g_stride, const float* gb,
                                int act_dtype, const float* w, float eps, float mult, float* out_res, void* out_act,
                                int n_rows, int W, int parts, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x_in || !y || !w || !out_res || W <= 0 || parts <= 0 || W % parts || !(eps > 0.f) || (g && g_stride < W))
        return IB_ERR_BAD_ARG;
    if (parts > 65535) return IB_ERR_TOO_LARGE;
    const int part = W / parts;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_rows, parts), block(part_threads(part));
    cudaError_t le;
    if (act_dtype == 0)
        le = launch_kernel(gated_norm_add_kernel<float>, grid, block, 0, s, x_in, (const float*)y, (const float*)g,
                           g_stride, gb, w, eps, mult, out_res, (float*)out_act, W, part);
    else if (act_dtype == 1)
        le = launch_kernel(gated_norm_add_kernel<bf16>, grid, block, 0, s, x_in, (const bf16*)y, (const bf16*)g,
                           g_stride, gb, w, eps, mult, out_res, (bf16*)out_act, W, part);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// The part norm of 32-bit rows written back in 32-bit (an embedding that is normed before
// it becomes the stream).
IB_EXPORT int ib_part_rmsnorm_f32(const float* x, const float* w, float eps, float* out, int n_rows, int W, int parts,
                                  void* stream) {
    return ib_part_rmsnorm(x, nullptr, w, eps, out, 0, n_rows, W, parts, stream);
}

// Two 32-bit streams side by side in the activation dtype: out[n] = [a[n] | b[n]], the
// input of a product that reads both.
template <typename T>
__global__ void concat_round_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out,
                                    int W) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < 2 * W; i += gridDim.y * blockDim.x)
        out[(size_t)row * 2 * W + i] = from_f32<T>(i < W ? a[(size_t)row * W + i] : b[(size_t)row * W + i - W]);
}

IB_EXPORT int ib_concat_round(const float* a, const float* b, void* out, int act_dtype, int n_rows, int W,
                              void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!a || !b || !out || W <= 0) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_rows, (2 * W + 1023) / 1024), block(128);
    cudaError_t le;
    if (act_dtype == 0)
        le = launch_kernel(concat_round_kernel<float>, grid, block, 0, s, a, b, (float*)out, W);
    else if (act_dtype == 1)
        le = launch_kernel(concat_round_kernel<bf16>, grid, block, 0, s, a, b, (bf16*)out, W);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// x[n, :] += v[:] on 32-bit rows, in place (a learned vector added to every token's stream).
__global__ void add_row_kernel(float* __restrict__ x, const float* __restrict__ v, int W) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < W; i += gridDim.y * blockDim.x)
        x[(size_t)row * W + i] += v[i];
}

IB_EXPORT int ib_add_row(float* x, const float* v, int n_rows, int W, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x || !v || W <= 0) return IB_ERR_BAD_ARG;
    cudaError_t le = launch_kernel(add_row_kernel, dim3(n_rows, (W + 1023) / 1024), dim3(128), 0, (cudaStream_t)stream,
                                   x, v, W);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
