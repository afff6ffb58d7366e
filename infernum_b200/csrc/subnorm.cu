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
    if (act_dtype == 0)
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
