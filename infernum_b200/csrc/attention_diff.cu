// Differential attention over the paged cache: every head has two score maps over
// the same values, combined as
//
//   o = softmax(s1) V - lambda * softmax(s2) V,   s_m = cap * tanh((q_m . k_m) * scale / cap)
//   out = o / sqrt(mean(o^2) + eps) * out_scale                       (per head, no weight)
//
// A query head's row is [q_1 | q_2] (2 d), a key head's cached row [k_1 | k_2] (2 d), the
// value row e wide; query head a reads key/value head a / (nh / nkv).  The pools are
// [pages, nkv, page_size, 2 d] and [pages, nkv, page_size, e]: both maps of a key sit in
// one row, so a visit of a key serves both maps and the value is fetched once.
//
//   conv_rope_append   rows [q | k | v] as projected -> the short causal convolution per
//                      channel (when there is one; state as in shortconv.cu), then the
//                      rotation of the first rd dimensions of every map of every query and
//                      key head, neighbours (2i, 2i + 1) paired, angle = position * f_i
//                      (32-bit), times mag; queries to q_out, keys and values to their pages.
//   attention_diff     one warp per (row, head): keys in tiles of 32 that start at absolute
//                      multiples of 32, a key a lane for the two scores, then the lanes hold
//                      the value's channels; two running softmaxes; 32-bit throughout.
#include "common.cuh"

using namespace ib;

#define IB_DIFF_MAX_TAPS 16

template <typename T>
__device__ __forceinline__ float conv_at(const T* __restrict__ x, int x_stride, const float* __restrict__ w,
                                         const float* __restrict__ st, int C, int taps, int first, int idx, int c) {
    if (taps <= 0) return to_f32(x[(size_t)(first + idx) * x_stride + c]);
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int src = idx - (taps - 1) + j;
        const float u = src >= 0 ? to_f32(x[(size_t)(first + src) * x_stride + c]) : st[(size_t)(taps - 1 + src) * C + c];
        acc = fmaf(w[(size_t)c * taps + j], u, acc);
    }
    return acc;
}

template <typename T>
__global__ void conv_rope_append_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ w, int taps,
                                        const float* __restrict__ state, long long state_stride,
                                        const int* __restrict__ positions, const int* __restrict__ row_entry,
                                        const int* __restrict__ cu_rows, const int* __restrict__ slot_ids,
                                        const int* __restrict__ block_tables, int max_blocks,
                                        const float* __restrict__ inv_freq, int rd, float mag, int nh, int nkv, int d,
                                        int e, T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                        int page_size, int num_pages, unsigned* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int en = row_entry[row];
    const int first = cu_rows[en], idx = row - first;
    const int pos = positions[row];
    const int qc = nh * 2 * d, kc = nkv * 2 * d, vc = nkv * e, C = qc + kc + vc;
    const float* st = taps > 1 ? state + (long long)slot_ids[en] * state_stride : nullptr;
    const int blk = pos / page_size;
    const int page = blk < max_blocks ? block_tables[(size_t)en * max_blocks + blk] : -1;
    const bool bad = page < 0 || page >= num_pages;
    if (bad && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(err, IB_FLAG_BAD_PAGE);
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float val = conv_at(x, x_stride, w, st, C, taps, first, idx, c);
        if (c < qc + kc) {
            const int i = (c < qc ? c : c - qc) % d;  // place inside the map
            if (i < rd) {
                const float other = conv_at(x, x_stride, w, st, C, taps, first, idx, c ^ 1);  // (maps start at even columns)
                float sn, cs;
                sincosf((float)pos * inv_freq[i >> 1], &sn, &cs);
                sn *= mag;
                cs *= mag;
                val = (i & 1) ? val * cs + other * sn : val * cs - other * sn;
            }
        }
        if (c < qc) {
            q_out[(size_t)row * qc + c] = from_f32<T>(val);
        } else if (bad) {
            continue;
        } else if (c < qc + kc) {
            const int ck = c - qc, g = ck / (2 * d);
            k_pool[(((size_t)page * nkv + g) * page_size + (pos % page_size)) * (2 * d) + ck % (2 * d)] = from_f32<T>(val);
        } else {
            const int cv = c - qc - kc, g = cv / e;
            v_pool[(((size_t)page * nkv + g) * page_size + (pos % page_size)) * e + cv % e] = from_f32<T>(val);
        }
    }
}

// x rows: [nh * 2d | nkv * 2d | nkv * e] of dtype `dtype`; w: float32 [C, taps] (taps 0: no convolution).
IB_EXPORT int ib_conv_rope_append(const void* x, int x_stride, int dtype, const float* w, int taps, const float* state,
                                  long long state_stride, const int* positions, const int* row_entry,
                                  const int* cu_rows, const int* slot_ids, const int* block_tables, int max_blocks,
                                  const float* inv_freq, int rd, float mag, int nh, int nkv, int d, int e, void* q_out,
                                  void* k_pool, void* v_pool, int page_size, int num_pages, int n_rows, unsigned* err,
                                  void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x || !positions || !row_entry || !cu_rows || !slot_ids || !block_tables || !q_out || !k_pool || !v_pool ||
        !err || nh <= 0 || nkv <= 0 || d <= 0 || e <= 0 || page_size <= 0 || num_pages <= 0 || max_blocks <= 0)
        return IB_ERR_BAD_ARG;
    const int C = (nh + nkv) * 2 * d + nkv * e;
    if (x_stride < C || rd < 0 || (rd & 1) || rd > d || (rd > 0 && (!inv_freq || (d & 1)))) return IB_ERR_BAD_ARG;
    if (taps < 0 || taps > IB_DIFF_MAX_TAPS) return IB_ERR_TOO_LARGE;
    if (taps > 0 && !w) return IB_ERR_BAD_ARG;
    if (taps > 1 && (!state || state_stride < (long long)(taps - 1) * C)) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 128;
    const dim3 grid(n_rows, min(64, (C + threads - 1) / threads));
    cudaError_t le;
    if (dtype == 0)
        le = launch_kernel(conv_rope_append_kernel<float>, grid, dim3(threads), 0, s, (const float*)x, x_stride, w, taps,
                           state, state_stride, positions, row_entry, cu_rows, slot_ids, block_tables, max_blocks,
                           inv_freq, rd, mag, nh, nkv, d, e, (float*)q_out, (float*)k_pool, (float*)v_pool, page_size,
                           num_pages, err);
    else if (dtype == 1)
        le = launch_kernel(conv_rope_append_kernel<bf16>, grid, dim3(threads), 0, s, (const bf16*)x, x_stride, w, taps,
                           state, state_stride, positions, row_entry, cu_rows, slot_ids, block_tables, max_blocks,
                           inv_freq, rd, mag, nh, nkv, d, e, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool, page_size,
                           num_pages, err);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// NV * 32 is the largest value size of a build; the maps' size d is bounded by shared memory only.
template <typename T, int NV>
__global__ void attention_diff_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                                      const T* __restrict__ v_pool, T* __restrict__ out,
                                      const int* __restrict__ positions, const int* __restrict__ row_entry,
                                      const int* __restrict__ block_tables, int max_blocks, int nh, int nkv, int d,
                                      int e, int page_size, int num_pages, float scale, float cap, float lambda,
                                      float eps, float out_scale, unsigned* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float qs_all[];
    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * (blockDim.x >> 5) + warp;
    if (head >= nh) return;
    float* qs = qs_all + (size_t)warp * 2 * d;
    const int g = head / (nh / nkv);
    const int pos = positions[row];
    const int* table = block_tables + (size_t)row_entry[row] * max_blocks;
    const T* qp = q + ((size_t)row * nh + head) * 2 * d;
    for (int i = lane; i < 2 * d; i += 32) qs[i] = to_f32(qp[i]);
    __syncwarp();

    float acc1[NV], acc2[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) acc1[i] = acc2[i] = 0.f;
    float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.f, l2 = 0.f;
    for (int j0 = 0; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const bool live = j <= pos;
        long long at = -1;  // the key's row among all rows of a pool
        if (live) {
            const int page = j / page_size < max_blocks ? table[j / page_size] : -1;
            if (page < 0 || page >= num_pages)
                atomicOr(err, IB_FLAG_BAD_PAGE);
            else
                at = ((long long)page * nkv + g) * page_size + (j % page_size);
        }
        float s1 = -INFINITY, s2 = -INFINITY;
        if (at >= 0) {
            const T* kp = k_pool + (size_t)at * 2 * d;
            float a = 0.f, b = 0.f;
            for (int i = 0; i < d; ++i) {
                a = fmaf(qs[i], to_f32(kp[i]), a);
                b = fmaf(qs[d + i], to_f32(kp[d + i]), b);
            }
            s1 = a * scale;
            s2 = b * scale;
            if (cap > 0.f) {
                s1 = cap * tanhf(s1 / cap);
                s2 = cap * tanhf(s2 / cap);
            }
        }
        const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
        if (n1 == -INFINITY) continue;  // (no key of the tile could be read; the whole warp takes this)
        const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);
        const float p1 = at >= 0 ? expf(s1 - n1) : 0.f, p2 = at >= 0 ? expf(s2 - n2) : 0.f;
        l1 = l1 * c1 + warp_sum(p1);
        l2 = l2 * c2 + warp_sum(p2);
        m1 = n1;
        m2 = n2;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            acc1[i] *= c1;
            acc2[i] *= c2;
        }
        const int count = min(32, pos - j0 + 1);
        for (int t = 0; t < count; ++t) {
            const long long vt = __shfl_sync(0xffffffffu, at, t);
            const float w1 = __shfl_sync(0xffffffffu, p1, t), w2 = __shfl_sync(0xffffffffu, p2, t);
            if (vt < 0) continue;
            const T* vp = v_pool + (size_t)vt * e;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int c = lane + 32 * i;
                if (c < e) {
                    const float v = to_f32(vp[c]);
                    acc1[i] = fmaf(w1, v, acc1[i]);
                    acc2[i] = fmaf(w2, v, acc2[i]);
                }
            }
        }
    }
    const float i1 = l1 > 0.f ? 1.f / l1 : 0.f, i2 = l2 > 0.f ? 1.f / l2 : 0.f;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        acc1[i] = c < e ? acc1[i] * i1 - lambda * (acc2[i] * i2) : 0.f;
        ss = fmaf(acc1[i], acc1[i], ss);
    }
    ss = warp_sum(ss);
    const float f = out_scale / sqrtf(ss / (float)e + eps);
    T* op = out + ((size_t)row * nh + head) * e;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < e) op[c] = from_f32<T>(acc1[i] * f);
    }
}

template <typename T, int NV>
static int launch_diff(const void* q, const void* k_pool, const void* v_pool, void* out, const int* positions,
                       const int* row_entry, const int* block_tables, int max_blocks, int n_rows, int nh, int nkv, int d,
                       int e, int page_size, int num_pages, float scale, float cap, float lambda, float eps,
                       float out_scale, unsigned* err, cudaStream_t s) {
    int warps = 4;
    while (warps > 1 && (size_t)warps * 2 * d * sizeof(float) > 48 * 1024) warps >>= 1;
    const size_t smem = (size_t)warps * 2 * d * sizeof(float);
    if (smem > 48 * 1024) return IB_ERR_TOO_LARGE;
    cudaError_t le = launch_kernel(attention_diff_kernel<T, NV>, dim3(n_rows, (nh + warps - 1) / warps), dim3(warps * 32),
                                   smem, s, (const T*)q, (const T*)k_pool, (const T*)v_pool, (T*)out, positions,
                                   row_entry, block_tables, max_blocks, nh, nkv, d, e, page_size, num_pages, scale, cap,
                                   lambda, eps, out_scale, err);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// q: contiguous [n_rows, nh, 2 d]; out: contiguous [n_rows, nh, e]; cap <= 0: scores are not capped.
IB_EXPORT int ib_attention_diff(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                                const int* positions, const int* row_entry, const int* block_tables, int max_blocks,
                                int n_rows, int nh, int nkv, int d, int e, int page_size, int num_pages, float scale,
                                float cap, float lambda, float eps, float out_scale, unsigned* err, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!q || !k_pool || !v_pool || !out || !positions || !row_entry || !block_tables || !err) return IB_ERR_BAD_ARG;
    if (nh <= 0 || nkv <= 0 || nh % nkv || d <= 0 || e <= 0 || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 ||
        !(eps > 0.f))
        return IB_ERR_BAD_ARG;
    if (e > 512) return IB_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
#define IB_DIFF(T, NV)                                                                                                 \
    return launch_diff<T, NV>(q, k_pool, v_pool, out, positions, row_entry, block_tables, max_blocks, n_rows, nh, nkv, \
                              d, e, page_size, num_pages, scale, cap, lambda, eps, out_scale, err, s)
    if (dtype == 0) {
        if (e <= 64) IB_DIFF(float, 2);
        if (e <= 128) IB_DIFF(float, 4);
        if (e <= 256) IB_DIFF(float, 8);
        IB_DIFF(float, 16);
    }
    if (dtype == 1) {
        if (e <= 64) IB_DIFF(bf16, 2);
        if (e <= 128) IB_DIFF(bf16, 4);
        if (e <= 256) IB_DIFF(bf16, 8);
        IB_DIFF(bf16, 16);
    }
#undef IB_DIFF
    return IB_ERR_UNSUPPORTED;
}
