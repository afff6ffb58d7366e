// Kernels around attention over a compressed (latent) key/value cache.
//
// A token's cache entry is one vector [ c : kv_rank | r : rot_dim ]: the RMS-normed
// latent from which every head's keys and values are projections, and one
// rotated key part shared by all heads.  The pool is
// [pages, 1, page_size, kv_rank + rot_dim].
//
//   latent_prepare   a row of the down projections [ dq : q_rank | dkv : kv_rank | rot : rot_dim ]
//                    (32-bit or the activation dtype) -> c_q = rmsnorm(dq) * wq in the activation dtype;
//                    c = rmsnorm(dkv) * wkv and r = rotate(rot, position) into the
//                    token's place in the pool.  Norms and angles in 32-bit.
//   latent_q_rotate  the rotated part of every head's query, [.. dim | rot_dim ..] per
//                    head, rotated by its position and written behind the head's
//                    latent-space query: q_abs[row, head, kv_rank : kv_rank + rot_dim].
//
// Rotation pairs element i with i + rd/2 (i < rd/2) of the rotated part, angle
// position * inv_freq[i]; elements from rd on pass unchanged.  With `adjacent`
// the pairs are the neighbours (2i, 2i + 1) instead, and `mag` multiplies both
// the cosine and the sine (frequency rescaling that comes with a magnitude).
#include "common.cuh"

using namespace ib;

template <typename TI, typename T>
__global__ void latent_prepare_kernel(const TI* __restrict__ lat, int lat_stride, int q_rank, int kv_rank,
                                      int rot_dim, int rd, const T* __restrict__ wq, const T* __restrict__ wkv,
                                      float eps, const float* __restrict__ inv_freq,
                                      const int* __restrict__ positions, const int* __restrict__ row_entry,
                                      const int* __restrict__ block_tables, int max_blocks, T* __restrict__ cq_out,
                                      T* __restrict__ pool, int page_size, int num_pages, int write_kv,
                                      int adjacent, float mag, unsigned* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[64];
    const int row = blockIdx.x;
    const TI* x = lat + (size_t)row * lat_stride;
    const TI* kv = x + q_rank;
    // the token's place in the pool first: the look-up runs under the sums
    int pos = 0, page = -1;
    if (write_kv) {
        pos = positions[row];
        const int blk = pos / page_size;
        page = blk < max_blocks ? block_tables[(size_t)row_entry[row] * max_blocks + blk] : -1;
    }
    // both sums of squares in one pass and one barrier; the order of the additions is fixed
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) sq += to_f32(x[i]) * to_f32(x[i]);
    if (write_kv)
        for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) sk += to_f32(kv[i]) * to_f32(kv[i]);
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    if (lane == 0) {
        scratch[warp] = sq;
        scratch[32 + warp] = sk;
    }
    __syncthreads();
    sq = 0.f;
    sk = 0.f;
    for (int w = 0; w < nwarps; ++w) {
        sq += scratch[w];
        sk += scratch[32 + w];
    }
    if (q_rank > 0) {
        const float inv = 1.f / sqrtf(sq / (float)q_rank + eps);
        T* o = cq_out + (size_t)row * q_rank;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) o[i] = from_f32<T>(to_f32(x[i]) * inv * to_f32(wq[i]));
    }
    if (!write_kv) return;
    if (page < 0 || page >= num_pages) {  // the whole block takes this branch
        if (threadIdx.x == 0) atomicOr(err, IB_FLAG_BAD_PAGE);
        return;
    }
    const int width = kv_rank + rot_dim;
    T* dst = pool + ((size_t)page * page_size + (pos % page_size)) * width;
    const float inv = 1.f / sqrtf(sk / (float)kv_rank + eps);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) dst[i] = from_f32<T>(to_f32(kv[i]) * inv * to_f32(wkv[i]));
    const TI* rt = kv + kv_rank;
    const int half = rd / 2;
    for (int i = threadIdx.x; i < rot_dim - half; i += blockDim.x) {
        if (i < half) {
            const int a = adjacent ? 2 * i : i, b = adjacent ? 2 * i + 1 : i + half;
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            sn *= mag;
            cs *= mag;
            const float u = to_f32(rt[a]), v = to_f32(rt[b]);
            dst[kv_rank + a] = from_f32<T>(u * cs - v * sn);
            dst[kv_rank + b] = from_f32<T>(v * cs + u * sn);
        } else {
            dst[kv_rank + i + half] = from_f32<T>(to_f32(rt[i + half]));
        }
    }
}

// dtype: of c_q, the norm weights and the pool (0 = f32, 1 = bf16); in_dtype: of `lat`.
IB_EXPORT int ib_latent_prepare_ex(const void* lat, int in_dtype, int lat_stride, int q_rank, int kv_rank, int rot_dim,
                                   int rd, const void* wq, const void* wkv, float eps, const float* inv_freq,
                                   const int* positions, const int* row_entry, const int* block_tables,
                                   int max_blocks, void* cq_out, void* pool, int dtype, int page_size, int num_pages,
                                   int write_kv, int n_rows, int adjacent, float mag, unsigned* err, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!lat || q_rank < 0 || !(eps > 0.f) || !err) return IB_ERR_BAD_ARG;
    if (q_rank > 0 && (!wq || !cq_out)) return IB_ERR_BAD_ARG;
    if (write_kv && (kv_rank <= 0 || rot_dim < 0 || rd < 0 || (rd & 1) || rd > rot_dim || !wkv || !positions ||
                     !row_entry || !block_tables || !pool || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 ||
                     (rd > 0 && !inv_freq)))
        return IB_ERR_BAD_ARG;
    if (lat_stride < q_rank + (write_kv ? kv_rank + rot_dim : 0)) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int widest = q_rank > kv_rank ? q_rank : kv_rank;
    const int threads = widest >= 1024 ? 256 : 128;
    cudaError_t le;
#define IB_PREP(TI, T)                                                                                              \
    le = launch_kernel(latent_prepare_kernel<TI, T>, dim3(n_rows), dim3(threads), 0, s, (const TI*)lat, lat_stride, \
                       q_rank, kv_rank, rot_dim, rd, (const T*)wq, (const T*)wkv, eps, inv_freq, positions,         \
                       row_entry, block_tables, max_blocks, (T*)cq_out, (T*)pool, page_size, num_pages, write_kv,   \
                       adjacent, mag, err)
    if (dtype == 0 && in_dtype == 0) IB_PREP(float, float);
    else if (dtype == 1 && in_dtype == 0) IB_PREP(float, bf16);
    else if (dtype == 1 && in_dtype == 1) IB_PREP(bf16, bf16);
    else return IB_ERR_UNSUPPORTED;
#undef IB_PREP
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

IB_EXPORT int ib_latent_prepare(const void* lat, int in_dtype, int lat_stride, int q_rank, int kv_rank, int rot_dim, int rd,
                                const void* wq, const void* wkv, float eps, const float* inv_freq,
                                const int* positions, const int* row_entry, const int* block_tables,
                                int max_blocks, void* cq_out, void* pool, int dtype, int page_size, int num_pages,
                                int write_kv, int n_rows, unsigned* err, void* stream) {
    return ib_latent_prepare_ex(lat, in_dtype, lat_stride, q_rank, kv_rank, rot_dim, rd, wq, wkv, eps, inv_freq, positions,
                                row_entry, block_tables, max_blocks, cq_out, pool, dtype, page_size, num_pages, write_kv,
                                n_rows, 0, 1.f, err, stream);
}

template <typename T>
__global__ void latent_q_rotate_kernel(const T* __restrict__ q, int q_stride, int heads, int dim, int rot_dim,
                                       int rd, const float* __restrict__ inv_freq,
                                       const int* __restrict__ positions, T* __restrict__ q_abs, int abs_stride,
                                       int abs_head, int abs_off, int adjacent, float mag) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int pos = positions[row];
    const int half = rd / 2;
    const int per_head = rot_dim - half;  // items: a pair each below half, a single element beyond
    for (int it = threadIdx.x; it < heads * per_head; it += blockDim.x) {
        const int h = it / per_head, i = it % per_head;
        const T* src = q + (size_t)row * q_stride + (size_t)h * (dim + rot_dim) + dim;
        T* dst = q_abs + (size_t)row * abs_stride + (size_t)h * abs_head + abs_off;
        if (i < half) {
            const int a = adjacent ? 2 * i : i, b = adjacent ? 2 * i + 1 : i + half;
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            sn *= mag;
            cs *= mag;
            const float u = to_f32(src[a]), v = to_f32(src[b]);
            dst[a] = from_f32<T>(u * cs - v * sn);
            dst[b] = from_f32<T>(v * cs + u * sn);
        } else {
            dst[i + half] = src[i + half];
        }
    }
}

IB_EXPORT int ib_latent_q_rotate_ex(const void* q, int q_stride, int heads, int dim, int rot_dim, int rd,
                                    const float* inv_freq, const int* positions, void* q_abs, int abs_stride,
                                    int abs_head, int abs_off, int dtype, int n_rows, int adjacent, float mag,
                                    void* stream) {
    if (n_rows <= 0 || rot_dim == 0) return IB_OK;
    if (!q || !q_abs || !positions || heads <= 0 || dim < 0 || rot_dim < 0 || rd < 0 || (rd & 1) || rd > rot_dim ||
        (rd > 0 && !inv_freq) || q_stride < heads * (dim + rot_dim))
        return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t le;
    if (dtype == 0)
        le = launch_kernel(latent_q_rotate_kernel<float>, dim3(n_rows), dim3(128), 0, s, (const float*)q, q_stride,
                           heads, dim, rot_dim, rd, inv_freq, positions, (float*)q_abs, abs_stride, abs_head, abs_off, adjacent,
                           mag);
    else if (dtype == 1)
        le = launch_kernel(latent_q_rotate_kernel<bf16>, dim3(n_rows), dim3(128), 0, s, (const bf16*)q, q_stride,
                           heads, dim, rot_dim, rd, inv_freq, positions, (bf16*)q_abs, abs_stride, abs_head, abs_off, adjacent,
                           mag);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

IB_EXPORT int ib_latent_q_rotate(const void* q, int q_stride, int heads, int dim, int rot_dim, int rd,
                                 const float* inv_freq, const int* positions, void* q_abs, int abs_stride,
                                 int abs_head, int abs_off, int dtype, int n_rows, void* stream) {
    return ib_latent_q_rotate_ex(q, q_stride, heads, dim, rot_dim, rd, inv_freq, positions, q_abs, abs_stride, abs_head,
                                 abs_off, dtype, n_rows, 0, 1.f, stream);
}
