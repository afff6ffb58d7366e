// Plain attention over the paged cache: one warp per (query row, head), keys
// visited one by one in order, online softmax, everything in 32-bit.  It takes
// any head size, page size, head grouping and window.  It is the attention of
// the 32-bit path and the yardstick the faster kernels are checked against.
//
// For query head a the key/value head is a / (nh / nkv); scores are
// (q . k) * scale; the query at absolute position p sees keys j with
// max(0, p - window + 1) <= j <= p (window <= 0: all keys 0..p) and, with
// keep_first > 0, also the keys j < keep_first however far back they lie (they
// keep their own positions); softmax with max subtraction and expf; output
// sum_j P_j v_j.  This restates
// infernum-cuda/kernels/paged_decode_attention.cu:540-644 (decode) and
// infernum-cuda/kernels/flash_prefill_attention_v2.cu:82-95,149-192 (prefill)
// as one kernel over a batch of rows that each carry their own position.
#include "common.cuh"

using namespace ib;

// Keys and values need not have the same size, nor live in different pools: a
// value may be the first `hdv` elements of a row of `v_width` elements (for a
// latent cache the value of a token is the first part of its key, and both
// pointers name the one pool).  Heads of a query or output row may be further
// apart than their size (`q_hs`, `o_hs`).
//
// A value may also be wider than a key (two pools).
//
// NREG * 32 is the largest key or value size a build of the kernel takes.
template <typename T, int PLAIN_MAX_REGS>
__global__ void attention_plain_kernel(const T* __restrict__ q, int q_stride,
                                       const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                       T* __restrict__ out, int out_stride,
                                       const int* __restrict__ positions,
                                       const int* __restrict__ row_entry,
                                       const int* __restrict__ block_tables, int max_blocks,
                                       int nh, int nkv, int hd, int page_size, int num_pages,
                                       int window, float scale, int hdv, int v_width, int q_hs, int o_hs,
                                       const float* __restrict__ sink, int keep_first,
                                       unsigned* __restrict__ err) {
    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * (blockDim.x >> 5) + warp;
    if (head >= nh) return;
    const int g = head / (nh / nkv);
    const int pos = positions[row];
    const int e = row_entry[row];
    const int* table = block_tables + (size_t)e * max_blocks;

    float qr[PLAIN_MAX_REGS], acc[PLAIN_MAX_REGS];
    const T* qp = q + (size_t)row * q_stride + (size_t)head * q_hs;
#pragma unroll
    for (int i = 0; i < PLAIN_MAX_REGS; ++i) {
        const int d = lane + 32 * i;
        qr[i] = d < hd ? to_f32(qp[d]) : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int kept = min(max(keep_first, 0), lo);  // keys below the window that stay visible
    for (int j = kept > 0 ? 0 : lo; j <= pos; ++j) {
        if (j == kept && j < lo) j = lo;
        const int page = j / page_size < max_blocks ? table[j / page_size] : -1;  // beyond the row: reported, not read
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicOr(err, IB_FLAG_BAD_PAGE);
            continue;
        }
        const size_t at = ((size_t)page * nkv + g) * page_size + (j % page_size);
        const T* kp = k_pool + at * hd;
        const T* vp = v_pool + at * v_width;
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < PLAIN_MAX_REGS; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) part += qr[i] * to_f32(kp[d]);
        }
        const float s = warp_sum(part) * scale;
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < PLAIN_MAX_REGS; ++i) {
            const int d = lane + 32 * i;
            if (d < hdv) acc[i] = acc[i] * corr + p * to_f32(vp[d]);
        }
        m = m_new;
    }
    if (sink) {
        // a learned logit per head that takes part in the denominator only: no key, no value, not scaled
        const float sk = sink[head];
        const float m_new = fmaxf(m, sk);
        const float corr = expf(m - m_new);
        l = l * corr + expf(sk - m_new);
#pragma unroll
        for (int i = 0; i < PLAIN_MAX_REGS; ++i) acc[i] *= corr;
    }
    T* op = out + (size_t)row * out_stride + (size_t)head * o_hs;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < PLAIN_MAX_REGS; ++i) {
        const int d = lane + 32 * i;
        if (d < hdv) op[d] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T, int NREG>
static int launch_plain(const void* q, int q_stride, const void* k_pool, const void* v_pool, void* out,
                        int out_stride, const int* positions, const int* row_entry, const int* block_tables,
                        int max_blocks, int n_rows, int nh, int nkv, int hd, int page_size, int num_pages,
                        int window, float scale, int hdv, int v_width, int q_hs, int o_hs, const float* sink,
                        int keep_first, unsigned* err, cudaStream_t s) {
    const int warps = 4;
    dim3 grid(n_rows, (nh + warps - 1) / warps);
    attention_plain_kernel<T, NREG><<<grid, warps * 32, 0, s>>>(
        (const T*)q, q_stride, (const T*)k_pool, (const T*)v_pool, (T*)out, out_stride, positions, row_entry,
        block_tables, max_blocks, nh, nkv, hd, page_size, num_pages, window, scale, hdv, v_width, q_hs, o_hs, sink,
        keep_first, err);
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// The general form: values of `hdv` elements in rows of `v_width`, query heads
// `q_hs` and output heads `o_hs` elements apart; `sink` (optional, float32 [nh])
// adds exp(sink[head]) to each softmax denominator.
// `keep_first`: the keys at positions below it stay visible behind a window.
IB_EXPORT int ib_attention_plain_mask(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                                      void* out, int out_stride, int act_dtype, const int* positions,
                                      const int* row_entry, const int* block_tables, int max_blocks, int n_rows,
                                      int nh, int nkv, int hd, int page_size, int num_pages, int window,
                                      float scale, int hdv, int v_width, int q_hs, int o_hs, const float* sink,
                                      int keep_first, unsigned* err, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!q || !k_pool || !v_pool || !out || !positions || !row_entry || !block_tables || !err)
        return IB_ERR_BAD_ARG;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || page_size <= 0 || max_blocks <= 0 ||
        num_pages <= 0 || hdv <= 0 || hdv > v_width || q_hs < hd || o_hs < hdv)
        return IB_ERR_BAD_ARG;
    const int wide = hd > hdv ? hd : hdv;
    if (wide > 32 * 32) return IB_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
#define IB_PLAIN(T, NREG)                                                                                   \
    return launch_plain<T, NREG>(q, q_stride, k_pool, v_pool, out, out_stride, positions, row_entry,        \
                                 block_tables, max_blocks, n_rows, nh, nkv, hd, page_size, num_pages, window, \
                                 scale, hdv, v_width, q_hs, o_hs, sink, keep_first, err, s)
    if (act_dtype == 0) {
        if (wide <= 256) IB_PLAIN(float, 8);
        if (wide <= 640) IB_PLAIN(float, 20);
        IB_PLAIN(float, 32);
    }
    if (act_dtype == 1) {
        if (wide <= 256) IB_PLAIN(bf16, 8);
        if (wide <= 640) IB_PLAIN(bf16, 20);
        IB_PLAIN(bf16, 32);
    }
#undef IB_PLAIN
    return IB_ERR_UNSUPPORTED;
}

IB_EXPORT int ib_attention_plain_ex(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                                    void* out, int out_stride, int act_dtype, const int* positions,
                                    const int* row_entry, const int* block_tables, int max_blocks, int n_rows,
                                    int nh, int nkv, int hd, int page_size, int num_pages, int window,
                                    float scale, int hdv, int v_width, int q_hs, int o_hs, const float* sink,
                                    unsigned* err, void* stream) {
    return ib_attention_plain_mask(q, q_stride, k_pool, v_pool, out, out_stride, act_dtype, positions, row_entry,
                                   block_tables, max_blocks, n_rows, nh, nkv, hd, page_size, num_pages, window,
                                   scale, hdv, v_width, q_hs, o_hs, sink, 0, err, stream);
}

IB_EXPORT int ib_attention_plain(const void* q, int q_stride, const void* k_pool,
                                 const void* v_pool, void* out, int out_stride, int act_dtype,
                                 const int* positions, const int* row_entry,
                                 const int* block_tables, int max_blocks, int n_rows, int nh,
                                 int nkv, int hd, int page_size, int num_pages, int window,
                                 float scale, unsigned* err, void* stream) {
    return ib_attention_plain_ex(q, q_stride, k_pool, v_pool, out, out_stride, act_dtype, positions, row_entry,
                                 block_tables, max_blocks, n_rows, nh, nkv, hd, page_size, num_pages, window,
                                 scale, hd, hd, hd, hd, nullptr, err, stream);
}
