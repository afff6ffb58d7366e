// Kernels around recurrent mixers (a state carried from token to token per
// request) and around attention with normed queries and keys and an output gate.
// The scans themselves are in scan.cu.  A step's rows are grouped in entries
// (one request's next tokens, in order): row_entry[row], cu_rows[entry],
// slot_ids[entry] live on the device, and a request's state is row `slot` of a
// float32 state tensor whose rows are `state_stride` floats apart.
//
//   token shift    m_j[t] = h_t + (h_{t-1} - h_t) * mu_j        j = 0 .. M-1
//                  h_{-1} of an entry's first row is the request's state, which
//                  then takes the entry's last row
//   causal conv    c_t[ch] = silu(b[ch] + sum_j w[ch][j] x_{t-(taps-1-j)}[ch]),
//                  inputs before the entry from the state (the last taps-1 inputs);
//                  part of the pass that prepares a state space scan's inputs
//   head norm      out = o / rms_head(o) * w * silu(g)          (rms over one head)
//   gated norm     v = y * silu(z); out = v / rms_group(v) * w   (rms over a group)
//   qk norm        q, k <- x / rms(x) * w per head; the normed key and the key
//                  as projected (the value) go to their pages
//   delta prepare  what a gated delta rule's scan reads: convolved, activated and
//                  unit-length queries and keys, values, write strengths and decays
//   rope norm      bias, rotation, then a weightless RMS norm of queries, keys and
//                  values per head; keys and values go to their pages
// All arithmetic is 32-bit; small parameter vectors are float32.
#include "common.cuh"

using namespace ib;

__device__ __forceinline__ float silu_f(float g) { return g / (1.f + expf(-g)); }

// ---------------------------------------------------------------------------
template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ x, const float* __restrict__ mu, float* __restrict__ state,
                                   long long state_stride, const int* __restrict__ row_entry,
                                   const int* __restrict__ cu_rows, const int* __restrict__ slot_ids,
                                   T* __restrict__ out, int n_rows, int D, int M) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int e = row_entry[row];
    const int first = cu_rows[e], last = cu_rows[e + 1] - 1;
    float* prev = state + (long long)slot_ids[e] * state_stride;
    const T* xr = x + (size_t)row * D;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < D; c += gridDim.y * blockDim.x) {
        const float h = to_f32(xr[c]);
        float hp;
        if (row == first) {
            hp = prev[c];
            prev[c] = to_f32(x[(size_t)last * D + c]);  // (only this thread reads prev[c] of this entry)
        } else {
            hp = to_f32(xr[c - D]);
        }
        const float d = hp - h;
        for (int m = 0; m < M; ++m)
            out[((size_t)m * n_rows + row) * D + c] = from_f32<T>(h + d * mu[(size_t)m * D + c]);
    }
}

IB_EXPORT int ib_token_shift(const void* x, int act_dtype, const float* mu, float* state, long long state_stride,
                             const int* row_entry, const int* cu_rows, const int* slot_ids, void* out, int n_rows,
                             int D, int M, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x || !mu || !state || !row_entry || !cu_rows || !slot_ids || !out || D <= 0 || M <= 0) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 128;
    // (a column a thread: few rows - decoded tokens - still fill the machine)
    const dim3 grid(n_rows, min(64, (D + threads - 1) / threads));
    cudaError_t le;
    if (act_dtype == 0)
        le = launch_kernel(token_shift_kernel<float>, grid, dim3(threads), 0, s, (const float*)x, mu, state,
                           state_stride, row_entry, cu_rows, slot_ids, (float*)out, n_rows, D, M);
    else if (act_dtype == 1)
        le = launch_kernel(token_shift_kernel<bf16>, grid, dim3(threads), 0, s, (const bf16*)x, mu, state,
                           state_stride, row_entry, cu_rows, slot_ids, (bf16*)out, n_rows, D, M);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
#define IB_MAX_TAPS 16

// The state after the step: the last taps-1 inputs of (old state ++ the entry's rows).
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state,
                                  long long state_stride, const int* __restrict__ cu_rows,
                                  const int* __restrict__ slot_ids, int C, int taps) {
    pdl_trigger();
    pdl_wait();
    const int e = blockIdx.x;
    const int first = cu_rows[e], n = cu_rows[e + 1] - first;
    if (n <= 0) return;
    float* st = state + (long long)slot_ids[e] * state_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float nv[IB_MAX_TAPS];
        for (int k = 0; k < taps - 1; ++k) {
            const int idx = n - (taps - 1 - k);  // place among the entry's rows; negative: in the old state
            nv[k] = idx >= 0 ? to_f32(x[(size_t)(first + idx) * x_stride + c]) : st[(size_t)(taps - 1 + idx) * C + c];
        }
        for (int k = 0; k < taps - 1; ++k) st[(size_t)k * C + c] = nv[k];
    }
}

// ---------------------------------------------------------------------------
// What the scans read, made in one parallel pass so that the scans themselves only
// copy: every transcendental of a token is computed here, in 32-bit.
//
// ssd_prepare: the causal convolution and SiLU of x | B | C (w null: the rows are
// taken as they are), written apart in 32-bit and by head, the way the scan
// fetches them - x [heads][rows][P], (B, C) pairs [groups][rows][state] - and per
// head (dt, exp(-exp(A_log) dt)) [heads][rows] with dt = softplus(dt_raw + dt_bias).
template <typename T>
__global__ void ssd_prepare_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ w,
                                   const float* __restrict__ b, const float* __restrict__ state,
                                   long long state_stride, const int* __restrict__ row_entry,
                                   const int* __restrict__ cu_rows, const int* __restrict__ slot_ids,
                                   const T* __restrict__ dt_raw, int dt_stride, const float* __restrict__ dt_bias,
                                   const float* __restrict__ a_log, float* __restrict__ xo, float2* __restrict__ bc,
                                   float2* __restrict__ dd, int inner, int gn, int heads, int taps, int n_rows,
                                   int P, int state_rows) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int C = inner + 2 * gn;
    int first = 0;
    const float* st = nullptr;
    if (w) {
        const int e = row_entry[row];
        first = cu_rows[e];
        st = state + (long long)slot_ids[e] * state_stride;
    }
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C + heads; c += gridDim.y * blockDim.x) {
        if (c >= C) {
            const int h = c - C;
            const float raw = to_f32(dt_raw[(size_t)row * dt_stride + h]) + dt_bias[h];
            const float dt = raw > 20.f ? raw : log1pf(expf(raw));
            dd[(size_t)h * n_rows + row] = make_float2(dt, expf(-expf(a_log[h]) * dt));
            continue;
        }
        float v;
        if (w) {
            float acc = b ? b[c] : 0.f;
            for (int j = 0; j < taps; ++j) {
                const int src = row - (taps - 1 - j);
                float in;
                if (src >= first) in = to_f32(x[(size_t)src * x_stride + c]);
                else in = st[(size_t)(taps - 1 - (first - src)) * C + c];
                acc += w[(size_t)c * taps + j] * in;
            }
            v = silu_f(acc);
        } else {
            v = to_f32(x[(size_t)row * x_stride + c]);
        }
        if (c < inner) {
            xo[((size_t)(c / P) * n_rows + row) * P + c % P] = v;
        } else {
            const int k = c < inner + gn ? c - inner : c - inner - gn;
            float2* dst = bc + ((size_t)(k / state_rows) * n_rows + row) * state_rows + k % state_rows;
            if (c < inner + gn) dst->x = v;
            else dst->y = v;
        }
    }
}

IB_EXPORT int ib_ssd_prepare(const void* x, int x_stride, int act_dtype, const float* w, const float* b,
                             float* state, long long state_stride, const int* row_entry, const int* cu_rows,
                             const int* slot_ids, const void* dt_raw, int dt_stride, const float* dt_bias,
                             const float* a_log, float* xo, void* bc, void* dd, int n_rows, int n_entries,
                             int inner, int gn, int heads, int state_rows, int taps, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x || !dt_raw || !dt_bias || !a_log || !xo || !bc || !dd || inner <= 0 || gn <= 0 || heads <= 0 ||
        inner % heads || state_rows <= 0 || gn % state_rows)
        return IB_ERR_BAD_ARG;
    const int P = inner / heads;
    if (w && (!state || !row_entry || !cu_rows || !slot_ids || taps <= 0 || taps > IB_MAX_TAPS || n_entries <= 0))
        return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int C = inner + 2 * gn;
    const int threads = 128;
    const int gy = min(64, (C + heads + threads - 1) / threads);
    cudaError_t le;
    if (act_dtype == 0) {
        le = launch_kernel(ssd_prepare_kernel<float>, dim3(n_rows, gy), dim3(threads), 0, s, (const float*)x, x_stride,
                           w, b, (const float*)state, state_stride, row_entry, cu_rows, slot_ids,
                           (const float*)dt_raw, dt_stride, dt_bias, a_log, xo, (float2*)bc, (float2*)dd, inner, gn,
                           heads, taps, n_rows, P, state_rows);
        if (le == cudaSuccess && w && taps > 1)
            le = launch_kernel(conv_state_kernel<float>, dim3(n_entries, gy), dim3(threads), 0, s, (const float*)x,
                               x_stride, state, state_stride, cu_rows, slot_ids, C, taps);
    } else if (act_dtype == 1) {
        le = launch_kernel(ssd_prepare_kernel<bf16>, dim3(n_rows, gy), dim3(threads), 0, s, (const bf16*)x, x_stride,
                           w, b, (const float*)state, state_stride, row_entry, cu_rows, slot_ids,
                           (const bf16*)dt_raw, dt_stride, dt_bias, a_log, xo, (float2*)bc, (float2*)dd, inner, gn,
                           heads, taps, n_rows, P, state_rows);
        if (le == cudaSuccess && w && taps > 1)
            le = launch_kernel(conv_state_kernel<bf16>, dim3(n_entries, gy), dim3(threads), 0, s, (const bf16*)x,
                               x_stride, state, state_stride, cu_rows, slot_ids, C, taps);
    } else {
        return IB_ERR_UNSUPPORTED;
    }
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// wkv_prepare: per key channel (r, k, w, u k) with w = exp(-exp(z + w0)), and v in 32-bit, both
// by head: [heads][rows][K].
template <typename T>
__global__ void wkv_prepare_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v, int ld,
                                   const float* __restrict__ z, const float* __restrict__ w0,
                                   const float* __restrict__ u, float4* __restrict__ f, float* __restrict__ vo,
                                   int hk, int K, int n_rows, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t row = idx / hk;
    const int c = (int)(idx % hk);
    const float rr = to_f32(r[row * ld + c]);
    const float kk = to_f32(k[row * ld + c]);
    const float w = expf(-expf(z[idx] + w0[c]));
    const size_t at = ((size_t)(c / K) * n_rows + row) * K + c % K;
    f[at] = make_float4(rr, kk, w, u[c] * kk);
    vo[at] = to_f32(v[row * ld + c]);
}

IB_EXPORT int ib_wkv_prepare(const void* r, const void* k, const void* v, int ld, int act_dtype, const float* z,
                             const float* w0, const float* u, void* f, float* vo, int n_rows, int hk, int K,
                             void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!r || !k || !v || !z || !w0 || !u || !f || !vo || hk <= 0 || K <= 0 || hk % K) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)n_rows * hk;
    const unsigned grid = (unsigned)((total + 255) / 256);
    cudaError_t le;
    if (act_dtype == 0)
        le = launch_kernel(wkv_prepare_kernel<float>, dim3(grid), dim3(256), 0, s, (const float*)r, (const float*)k,
                           (const float*)v, ld, z, w0, u, (float4*)f, vo, hk, K, n_rows, total);
    else if (act_dtype == 1)
        le = launch_kernel(wkv_prepare_kernel<bf16>, dim3(grid), dim3(256), 0, s, (const bf16*)r, (const bf16*)k,
                           (const bf16*)v, ld, z, w0, u, (float4*)f, vo, hk, K, n_rows, total);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
// One warp per (row, head): out = o / sqrt(mean_head(o^2) + eps) * w * silu(g).
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ g, int g_stride,
                                      const float* __restrict__ w, T* __restrict__ out, int n_rows, int heads, int K,
                                      float eps) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)n_rows * heads) return;
    const int row = (int)(item / heads), head = (int)(item % heads);
    const float* op = o + ((size_t)row * heads + head) * K;
    float ss = 0.f;
    for (int i = lane; i < K; i += 32) ss += op[i] * op[i];
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)K + eps);
    const T* gp = g ? g + (size_t)row * g_stride + (size_t)head * K : nullptr;
    T* dst = out + ((size_t)row * heads + head) * K;
    for (int i = lane; i < K; i += 32) {
        float v = op[i] * inv * w[(size_t)head * K + i];
        if (gp) v *= silu_f(to_f32(gp[i]));
        dst[i] = from_f32<T>(v);
    }
}

IB_EXPORT int ib_head_norm_gate(const float* o, const void* g, int g_stride, int act_dtype, const float* w, void* out,
                                int n_rows, int heads, int K, float eps, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!o || !w || !out || heads <= 0 || K <= 0 || !(eps > 0.f)) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const long long items = (long long)n_rows * heads;
    const unsigned grid = (unsigned)((items + 3) / 4);
    cudaError_t le;
    if (act_dtype == 0)
        le = launch_kernel(head_norm_gate_kernel<float>, dim3(grid), dim3(128), 0, s, o, (const float*)g, g_stride, w,
                           (float*)out, n_rows, heads, K, eps);
    else if (act_dtype == 1)
        le = launch_kernel(head_norm_gate_kernel<bf16>, dim3(grid), dim3(128), 0, s, o, (const bf16*)g, g_stride, w,
                           (bf16*)out, n_rows, heads, K, eps);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// One block per (row, group): v = y * silu(z); out = v / sqrt(mean_group(v^2) + eps) * w.
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, int z_stride,
                                        const float* __restrict__ w, T* __restrict__ out, int inner, int group,
                                        float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int row = blockIdx.x, g0 = blockIdx.y * group;
    const float* yp = y + (size_t)row * inner + g0;
    const T* zp = z + (size_t)row * z_stride + g0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        const float v = yp[i] * silu_f(to_f32(zp[i]));
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)group + eps);
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        const float v = yp[i] * silu_f(to_f32(zp[i]));
        out[(size_t)row * inner + g0 + i] = from_f32<T>(v * inv * w[g0 + i]);
    }
}

IB_EXPORT int ib_gated_group_norm(const float* y, const void* z, int z_stride, int act_dtype, const float* w,
                                  void* out, int n_rows, int inner, int groups, float eps, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!y || !z || !w || !out || inner <= 0 || groups <= 0 || inner % groups || !(eps > 0.f)) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int group = inner / groups;
    const int threads = group >= 2048 ? 512 : (group >= 512 ? 256 : 128);
    cudaError_t le;
    if (act_dtype == 0)
        le = launch_kernel(gated_group_norm_kernel<float>, dim3(n_rows, groups), dim3(threads), 0, s, y,
                           (const float*)z, z_stride, w, (float*)out, inner, group, eps);
    else if (act_dtype == 1)
        le = launch_kernel(gated_group_norm_kernel<bf16>, dim3(n_rows, groups), dim3(threads), 0, s, y,
                           (const bf16*)z, z_stride, w, (bf16*)out, inner, group, eps);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
// Query/key norm and the write of keys and values into their pages.  x rows
// hold nh query heads followed by nkv key heads of hd values.  One warp per
// (row, head).  Queries are normed in place.  A key is written normed to the
// key pool; the value pool gets the key as projected (value_from_key) or the
// value head found `v_off` elements into the row.
template <typename T>
__global__ void qk_norm_append_kernel(T* __restrict__ x, int x_stride, const float* __restrict__ qw,
                                      const float* __restrict__ kw, float eps, const int* __restrict__ positions,
                                      const int* __restrict__ row_entry, const int* __restrict__ block_tables,
                                      int max_blocks, T* __restrict__ k_pool, T* __restrict__ v_pool, int n_rows,
                                      int nh, int nkv, int hd, int v_off, int page_size, int num_pages,
                                      unsigned* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int per_row = nh + nkv;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)n_rows * per_row) return;
    const int row = (int)(item / per_row), head = (int)(item % per_row);
    T* p = x + (size_t)row * x_stride + (size_t)head * hd;
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
        const float v = to_f32(p[i]);
        ss += v * v;
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)hd + eps);
    if (head < nh) {
        for (int i = lane; i < hd; i += 32) {
            float v = to_f32(p[i]);
            if (qw) v = v * inv * qw[i];
            p[i] = from_f32<T>(v);
        }
        return;
    }
    const int g = head - nh;
    const int pos = positions[row], e = row_entry[row];
    const int slot_idx = pos / page_size;
    const int page = (pos >= 0 && slot_idx < max_blocks) ? block_tables[(size_t)e * max_blocks + slot_idx] : -1;
    if (page < 0 || page >= num_pages) {
        if (lane == 0) atomicOr(err, IB_FLAG_BAD_PAGE);
        return;
    }
    const size_t at = (((size_t)page * nkv + g) * page_size + (pos % page_size)) * hd;
    const T* vsrc = v_off >= 0 ? x + (size_t)row * x_stride + v_off + (size_t)g * hd : p;
    for (int i = lane; i < hd; i += 32) {
        const float raw = to_f32(p[i]);
        v_pool[at + i] = vsrc[i];
        k_pool[at + i] = from_f32<T>(kw ? raw * inv * kw[i] : raw);
    }
}

IB_EXPORT int ib_qk_norm_append(void* x, int x_stride, int act_dtype, const float* qw, const float* kw, float eps,
                                const int* positions, const int* row_entry, const int* block_tables, int max_blocks,
                                void* k_pool, void* v_pool, int n_rows, int nh, int nkv, int hd, int v_off,
                                int page_size, int num_pages, unsigned* err, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x || !positions || !row_entry || !block_tables || !k_pool || !v_pool || !err || nh <= 0 || nkv <= 0 ||
        hd <= 0 || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || !(eps > 0.f))
        return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const long long items = (long long)n_rows * (nh + nkv);
    const unsigned grid = (unsigned)((items + 3) / 4);
    cudaError_t le;
    if (act_dtype == 0)
        le = launch_kernel(qk_norm_append_kernel<float>, dim3(grid), dim3(128), 0, s, (float*)x, x_stride, qw, kw, eps,
                           positions, row_entry, block_tables, max_blocks, (float*)k_pool, (float*)v_pool, n_rows, nh,
                           nkv, hd, v_off, page_size, num_pages, err);
    else if (act_dtype == 1)
        le = launch_kernel(qk_norm_append_kernel<bf16>, dim3(grid), dim3(128), 0, s, (bf16*)x, x_stride, qw, kw, eps,
                           positions, row_entry, block_tables, max_blocks, (bf16*)k_pool, (bf16*)v_pool, n_rows, nh,
                           nkv, hd, v_off, page_size, num_pages, err);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
// Elementwise: op 0: a <- a * sigmoid(b)   (an output gate)
//              op 1: a <- ca * a + cb * b  (two mixers side by side)
//              op 2: a <- tanh(a)
// a is [rows, cols] contiguous, b has rows `b_stride` apart.
template <typename T>
__global__ void pointwise_kernel(T* __restrict__ a, const T* __restrict__ b, int b_stride, int cols, size_t total,
                                 int op, float ca, float cb) {
    pdl_trigger();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const float av = to_f32(a[idx]);
    float bv = 0.f;
    if (b) bv = to_f32(b[(idx / cols) * (size_t)b_stride + idx % cols]);
    float r;
    if (op == 0) r = av / (1.f + expf(-bv));
    else if (op == 1) r = ca * av + cb * bv;
    else r = tanhf(av);
    a[idx] = from_f32<T>(r);
}

IB_EXPORT int ib_pointwise(void* a, const void* b, int b_stride, int act_dtype, int rows, int cols, int op, float ca,
                           float cb, void* stream) {
    if (rows <= 0 || cols <= 0) return IB_OK;
    if (!a || (op != 2 && !b) || op < 0 || op > 2) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)rows * cols;
    const unsigned grid = (unsigned)((total + 255) / 256);
    cudaError_t le;
    if (act_dtype == 0)
        le = launch_kernel(pointwise_kernel<float>, dim3(grid), dim3(256), 0, s, (float*)a, (const float*)b, b_stride,
                           cols, total, op, ca, cb);
    else if (act_dtype == 1)
        le = launch_kernel(pointwise_kernel<bf16>, dim3(grid), dim3(256), 0, s, (bf16*)a, (const bf16*)b, b_stride,
                           cols, total, op, ca, cb);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
// delta_prepare: the pass before the scan of a gated delta rule.  A row of `x`
// holds, from `c_off` on, C = 2 G dk + H dv channels q | k | v (G key heads of dk,
// H value heads of dv) and, at `b_off` and `a_off`, H write-strength and H decay
// pre-activations.  Per channel: the causal convolution (w [C, taps], the last
// column the current token's, no bias; inputs before the entry's rows from the
// last taps - 1 inputs kept in the state; taps 0: no convolution), then SiLU.
// Per key head: q <- q / sqrt(sum q^2 + 1e-6) * dk^-1/2, k <- k / sqrt(sum k^2 + 1e-6).
// Per value head: beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)).
// Written in 32-bit the way the scan fetches: (k, q) pairs [G][rows][dk], values
// [H][rows][dv], and (beta, g, k . q, 0) [H][rows].
// One CTA per row; the row's channels meet in shared memory.
template <typename T>
__global__ void delta_prepare_kernel(const T* __restrict__ x, int x_stride, int c_off, int b_off, int a_off,
                                     const float* __restrict__ w, int taps, const float* __restrict__ state,
                                     long long state_stride, const int* __restrict__ row_entry,
                                     const int* __restrict__ cu_rows, const int* __restrict__ slot_ids,
                                     const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                     float2* __restrict__ kq, float* __restrict__ vo, float4* __restrict__ dd,
                                     int n_rows, int G, int H, int dk, int dv) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float ch[];  // [C] channels, then [G] k . q
    const int row = blockIdx.x;
    const int C = 2 * G * dk + H * dv;
    float* dots = ch + C;
    int first = 0;
    const float* st = nullptr;
    if (taps > 1) {
        const int e = row_entry[row];
        first = cu_rows[e];
        st = state + (long long)slot_ids[e] * state_stride;
    }
    const T* xr = x + c_off;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc;
        if (taps >= 1) {
            acc = 0.f;
            for (int j = 0; j < taps; ++j) {
                const int src = row - (taps - 1 - j);
                float in;
                if (src >= first) in = to_f32(xr[(size_t)src * x_stride + c]);
                else in = st[(size_t)(taps - 1 - (first - src)) * C + c];
                acc = fmaf(w[(size_t)c * taps + j], in, acc);
            }
        } else {
            acc = to_f32(xr[(size_t)row * x_stride + c]);
        }
        ch[c] = silu_f(acc);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int g = warp; g < G; g += nwarps) {
        const float* q = ch + g * dk;
        const float* k = ch + G * dk + g * dk;
        float sq = 0.f, sk = 0.f, qk = 0.f;
        for (int i = lane; i < dk; i += 32) {
            sq = fmaf(q[i], q[i], sq);
            sk = fmaf(k[i], k[i], sk);
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        const float iq = (float)(1.0 / sqrt((double)dk)) / sqrtf(sq + 1e-6f), ik = 1.f / sqrtf(sk + 1e-6f);
        float2* dst = kq + ((size_t)g * n_rows + row) * dk;
        for (int i = lane; i < dk; i += 32) {
            const float kn = k[i] * ik, qn = q[i] * iq;
            dst[i] = make_float2(kn, qn);
            qk = fmaf(kn, qn, qk);
        }
        qk = warp_sum(qk);
        if (lane == 0) dots[g] = qk;
    }
    const float* v = ch + 2 * G * dk;
    for (int c = threadIdx.x; c < H * dv; c += blockDim.x)
        vo[((size_t)(c / dv) * n_rows + row) * dv + c % dv] = v[c];
    __syncthreads();
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float b = to_f32(x[(size_t)row * x_stride + b_off + h]);
        const float a = to_f32(x[(size_t)row * x_stride + a_off + h]) + dt_bias[h];
        const float sp = a > 20.f ? a : log1pf(expf(a));
        dd[(size_t)h * n_rows + row] = make_float4(1.f / (1.f + expf(-b)), expf(-expf(a_log[h]) * sp),
                                                   dots[h / (H / G)], 0.f);
    }
}

IB_EXPORT int ib_delta_prepare(const void* x, int x_stride, int act_dtype, int c_off, int b_off, int a_off,
                               const float* w, int taps, float* state, long long state_stride, const int* row_entry,
                               const int* cu_rows, const int* slot_ids, const float* a_log, const float* dt_bias,
                               void* kq, float* vo, void* dd, int n_rows, int n_entries, int G, int H, int dk, int dv,
                               void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x || !a_log || !dt_bias || !kq || !vo || !dd || G <= 0 || H <= 0 || H % G || dk <= 0 || dv <= 0 || taps < 0 ||
        taps > IB_MAX_TAPS || ((uintptr_t)kq & 7) || ((uintptr_t)dd & 15))
        return IB_ERR_BAD_ARG;
    if (taps >= 1 && !w) return IB_ERR_BAD_ARG;
    if (taps > 1 && (!state || !row_entry || !cu_rows || !slot_ids || n_entries <= 0)) return IB_ERR_BAD_ARG;
    const int C = 2 * G * dk + H * dv;
    const size_t smem = (size_t)(C + G) * sizeof(float);
    if (smem > 200 * 1024) return IB_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = C >= 2048 ? 512 : 256;
    const int gy = min(64, (C + 127) / 128);
    cudaError_t le;
    if (act_dtype == 0) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(delta_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        le = launch_kernel(delta_prepare_kernel<float>, dim3(n_rows), dim3(threads), smem, s, (const float*)x, x_stride,
                           c_off, b_off, a_off, w, taps, (const float*)state, state_stride, row_entry, cu_rows,
                           slot_ids, a_log, dt_bias, (float2*)kq, vo, (float4*)dd, n_rows, G, H, dk, dv);
        if (le == cudaSuccess && taps > 1)
            le = launch_kernel(conv_state_kernel<float>, dim3(n_entries, gy), dim3(128), 0, s, (const float*)x + c_off,
                               x_stride, state, state_stride, cu_rows, slot_ids, C, taps);
    } else if (act_dtype == 1) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(delta_prepare_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        le = launch_kernel(delta_prepare_kernel<bf16>, dim3(n_rows), dim3(threads), smem, s, (const bf16*)x, x_stride,
                           c_off, b_off, a_off, w, taps, (const float*)state, state_stride, row_entry, cu_rows,
                           slot_ids, a_log, dt_bias, (float2*)kq, vo, (float4*)dd, n_rows, G, H, dk, dv);
        if (le == cudaSuccess && taps > 1)
            le = launch_kernel(conv_state_kernel<bf16>, dim3(n_entries, gy), dim3(128), 0, s, (const bf16*)x + c_off,
                               x_stride, state, state_stride, cu_rows, slot_ids, C, taps);
    } else {
        return IB_ERR_UNSUPPORTED;
    }
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
// rope_norm_append: rows of x hold nh query heads of hd, then nkv key heads of
// hd, then nkv value heads of hdv.  One warp per (row, head):
//   the head's bias is added (bias: one vector over the whole row, or null);
//   queries and keys: the first rd dimensions are rotated, dimension i with
//   i + rd/2, by the angle position * inv_freq[i] (32-bit product, sincosf);
//   with `norm_qk` they are then divided by sqrt(mean(.^2) + eps) over hd;
//   values: with `norm_v` divided by sqrt(mean(.^2) + eps) over hdv.
// Queries are written back in place; keys and values go to their place in the
// pages (key pool rows of hd, value pool rows of hdv).
#define IB_RNA_MAX_DIM 1024
template <typename T>
__global__ void rope_norm_append_kernel(T* __restrict__ x, int x_stride, const float* __restrict__ bias,
                                        const float* __restrict__ inv_freq, int rd, int norm_qk, int norm_v,
                                        float eps, const int* __restrict__ positions,
                                        const int* __restrict__ row_entry, const int* __restrict__ block_tables,
                                        int max_blocks, T* __restrict__ k_pool, T* __restrict__ v_pool, int n_rows,
                                        int nh, int nkv, int hd, int hdv, int page_size, int num_pages,
                                        unsigned* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float hbuf[];  // [warps][max(hd, hdv)]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per_row = nh + 2 * nkv;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long long)n_rows * per_row) return;
    const int row = (int)(item / per_row), head = (int)(item % per_row);
    const bool is_v = head >= nh + nkv;
    const int d = is_v ? hdv : hd;
    const int col = is_v ? (nh + nkv) * hd + (head - nh - nkv) * hdv : head * hd;
    float* buf = hbuf + (size_t)warp * max(hd, hdv);
    T* p = x + (size_t)row * x_stride + col;
    for (int i = lane; i < d; i += 32) buf[i] = to_f32(p[i]) + (bias ? bias[col + i] : 0.f);
    __syncwarp();
    const int pos = positions[row];
    if (!is_v && rd > 0) {
        const int rhalf = rd / 2;
        for (int i = lane; i < rhalf; i += 32) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            const float a = buf[i], b = buf[i + rhalf];
            buf[i] = a * cs - b * sn;
            buf[i + rhalf] = b * cs + a * sn;
        }
        __syncwarp();
    }
    float inv = 1.f;
    if (is_v ? norm_v : norm_qk) {
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) ss = fmaf(buf[i], buf[i], ss);
        ss = warp_sum(ss);
        inv = 1.f / sqrtf(ss / (float)d + eps);
    }
    if (head < nh) {
        for (int i = lane; i < d; i += 32) p[i] = from_f32<T>(buf[i] * inv);
        return;
    }
    const int e = row_entry[row];
    const int slot_idx = pos / page_size;
    const int page = (pos >= 0 && slot_idx < max_blocks) ? block_tables[(size_t)e * max_blocks + slot_idx] : -1;
    if (page < 0 || page >= num_pages) {
        if (lane == 0) atomicOr(err, IB_FLAG_BAD_PAGE);
        return;
    }
    const int g = is_v ? head - nh - nkv : head - nh;
    T* dst = (is_v ? v_pool : k_pool) + (((size_t)page * nkv + g) * page_size + (pos % page_size)) * d;
    for (int i = lane; i < d; i += 32) dst[i] = from_f32<T>(buf[i] * inv);
}

IB_EXPORT int ib_rope_norm_append(void* x, int x_stride, int act_dtype, const float* bias, const float* inv_freq,
                                  int rd, int norm_qk, int norm_v, float eps, const int* positions,
                                  const int* row_entry, const int* block_tables, int max_blocks, void* k_pool,
                                  void* v_pool, int n_rows, int nh, int nkv, int hd, int hdv, int page_size,
                                  int num_pages, unsigned* err, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x || !positions || !row_entry || !block_tables || !k_pool || !v_pool || !err || nh <= 0 || nkv <= 0 ||
        hd <= 0 || hdv <= 0 || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || rd < 0 || rd > hd || (rd & 1) ||
        (rd > 0 && !inv_freq) || ((norm_qk || norm_v) && !(eps > 0.f)))
        return IB_ERR_BAD_ARG;
    if (hd > IB_RNA_MAX_DIM || hdv > IB_RNA_MAX_DIM) return IB_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    const long long items = (long long)n_rows * (nh + 2 * nkv);
    const unsigned grid = (unsigned)((items + 3) / 4);
    const size_t smem = (size_t)4 * max(hd, hdv) * sizeof(float);
    cudaError_t le;
    if (act_dtype == 0)
        le = launch_kernel(rope_norm_append_kernel<float>, dim3(grid), dim3(128), smem, s, (float*)x, x_stride, bias,
                           inv_freq, rd, norm_qk, norm_v, eps, positions, row_entry, block_tables, max_blocks,
                           (float*)k_pool, (float*)v_pool, n_rows, nh, nkv, hd, hdv, page_size, num_pages, err);
    else if (act_dtype == 1)
        le = launch_kernel(rope_norm_append_kernel<bf16>, dim3(grid), dim3(128), smem, s, (bf16*)x, x_stride, bias,
                           inv_freq, rd, norm_qk, norm_v, eps, positions, row_entry, block_tables, max_blocks,
                           (bf16*)k_pool, (bf16*)v_pool, n_rows, nh, nkv, hd, hdv, page_size, num_pages, err);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
