// Token-by-token scans of recurrent mixers whose per-head state is a matrix of
// ROWS x P 32-bit floats (ROWS = IB_ROWS, fixed when this file is compiled; P at
// run time).  The state lives in the request's state slot and is carried from
// step to step; inside a step the tokens of an entry are walked in order, so a
// position's result is the same however the prompt was cut.
//
//   wkv:  o_t[j] = sum_i r_t[i] (S[i][j] + u[i] k_t[i] v_t[j])        (u only for the current token)
//         S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j]
//   ssd:  S[n][p] <- a_t S[n][p] + B_t[n] (dt_t x_t[p]),   y_t[p] = sum_n C_t[n] S[n][p] + D x_t[p]
//   delta: S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//         (a gated delta rule; o_t is taken from the state after its update)
//
// Everything a token brings - (r, k, w, u k) per key channel and v for wkv; (B, C)
// per state row, x, and (dt, a) per head for ssd - has been made in 32-bit by a
// parallel pass before (recurrent.cu: wkv_prepare, ssd_prepare), so the scan only
// copies: CHUNK tokens at a time go to shared memory by cp.async, two stages deep,
// while the tokens of the chunk before are walked.
//
// The prepared arrays are laid out by head (or group), then token, so what a CTA
// needs of a chunk is one contiguous run: [head][token][ROWS] factors, [head]
// [token][P] values, and for ssd [group][token][ROWS] (B, C) and [head][token]
// (dt, a).  The state is stored column by column, [head][P][ROWS], so the lanes
// of a column read and write neighbouring floats.
//
// One CTA per (entry, head, slice of columns).  A column j of the state is held
// by SPLIT neighbouring lanes, each with ROWS / SPLIT rows in registers (row
// i = ii * SPLIT + part); the partial sums of the SPLIT lanes meet by shuffles in
// a fixed order, so a column's arithmetic is the same in every slicing and batch.
// A token's arithmetic is a short dependent chain, so the scan lives on many
// warps per SM: SPLIT is as wide as the rows allow.
//
// Launch.  The package's kernels start as programmatic dependents, under their
// predecessor's tail.  The scans are launched in order instead: a scan has about as
// many CTAs as the GPU has SMs and runs as long as its busiest SM, and as a
// dependent its CTAs take whichever SMs the predecessor's thousands of CTAs free
// first, several to an SM while others stay empty (a prompt step of 2,048 tokens
// at 2,048 wide, 8 layers: 10.7 ms with the scans as dependents, 7.3 ms in order).
// They let their own successor start when their tokens are done.
#include "common.cuh"

using namespace ib;

#ifndef IB_ROWS
#error "compile with -DIB_ROWS=<rows of the state matrix>"
#endif

constexpr int ROWS = IB_ROWS;
constexpr int pick_split() {
    // the widest power of two up to 16 that divides the rows and leaves a thread at least four of them
    for (int s = 16; s > 1; s >>= 1)
        if (ROWS % s == 0 && ROWS / s >= 4) return s;
    for (int s = 16; s > 1; s >>= 1)
        if (ROWS % s == 0 && ROWS / s >= 2) return s;
    return 1;
}
#ifdef IB_SCAN_SPLIT  // (tuning: -DIB_SCAN_SPLIT=n, a power of two up to 32 that divides the rows)
constexpr int SPLIT = IB_SCAN_SPLIT;
#else
constexpr int SPLIT = pick_split();
#endif
constexpr int RPT = ROWS / SPLIT;  // rows of a column one thread holds
// Tokens per stage: up to 16, a stage of per-row factors at most 16 KB (two stages and the
// values stay under the 48 KB a CTA gets without asking).  Measured at 128 rows, one prompt of
// 2,048 tokens: 8 tokens a stage 0.57 ms, 16 tokens with two tokens interleaved 0.47 ms.
#ifdef IB_SCAN_CHUNK  // (tuning: -DIB_SCAN_CHUNK=n)
constexpr int CHUNK_WKV = IB_SCAN_CHUNK, CHUNK_SSD = IB_SCAN_CHUNK;
#else
constexpr int clamp_chunk(int n) { return n >= 16 ? 16 : (n >= 8 ? 8 : (n >= 4 ? 4 : 2)); }
constexpr int CHUNK_WKV = clamp_chunk(1024 / ROWS);  // 16 bytes a row
constexpr int CHUNK_SSD = clamp_chunk(2048 / ROWS);  // 8 bytes a row
#endif
#ifdef IB_SCAN_UNROLL  // (tuning: tokens of a chunk whose instructions the compiler may interleave)
constexpr int UNROLL = IB_SCAN_UNROLL;
#else
constexpr int UNROLL = 2;
#endif
static_assert(ROWS >= 1 && ROWS <= 512, "state rows out of range");

__device__ __forceinline__ float split_sum(float v) {
#pragma unroll
    for (int o = 1; o < SPLIT; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int BYTES>
__device__ __forceinline__ void cp_async(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;\n" ::"r"(s), "l"(gmem), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

struct WkvParams {
    const float4* f;    // [heads][rows][ROWS]: r, k, w, u * k
    const float* v;     // [heads][rows][P]
    int n_rows;         // rows of the whole step
    float* state;       // request slot s, head h: state + s * state_stride + h * P * ROWS, [P][ROWS]
    long long state_stride;
    const int* cu_rows;
    const int* slot_ids;
    float* out;         // [rows][heads * P]
    int heads, P, cols; // cols: columns of one CTA
};

__global__ void __launch_bounds__(512) wkv_scan_kernel(const WkvParams p) {
    pdl_wait();
    extern __shared__ float4 smem4[];
    float4* s_f = smem4;                                             // [2][CHUNK_WKV][ROWS]
    float* s_v = reinterpret_cast<float*>(smem4 + 2 * CHUNK_WKV * ROWS);  // [2][CHUNK_WKV][cols]
    const int e = blockIdx.x, head = blockIdx.y, j0 = blockIdx.z * p.cols;
    const int first = p.cu_rows[e], end = p.cu_rows[e + 1];
    if (end <= first) return;
    const int part = threadIdx.x % SPLIT;
    const int col_raw = threadIdx.x / SPLIT;
    const bool active = col_raw < p.cols;
    const int col = active ? col_raw : p.cols - 1;
    float* st = p.state + (long long)p.slot_ids[e] * p.state_stride + (size_t)head * ROWS * p.P;
    float* sc = st + (size_t)(j0 + col) * ROWS + part;
    float S[RPT];
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) S[ii] = sc[ii * SPLIT];
    const size_t hp = (size_t)head * p.P;
    const int ldo = p.heads * p.P;
    const float4* fh = p.f + (size_t)head * p.n_rows * ROWS;
    const float* vh = p.v + (size_t)head * p.n_rows * p.P + j0;

    auto fetch = [&](int c0, int buf) {
        const int nt = min(CHUNK_WKV, end - c0);
        float4* df = s_f + buf * CHUNK_WKV * ROWS;
        float* dv = s_v + buf * CHUNK_WKV * p.cols;
        const float4* src = fh + (size_t)c0 * ROWS;  // the chunk's factors are one contiguous run
        for (int idx = threadIdx.x; idx < nt * ROWS; idx += blockDim.x) cp_async<16>(df + idx, src + idx);
        for (int idx = threadIdx.x; idx < nt * p.cols; idx += blockDim.x)
            cp_async<4>(dv + idx, vh + (size_t)(c0 + idx / p.cols) * p.P + idx % p.cols);
        cp_async_commit();
    };
    fetch(first, 0);
    int buf = 0;
    for (int c0 = first; c0 < end; c0 += CHUNK_WKV, buf ^= 1) {
        const int nt = min(CHUNK_WKV, end - c0);
        if (c0 + CHUNK_WKV < end) {
            fetch(c0 + CHUNK_WKV, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const float4* cf = s_f + buf * CHUNK_WKV * ROWS + part;
        const float* cv = s_v + buf * CHUNK_WKV * p.cols + col;
#pragma unroll UNROLL
        for (int t = 0; t < nt; ++t) {
            const float vj = cv[t * p.cols];
            const float4* f = cf + t * ROWS;
            float acc = 0.f;
#pragma unroll
            for (int ii = 0; ii < RPT; ++ii) {
                const float4 q = f[ii * SPLIT];
                acc = fmaf(q.x, fmaf(q.w, vj, S[ii]), acc);
                S[ii] = fmaf(q.z, S[ii], q.y * vj);
            }
            acc = split_sum(acc);
            if (active && part == 0) p.out[(size_t)(c0 + t) * ldo + hp + j0 + col] = acc;
        }
        __syncthreads();  // this stage is refilled by the fetch after next
    }
    pdl_trigger();
    if (active) {
#pragma unroll
        for (int ii = 0; ii < RPT; ++ii) sc[ii * SPLIT] = S[ii];
    }
}

struct SsdParams {
    const float* x;     // [heads][rows][P]
    const float2* bc;   // [groups][rows][ROWS]: B, C
    const float2* dd;   // [heads][rows]: dt, exp(-exp(A_log) dt)
    int n_rows;         // rows of the whole step
    const float* d_skip;
    float* state;
    long long state_stride;
    const int* cu_rows;
    const int* slot_ids;
    float* out;         // [rows][heads * P]
    int heads, groups, P, cols;
};

__global__ void __launch_bounds__(512) ssd_scan_kernel(const SsdParams p) {
    pdl_wait();
    extern __shared__ float4 smem4[];
    float2* s_bc = reinterpret_cast<float2*>(smem4);       // [2][CHUNK_SSD][ROWS]
    float2* s_dd = s_bc + 2 * CHUNK_SSD * ROWS;                 // [2][CHUNK_SSD]
    float* s_x = reinterpret_cast<float*>(s_dd + 2 * CHUNK_SSD);  // [2][CHUNK_SSD][cols]
    const int e = blockIdx.x, head = blockIdx.y, j0 = blockIdx.z * p.cols;
    const int first = p.cu_rows[e], end = p.cu_rows[e + 1];
    if (end <= first) return;
    const int part = threadIdx.x % SPLIT;
    const int col_raw = threadIdx.x / SPLIT;
    const bool active = col_raw < p.cols;
    const int col = active ? col_raw : p.cols - 1;
    float* st = p.state + (long long)p.slot_ids[e] * p.state_stride + (size_t)head * ROWS * p.P;
    float* sc = st + (size_t)(j0 + col) * ROWS + part;
    float S[RPT];
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) S[ii] = sc[ii * SPLIT];
    const int inner = p.heads * p.P;
    const int grp = head / (p.heads / p.groups);
    const float dsk = p.d_skip[head];
    const float2* bg = p.bc + (size_t)grp * p.n_rows * ROWS;
    const float* xh = p.x + (size_t)head * p.n_rows * p.P + j0;
    const float2* dh = p.dd + (size_t)head * p.n_rows;

    auto fetch = [&](int c0, int buf) {
        const int nt = min(CHUNK_SSD, end - c0);
        float2* db = s_bc + buf * CHUNK_SSD * ROWS;
        float* dx = s_x + buf * CHUNK_SSD * p.cols;
        const float2* src = bg + (size_t)c0 * ROWS;  // the chunk's (B, C) are one contiguous run
        if (ROWS % 2 == 0) {
            for (int idx = threadIdx.x; idx < nt * (ROWS / 2); idx += blockDim.x)
                cp_async<16>(db + 2 * idx, src + 2 * idx);
        } else {
            for (int idx = threadIdx.x; idx < nt * ROWS; idx += blockDim.x) cp_async<8>(db + idx, src + idx);
        }
        for (int idx = threadIdx.x; idx < nt * p.cols; idx += blockDim.x)
            cp_async<4>(dx + idx, xh + (size_t)(c0 + idx / p.cols) * p.P + idx % p.cols);
        if (threadIdx.x < nt) cp_async<8>(s_dd + buf * CHUNK_SSD + threadIdx.x, dh + c0 + threadIdx.x);
        cp_async_commit();
    };
    fetch(first, 0);
    int buf = 0;
    for (int c0 = first; c0 < end; c0 += CHUNK_SSD, buf ^= 1) {
        const int nt = min(CHUNK_SSD, end - c0);
        if (c0 + CHUNK_SSD < end) {
            fetch(c0 + CHUNK_SSD, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const float2* cb = s_bc + buf * CHUNK_SSD * ROWS + part;
        const float* cx = s_x + buf * CHUNK_SSD * p.cols + col;
        const float2* cd = s_dd + buf * CHUNK_SSD;
#pragma unroll UNROLL
        for (int t = 0; t < nt; ++t) {
            const float xj = cx[t * p.cols];
            const float2 d = cd[t];
            const float dtx = d.x * xj;
            const float2* f = cb + t * ROWS;
            float acc = 0.f;
#pragma unroll
            for (int ii = 0; ii < RPT; ++ii) {
                const float2 q = f[ii * SPLIT];
                S[ii] = fmaf(d.y, S[ii], q.x * dtx);
                acc = fmaf(q.y, S[ii], acc);
            }
            acc = split_sum(acc);
            if (active && part == 0)
                p.out[(size_t)(c0 + t) * inner + (size_t)head * p.P + j0 + col] = fmaf(dsk, xj, acc);
        }
        __syncthreads();
    }
    pdl_trigger();
    if (active) {
#pragma unroll
        for (int ii = 0; ii < RPT; ++ii) sc[ii * SPLIT] = S[ii];
    }
}

// The delta rule per column j of S, with the dot products taken on the state as
// the token finds it so that the two of them run side by side instead of one
// after the other:
//   a = k . S_j,  b = q . S_j;   u = beta (v_j - g a);   o_j = g b + (k . q) u;   S_j <- g S_j + k u
// which is S' = g S + k u^T and o = S'^T q written out (k . q comes prepared).
struct DeltaParams {
    const float* v;     // [heads][rows][P]
    const float2* kq;   // [groups][rows][ROWS]: k, q (unit length; q scaled)
    const float4* dd;   // [heads][rows]: beta, g, k . q, unused
    int n_rows;
    float* state;
    long long state_stride;
    const int* cu_rows;
    const int* slot_ids;
    float* out;         // [rows][heads * P]
    int heads, groups, P, cols;
};

__global__ void __launch_bounds__(512) delta_scan_kernel(const DeltaParams p) {
    pdl_wait();
    extern __shared__ float4 smem4[];
    float4* s_dd = smem4;                                             // [2][CHUNK_SSD]
    float2* s_kq = reinterpret_cast<float2*>(s_dd + 2 * CHUNK_SSD);   // [2][CHUNK_SSD][ROWS]
    float* s_v = reinterpret_cast<float*>(s_kq + 2 * CHUNK_SSD * ROWS);  // [2][CHUNK_SSD][cols]
    const int e = blockIdx.x, head = blockIdx.y, j0 = blockIdx.z * p.cols;
    const int first = p.cu_rows[e], end = p.cu_rows[e + 1];
    if (end <= first) return;
    const int part = threadIdx.x % SPLIT;
    const int col_raw = threadIdx.x / SPLIT;
    const bool active = col_raw < p.cols;
    const int col = active ? col_raw : p.cols - 1;
    float* st = p.state + (long long)p.slot_ids[e] * p.state_stride + (size_t)head * ROWS * p.P;
    float* sc = st + (size_t)(j0 + col) * ROWS + part;
    float S[RPT];
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) S[ii] = sc[ii * SPLIT];
    const int inner = p.heads * p.P;
    const int grp = head / (p.heads / p.groups);
    const float2* kg = p.kq + (size_t)grp * p.n_rows * ROWS;
    const float* vh = p.v + (size_t)head * p.n_rows * p.P + j0;
    const float4* dh = p.dd + (size_t)head * p.n_rows;

    auto fetch = [&](int c0, int buf) {
        const int nt = min(CHUNK_SSD, end - c0);
        float2* dk = s_kq + buf * CHUNK_SSD * ROWS;
        float* dv = s_v + buf * CHUNK_SSD * p.cols;
        const float2* src = kg + (size_t)c0 * ROWS;  // the chunk's (k, q) are one contiguous run
        if (ROWS % 2 == 0) {
            for (int idx = threadIdx.x; idx < nt * (ROWS / 2); idx += blockDim.x)
                cp_async<16>(dk + 2 * idx, src + 2 * idx);
        } else {
            for (int idx = threadIdx.x; idx < nt * ROWS; idx += blockDim.x) cp_async<8>(dk + idx, src + idx);
        }
        for (int idx = threadIdx.x; idx < nt * p.cols; idx += blockDim.x)
            cp_async<4>(dv + idx, vh + (size_t)(c0 + idx / p.cols) * p.P + idx % p.cols);
        if (threadIdx.x < nt) cp_async<16>(s_dd + buf * CHUNK_SSD + threadIdx.x, dh + c0 + threadIdx.x);
        cp_async_commit();
    };
    fetch(first, 0);
    int buf = 0;
    for (int c0 = first; c0 < end; c0 += CHUNK_SSD, buf ^= 1) {
        const int nt = min(CHUNK_SSD, end - c0);
        if (c0 + CHUNK_SSD < end) {
            fetch(c0 + CHUNK_SSD, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const float2* ck = s_kq + buf * CHUNK_SSD * ROWS + part;
        const float* cv = s_v + buf * CHUNK_SSD * p.cols + col;
        const float4* cd = s_dd + buf * CHUNK_SSD;
#pragma unroll UNROLL
        for (int t = 0; t < nt; ++t) {
            const float vj = cv[t * p.cols];
            const float4 d = cd[t];  // beta, g, k . q
            const float2* f = ck + t * ROWS;
            float2 kqr[RPT];
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int ii = 0; ii < RPT; ++ii) {
                kqr[ii] = f[ii * SPLIT];
                a = fmaf(kqr[ii].x, S[ii], a);
                b = fmaf(kqr[ii].y, S[ii], b);
            }
            a = split_sum(a);
            b = split_sum(b);
            const float u = d.x * (vj - d.y * a);
#pragma unroll
            for (int ii = 0; ii < RPT; ++ii) S[ii] = fmaf(d.y, S[ii], kqr[ii].x * u);
            if (active && part == 0)
                p.out[(size_t)(c0 + t) * inner + (size_t)head * p.P + j0 + col] = fmaf(d.y, b, d.z * u);
        }
        __syncthreads();
    }
    pdl_trigger();
    if (active) {
#pragma unroll
        for (int ii = 0; ii < RPT; ++ii) sc[ii * SPLIT] = S[ii];
    }
}

IB_EXPORT int ib_scan_rows() { return ROWS; }
IB_EXPORT int ib_scan_split() { return SPLIT; }

static int scan_geometry(int P, int col_slices, int* cols, int* threads) {
    if (P <= 0 || col_slices <= 0 || P % col_slices) return IB_ERR_BAD_ARG;
    *cols = P / col_slices;
    *threads = ((*cols * SPLIT + 31) / 32) * 32;
    if (*threads > 512) return IB_ERR_TOO_LARGE;
    return IB_OK;
}

// f: float4 [heads][rows][ROWS]; v: float32 [heads][rows][P]; out: float32 [rows][heads * P].
// `col_slices` CTAs share the columns of a head (it must divide P).
IB_EXPORT int ib_wkv_scan(const void* f, const float* v, int n_rows, float* state, long long state_stride,
                          const int* cu_rows, const int* slot_ids, float* out, int n_entries, int heads, int P,
                          int col_slices, void* stream) {
    if (n_entries <= 0) return IB_OK;
    if (!f || !v || !state || !cu_rows || !slot_ids || !out || heads <= 0 || ((uintptr_t)f & 15)) return IB_ERR_BAD_ARG;
    int cols, threads;
    const int g = scan_geometry(P, col_slices, &cols, &threads);
    if (g != IB_OK) return g;
    WkvParams p{(const float4*)f, v, n_rows, state, state_stride, cu_rows, slot_ids, out, heads, P, cols};
    const size_t smem = 2 * ((size_t)CHUNK_WKV * ROWS * sizeof(float4) + (size_t)CHUNK_WKV * cols * sizeof(float));
    if (smem > 48 * 1024) return IB_ERR_TOO_LARGE;
    cudaError_t le = launch_kernel_in_order(wkv_scan_kernel, dim3(n_entries, heads, col_slices), dim3(threads), smem,
                                   (cudaStream_t)stream, p);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// x: float32 [heads][rows][P]; bc: float2 [groups][rows][ROWS]; dd: float2 [heads][rows];
// out: float32 [rows][heads * P].
IB_EXPORT int ib_ssd_scan(const float* x, const void* bc, const void* dd, int n_rows, const float* d_skip,
                          float* state, long long state_stride, const int* cu_rows, const int* slot_ids, float* out,
                          int n_entries, int heads, int groups, int P, int col_slices, void* stream) {
    if (n_entries <= 0) return IB_OK;
    if (!x || !bc || !dd || !d_skip || !state || !cu_rows || !slot_ids || !out || heads <= 0 || groups <= 0 ||
        heads % groups || ((uintptr_t)bc & 15) || ((uintptr_t)dd & 7))
        return IB_ERR_BAD_ARG;
    int cols, threads;
    const int g = scan_geometry(P, col_slices, &cols, &threads);
    if (g != IB_OK) return g;
    SsdParams p{x, (const float2*)bc, (const float2*)dd, n_rows, d_skip, state, state_stride, cu_rows, slot_ids, out,
                heads, groups, P, cols};
    const size_t smem = 2 * ((size_t)CHUNK_SSD * ROWS * sizeof(float2) + (size_t)CHUNK_SSD * sizeof(float2) +
                             (size_t)CHUNK_SSD * cols * sizeof(float));
    if (smem > 48 * 1024) return IB_ERR_TOO_LARGE;
    cudaError_t le = launch_kernel_in_order(ssd_scan_kernel, dim3(n_entries, heads, col_slices), dim3(threads), smem,
                                   (cudaStream_t)stream, p);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// v: float32 [heads][rows][P]; kq: float2 [groups][rows][ROWS]; dd: float4 [heads][rows];
// out: float32 [rows][heads * P].
IB_EXPORT int ib_delta_scan(const float* v, const void* kq, const void* dd, int n_rows, float* state,
                            long long state_stride, const int* cu_rows, const int* slot_ids, float* out,
                            int n_entries, int heads, int groups, int P, int col_slices, void* stream) {
    if (n_entries <= 0) return IB_OK;
    if (!v || !kq || !dd || !state || !cu_rows || !slot_ids || !out || heads <= 0 || groups <= 0 || heads % groups ||
        ((uintptr_t)kq & 15) || ((uintptr_t)dd & 15))
        return IB_ERR_BAD_ARG;
    int cols, threads;
    const int g = scan_geometry(P, col_slices, &cols, &threads);
    if (g != IB_OK) return g;
    DeltaParams p{v, (const float2*)kq, (const float4*)dd, n_rows, state, state_stride, cu_rows, slot_ids, out,
                  heads, groups, P, cols};
    const size_t smem = 2 * ((size_t)CHUNK_SSD * ROWS * sizeof(float2) + (size_t)CHUNK_SSD * sizeof(float4) +
                             (size_t)CHUNK_SSD * cols * sizeof(float));
    if (smem > 48 * 1024) return IB_ERR_TOO_LARGE;
    cudaError_t le = launch_kernel_in_order(delta_scan_kernel, dim3(n_entries, heads, col_slices), dim3(threads), smem,
                                            (cudaStream_t)stream, p);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
