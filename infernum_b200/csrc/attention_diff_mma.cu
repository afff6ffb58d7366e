// Differential attention on the tensor cores (bf16 mma.sync m16n8k16), for prompts and decoded
// tokens alike.  Compiled per (DIFF_D, DIFF_E): the size of one score map and of a value.
//
//   o(i) = sum_j w(i, j) v(j),   w = softmax(s_1)(i, j) - lambda * softmax(s_2)(i, j),   j <= i
//   s_m = cap * tanh(q_m . k_m * scale / cap);   out = o / sqrt(mean(o^2) + eps) * out_scale
//
// The two maps have their own maxima and denominators, so two accumulators would be the
// straight way; with values twice as wide as a map they do not fit a warp's registers.  The
// kernel walks the keys twice instead: the first walk computes both maps' scores and keeps
// only each row's two maxima and denominators; the second computes the scores again, forms
// the final signed weights w (32-bit, rounded to bf16 for the product as the package's other
// bf16 attention kernels round their probabilities) and accumulates one product w V.  The
// multiply-adds are the same as with two accumulators (two score products more, one value
// product less), the keys are read twice.
//
// A CTA (four warps) takes 64 packed rows - (query row, head of the group) pairs that share a
// key/value head - of one entry; a warp 16 of them.  Keys come in tiles of 32 that start at
// absolute multiples of 32 whatever the step's cut, through the block table, by cp.async into
// padded shared memory, two stages: a tile is fetched while the one before it is computed on.
// Rows beyond the last key any row of the CTA sees are zero-filled, so what an earlier user
// left in a page never meets a zero weight.
//
// Steps of few rows (decoded tokens) would leave one CTA per entry and key/value head walking
// all keys alone.  For those the keys are cut in slices over several CTAs and the two walks
// become two launches: the first writes every slice's maxima and denominators, the second
// merges them, walks its slice again and writes its share of w V in 32-bit; a third kernel
// adds the shares in slice order and norms.
#include "common.cuh"

using namespace ib;

#ifndef DIFF_D
#define DIFF_D 128
#endif
#ifndef DIFF_E
#define DIFF_E 256
#endif

namespace {
constexpr int D = DIFF_D, E = DIFF_E, KW = 2 * DIFF_D;
constexpr int BM = 64, BN = 32, WARPS = 4, THREADS = WARPS * 32;
constexpr int QS = KW + 8, KS = KW + 8, VS = E + 8;  // row strides in shared memory (elements): 16 bytes of padding
constexpr int NT_E = E / 8;                          // accumulator tiles of 8 columns
static_assert(D % 16 == 0 && E % 16 == 0 && D >= 16 && E >= 16 && E <= 256 && D <= 256, "sizes this kernel takes");

__device__ __forceinline__ void ldsm_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const bf16* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const bf16* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}
__device__ __forceinline__ void cp_async16(bf16* smem, const bf16* gmem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(gmem));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
// all but the newest group of copies have landed
__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }

// One tile of keys (and, with_v, values) into shared memory; rows of keys beyond `last_key` are zeros.
__device__ __forceinline__ void load_tile(bf16* ks, bf16* vs, const bf16* __restrict__ k_pool,
                                          const bf16* __restrict__ v_pool, const int* __restrict__ table, int max_blocks,
                                          int j0, int last_key, int g, int nkv, int page_size, int num_pages,
                                          bool with_v, unsigned* err) {
    constexpr int KC = KW / 8, VC = E / 8;  // 16-byte chunks in a row
    for (int c = threadIdx.x; c < BN * KC; c += THREADS) {
        const int key = c / KC, part = c % KC, j = j0 + key;
        bf16* dst = ks + key * KS + part * 8;
        int page = -1;
        if (j <= last_key) {
            page = j / page_size < max_blocks ? table[j / page_size] : -1;
            if (page < 0 || page >= num_pages) {
                if (part == 0) atomicOr(err, IB_FLAG_BAD_PAGE);
                page = -1;
            }
        }
        if (page >= 0)
            cp_async16(dst, k_pool + (((size_t)page * nkv + g) * page_size + (j % page_size)) * KW + part * 8);
        else
            *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    if (with_v) {
        for (int c = threadIdx.x; c < BN * VC; c += THREADS) {
            const int key = c / VC, part = c % VC, j = j0 + key;
            bf16* dst = vs + key * VS + part * 8;
            int page = -1;
            if (j <= last_key) {
                page = j / page_size < max_blocks ? table[j / page_size] : -1;
                if (page < 0 || page >= num_pages) page = -1;
            }
            if (page >= 0)
                cp_async16(dst, v_pool + (((size_t)page * nkv + g) * page_size + (j % page_size)) * E + part * 8);
            else
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
}

// Both maps' scores of a warp's 16 rows against the tile's 32 keys: s[map][tile of 8 keys][4].
__device__ __forceinline__ void scores(float (&s)[2][4][4], const bf16* qs_warp, const bf16* ks, int lane) {
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[m][n][i] = 0.f;
    const int a_row = lane & 15, a_col = (lane >> 4) * 8;
    const int b_key = ((lane >> 4) * 8) + (lane & 7), b_col = ((lane >> 3) & 1) * 8;
    // (the two maps side by side in every step: eight accumulators between two uses of one)
#pragma unroll 4
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            unsigned a[4];
            ldsm_x4(a[0], a[1], a[2], a[3], qs_warp + a_row * QS + m * D + kk * 16 + a_col);
#pragma unroll
            for (int pr = 0; pr < 2; ++pr) {
                unsigned b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3, ks + (pr * 16 + b_key) * KS + m * D + kk * 16 + b_col);
                mma_bf16(s[m][2 * pr], a, b0, b1);
                mma_bf16(s[m][2 * pr + 1], a, b2, b3);
            }
        }
    }
}

// cap * tanh(s * scale / cap) with tanh(x) = 1 - 2 / (exp(2 x) + 1) on the fast exponential and division
// (absolute error of a score some 1e-7 of the cap; |x| beyond 15 is +-1 in 32-bit anyway).
__device__ __forceinline__ float capped(float s, float scale, float cap, float inv_cap) {
    s *= scale;
    if (cap <= 0.f) return s;
    const float x = fminf(fmaxf(s * inv_cap, -15.f), 15.f);
    return cap * (1.f - __fdividef(2.f, __expf(2.f * x) + 1.f));
}

// MODE 0: both walks over all keys, the normed result to `out`.  MODE 1: the first walk over the
// CTA's slice of the keys; maxima and denominators to `stats` [splits][rows][heads][4].  MODE 2:
// the slices' maxima and denominators merged, the second walk over the CTA's slice, its share
// of w V to `part` [splits][rows][heads][E] (32-bit, not normed).
template <int MODE>
__global__ void __launch_bounds__(THREADS, 2)
attention_diff_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                          bf16* __restrict__ out, const int* __restrict__ cu_rows, const int* __restrict__ positions,
                          const int* __restrict__ block_tables, int max_blocks, int nh, int nkv, int page_size,
                          int num_pages, float scale, float cap, float lambda, float eps, float out_scale,
                          unsigned* __restrict__ err, int splits, int slice_len, int n_total_rows,
                          float* __restrict__ stats, float* __restrict__ part) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* ks_all = qs + BM * QS;           // two stages of keys
    bf16* vs_all = ks_all + 2 * BN * KS;   // two stages of values
    const int en = blockIdx.y, g = MODE == 0 ? blockIdx.z : blockIdx.z / splits;
    const int sp = MODE == 0 ? 0 : blockIdx.z % splits;
    const int R = nh / nkv;
    const int row0 = cu_rows[en], n_rows = cu_rows[en + 1] - row0;
    const int n_packed = n_rows * R;
    // (the row tiles that see the most keys start first)
    const int tile0 = (int)(gridDim.x - 1 - blockIdx.x) * BM;
    if (tile0 >= n_packed) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, tq = lane & 3;
    const int* table = block_tables + (size_t)en * max_blocks;
    const int pos0 = positions[row0];  // an entry's rows are consecutive positions
    const int packed_here = min(BM, n_packed - tile0);
    const int last_seen = pos0 + (tile0 + packed_here - 1) / R;  // what the CTA's last row sees
    const int first_key = MODE == 0 ? 0 : sp * slice_len;         // (slices are multiples of a tile)
    const int last_key = MODE == 0 ? last_seen : min(last_seen, first_key + slice_len - 1);

    // queries: packed row p = (row p / R, head g R + p % R), both maps side by side
    {
        constexpr int QC = KW / 8;
        for (int c = threadIdx.x; c < BM * QC; c += THREADS) {
            const int r = c / QC, part = c % QC, p = tile0 + r;
            bf16* dst = qs + r * QS + part * 8;
            if (p < n_packed)
                cp_async16(dst, q + ((size_t)(row0 + p / R) * nh + g * R + p % R) * KW + part * 8);
            else
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
    const bf16* qs_warp = qs + warp * 16 * QS;
    const int p_lo = tile0 + warp * 16 + gq, p_hi = p_lo + 8;
    const int pos_lo = p_lo < n_packed ? pos0 + p_lo / R : -1, pos_hi = p_hi < n_packed ? pos0 + p_hi / R : -1;
    const int warp_last = min(tile0 + warp * 16 + 15, n_packed - 1);
    const int warp_last_key = tile0 + warp * 16 < n_packed ? pos0 + warp_last / R : -1;  // -1: the warp has no row
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;

    // ---- first walk: maxima and denominators of both maps
    float mx[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}}, den[2][2] = {{0.f, 0.f}, {0.f, 0.f}};  // [map][lo, hi]
    const int n_tiles = last_key >= first_key ? (last_key - first_key) / BN + 1 : 0;
    if (MODE != 2 && n_tiles > 0) {
        load_tile(ks_all, vs_all, k_pool, v_pool, table, max_blocks, first_key, last_key, g, nkv, page_size, num_pages,
                  false, err);
        cp_async_commit();
    }
    for (int t = 0; MODE != 2 && t < n_tiles; ++t) {
        const int j0 = first_key + t * BN;
        const bf16* ks = ks_all + (t & 1) * BN * KS;
        if (t + 1 < n_tiles) {
            load_tile(ks_all + ((t + 1) & 1) * BN * KS, vs_all, k_pool, v_pool, table, max_blocks, j0 + BN, last_key, g,
                      nkv, page_size, num_pages, false, err);
            cp_async_commit();
            cp_async_wait_but_one();
        } else {
            cp_async_wait_all();
        }
        __syncthreads();
        if (j0 <= warp_last_key) {  // (the whole warp)
        float s[2][4][4];
        scores(s, qs_warp, ks, lane);
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float t_lo = -INFINITY, t_hi = -INFINITY;
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int j = j0 + n * 8 + 2 * tq + (i & 1);
                    const bool hi = i >= 2;
                    const float v = j <= (hi ? pos_hi : pos_lo) ? capped(s[m][n][i], scale, cap, inv_cap) : -INFINITY;
                    s[m][n][i] = v;
                    if (hi) t_hi = fmaxf(t_hi, v); else t_lo = fmaxf(t_lo, v);
                }
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 1));
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 2));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 1));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 2));
            const float n_lo = fmaxf(mx[m][0], t_lo), n_hi = fmaxf(mx[m][1], t_hi);
            float a_lo = 0.f, a_hi = 0.f;
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float v = s[m][n][i];
                    if (v != -INFINITY) {
                        if (i >= 2) a_hi += __expf(v - n_hi); else a_lo += __expf(v - n_lo);
                    }
                }
            a_lo += __shfl_xor_sync(0xffffffffu, a_lo, 1);
            a_lo += __shfl_xor_sync(0xffffffffu, a_lo, 2);
            a_hi += __shfl_xor_sync(0xffffffffu, a_hi, 1);
            a_hi += __shfl_xor_sync(0xffffffffu, a_hi, 2);
            den[m][0] = (n_lo == -INFINITY ? 0.f : den[m][0] * expf(mx[m][0] - n_lo)) + a_lo;
            den[m][1] = (n_hi == -INFINITY ? 0.f : den[m][1] * expf(mx[m][1] - n_hi)) + a_hi;
            mx[m][0] = n_lo;
            mx[m][1] = n_hi;
        }
        }
        __syncthreads();  // the stage is free for the tile after the next
    }
    if (MODE == 1) {
        cp_async_wait_all();  // (the queries, when the slice held no key)
        if (tq == 0) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int p = h ? p_hi : p_lo;
                if (p < n_packed) {
                    float* dst = stats + (((size_t)sp * n_total_rows + row0 + p / R) * nh + g * R + p % R) * 4;
                    dst[0] = mx[0][h];
                    dst[1] = den[0][h];
                    dst[2] = mx[1][h];
                    dst[3] = den[1][h];
                }
            }
        }
        return;
    }
    if (MODE == 2) {
        // the slices' maxima and denominators merged in slice order
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int p = h ? p_hi : p_lo;
            if (p >= n_packed) continue;
            const float* src = stats + (((size_t)(row0 + p / R)) * nh + g * R + p % R) * 4;
            const size_t step = (size_t)n_total_rows * nh * 4;
            for (int m = 0; m < 2; ++m) {
                float best = -INFINITY;
                for (int k = 0; k < splits; ++k) best = fmaxf(best, src[k * step + 2 * m]);
                float sum = 0.f;
                for (int k = 0; k < splits; ++k) {
                    const float mk = src[k * step + 2 * m];
                    if (mk != -INFINITY) sum += src[k * step + 2 * m + 1] * expf(mk - best);
                }
                mx[m][h] = best;
                den[m][h] = sum;
            }
        }
    }
    float inv[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h) inv[m][h] = den[m][h] > 0.f ? (m == 0 ? 1.f : -lambda) / den[m][h] : 0.f;

    // ---- second walk: the signed weights and their product with the values
    float acc[NT_E][4];
#pragma unroll
    for (int n = 0; n < NT_E; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
    const int v_key = ((lane >> 3) & 1) * 8 + (lane & 7), v_col = (lane >> 4) * 8;
    if (MODE == 2 && n_tiles == 0) cp_async_wait_all();  // (the queries; nothing else follows)
    if (n_tiles > 0) {
        load_tile(ks_all, vs_all, k_pool, v_pool, table, max_blocks, first_key, last_key, g, nkv, page_size, num_pages,
                  true, err);
        cp_async_commit();
    }
    for (int t = 0; t < n_tiles; ++t) {
        const int j0 = first_key + t * BN;
        const bf16* ks = ks_all + (t & 1) * BN * KS;
        const bf16* vs = vs_all + (t & 1) * BN * VS;
        if (t + 1 < n_tiles) {
            load_tile(ks_all + ((t + 1) & 1) * BN * KS, vs_all + ((t + 1) & 1) * BN * VS, k_pool, v_pool, table, max_blocks,
                      j0 + BN, last_key, g, nkv, page_size, num_pages, true, err);
            cp_async_commit();
            cp_async_wait_but_one();
        } else {
            cp_async_wait_all();
        }
        __syncthreads();
        if (j0 <= warp_last_key) {
        float s[2][4][4];
        scores(s, qs_warp, ks, lane);
        unsigned w[4][2];  // [tile of 8 keys][lo, hi] as pairs of bf16
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            float wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int j = j0 + n * 8 + 2 * tq + (i & 1);
                const int h = i >> 1;
                float v = 0.f;
                if (j <= (h ? pos_hi : pos_lo)) {
                    v = __expf(capped(s[0][n][i], scale, cap, inv_cap) - mx[0][h]) * inv[0][h]
                        + __expf(capped(s[1][n][i], scale, cap, inv_cap) - mx[1][h]) * inv[1][h];
                }
                wv[i] = v;
            }
            w[n][0] = pack_bf16(wv[0], wv[1]);
            w[n][1] = pack_bf16(wv[2], wv[3]);
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {  // 16 keys a step
            const unsigned a[4] = {w[2 * kk][0], w[2 * kk][1], w[2 * kk + 1][0], w[2 * kk + 1][1]};
#pragma unroll
            for (int pr = 0; pr < NT_E / 2; ++pr) {
                unsigned b0, b1, b2, b3;
                ldsm_x4_trans(b0, b1, b2, b3, vs + (kk * 16 + v_key) * VS + pr * 16 + v_col);
                mma_bf16(acc[2 * pr], a, b0, b1);
                mma_bf16(acc[2 * pr + 1], a, b2, b3);
            }
        }
        }
        __syncthreads();
    }

    if (MODE == 2) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int p = h ? p_hi : p_lo;
            if (p >= n_packed) continue;
            float* dst = part + (((size_t)sp * n_total_rows + row0 + p / R) * nh + g * R + p % R) * E;
#pragma unroll
            for (int n = 0; n < NT_E; ++n)
                *reinterpret_cast<float2*>(dst + n * 8 + 2 * tq) = make_float2(acc[n][2 * h], acc[n][2 * h + 1]);
        }
        return;
    }
    // ---- each row divided by its root mean square, times out_scale
    float ss_lo = 0.f, ss_hi = 0.f;
#pragma unroll
    for (int n = 0; n < NT_E; ++n) {
        ss_lo = fmaf(acc[n][0], acc[n][0], fmaf(acc[n][1], acc[n][1], ss_lo));
        ss_hi = fmaf(acc[n][2], acc[n][2], fmaf(acc[n][3], acc[n][3], ss_hi));
    }
    ss_lo += __shfl_xor_sync(0xffffffffu, ss_lo, 1);
    ss_lo += __shfl_xor_sync(0xffffffffu, ss_lo, 2);
    ss_hi += __shfl_xor_sync(0xffffffffu, ss_hi, 1);
    ss_hi += __shfl_xor_sync(0xffffffffu, ss_hi, 2);
    const float f_lo = out_scale / sqrtf(ss_lo / (float)E + eps), f_hi = out_scale / sqrtf(ss_hi / (float)E + eps);
    if (p_lo < n_packed) {
        bf16* op = out + ((size_t)(row0 + p_lo / R) * nh + g * R + p_lo % R) * E;
#pragma unroll
        for (int n = 0; n < NT_E; ++n)
            *reinterpret_cast<unsigned*>(op + n * 8 + 2 * tq) = pack_bf16(acc[n][0] * f_lo, acc[n][1] * f_lo);
    }
    if (p_hi < n_packed) {
        bf16* op = out + ((size_t)(row0 + p_hi / R) * nh + g * R + p_hi % R) * E;
#pragma unroll
        for (int n = 0; n < NT_E; ++n)
            *reinterpret_cast<unsigned*>(op + n * 8 + 2 * tq) = pack_bf16(acc[n][2] * f_hi, acc[n][3] * f_hi);
    }
}
// The slices' shares added in slice order, each (row, head) divided by its root mean square: a warp each.
__global__ void attention_diff_merge_kernel(const float* __restrict__ part, bf16* __restrict__ out, int splits,
                                            int n_rows, int nh, float eps, float out_scale) {
    pdl_trigger();
    pdl_wait();
    const int item = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (item >= n_rows * nh) return;
    constexpr int PER = (E + 31) / 32;
    float v[PER];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = lane + 32 * i;
        float a = 0.f;
        if (c < E) {
            // four loads in flight; the sums are taken in slice order all the same
            const size_t step = (size_t)n_rows * nh * E;
            const float* src = part + (size_t)item * E + c;
            int k = 0;
            for (; k + 4 <= splits; k += 4) {
                const float p0 = src[(size_t)k * step], p1 = src[(size_t)(k + 1) * step], p2 = src[(size_t)(k + 2) * step],
                            p3 = src[(size_t)(k + 3) * step];
                a = (((a + p0) + p1) + p2) + p3;
            }
            for (; k < splits; ++k) a += src[(size_t)k * step];
        }
        v[i] = a;
        ss = fmaf(a, a, ss);
    }
    ss = warp_sum(ss);
    const float f = out_scale / sqrtf(ss / (float)E + eps);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = lane + 32 * i;
        if (c < E) out[(size_t)item * E + c] = __float2bfloat16_rn(v[i] * f);
    }
}

// ---- entries of at most 16 packed rows (decoded tokens): one walk ----------------------------
// Every warp computes both maps' scores of the same 16 rows against the tile and owns a quarter of
// the value's columns, for which it keeps both maps' running sums (two accumulators of E / 4 columns
// fit).  A CTA takes one slice of an entry's keys and writes, per row and head, both maps' maxima and
// denominators and both unnormed sums in 32-bit; the merge below weighs the slices and takes the
// difference.  The keys are read once.
constexpr int NT_W = E >= 64 ? E / 32 : 2;  // accumulator tiles of a warp's quarter (E a multiple of 64; else not run)

__global__ void __launch_bounds__(THREADS, 2)
attention_diff_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                             const int* __restrict__ cu_rows, const int* __restrict__ positions,
                             const int* __restrict__ block_tables, int max_blocks, int nh, int nkv, int page_size,
                             int num_pages, float scale, float cap, unsigned* __restrict__ err, int splits, int slice_len,
                             int n_total_rows, float* __restrict__ stats, float* __restrict__ part) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* ks_all = qs + 16 * QS;
    bf16* vs_all = ks_all + 2 * BN * KS;
    const int en = blockIdx.y, g = blockIdx.z / splits, sp = blockIdx.z % splits;
    const int R = nh / nkv;
    const int row0 = cu_rows[en], n_rows = cu_rows[en + 1] - row0;
    const int n_packed = min(n_rows * R, 16);
    if (n_packed <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, tq = lane & 3;
    const int* table = block_tables + (size_t)en * max_blocks;
    const int pos0 = positions[row0];
    const int last_seen = pos0 + (n_packed - 1) / R;
    const int first_key = sp * slice_len;
    const int last_key = min(last_seen, first_key + slice_len - 1);
    {
        constexpr int QC = KW / 8;
        for (int c = threadIdx.x; c < 16 * QC; c += THREADS) {
            const int r = c / QC, part_i = c % QC;
            bf16* dst = qs + r * QS + part_i * 8;
            if (r < n_packed)
                cp_async16(dst, q + ((size_t)(row0 + r / R) * nh + g * R + r % R) * KW + part_i * 8);
            else
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
    const int p_lo = gq, p_hi = gq + 8;
    const int pos_lo = p_lo < n_packed ? pos0 + p_lo / R : -1, pos_hi = p_hi < n_packed ? pos0 + p_hi / R : -1;
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
    float mx[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}}, den[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    float acc[2][NT_W][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < NT_W; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;
    const int v_key = ((lane >> 3) & 1) * 8 + (lane & 7), v_col = warp * (E / 4) + (lane >> 4) * 8;
    const int n_tiles = last_key >= first_key ? (last_key - first_key) / BN + 1 : 0;
    if (n_tiles > 0) {
        load_tile(ks_all, vs_all, k_pool, v_pool, table, max_blocks, first_key, last_key, g, nkv, page_size, num_pages,
                  true, err);
        cp_async_commit();
    } else {
        cp_async_wait_all();
    }
    for (int t = 0; t < n_tiles; ++t) {
        const int j0 = first_key + t * BN;
        const bf16* ks = ks_all + (t & 1) * BN * KS;
        const bf16* vs = vs_all + (t & 1) * BN * VS;
        if (t + 1 < n_tiles) {
            load_tile(ks_all + ((t + 1) & 1) * BN * KS, vs_all + ((t + 1) & 1) * BN * VS, k_pool, v_pool, table, max_blocks,
                      j0 + BN, last_key, g, nkv, page_size, num_pages, true, err);
            cp_async_commit();
            cp_async_wait_but_one();
        } else {
            cp_async_wait_all();
        }
        __syncthreads();
        float s[2][4][4];
        scores(s, qs, ks, lane);
        unsigned w[2][4][2];  // [map][tile of 8 keys][lo, hi]: the probabilities as pairs of bf16
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float t_lo = -INFINITY, t_hi = -INFINITY;
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int j = j0 + n * 8 + 2 * tq + (i & 1);
                    const bool hi = i >= 2;
                    const float v = j <= (hi ? pos_hi : pos_lo) ? capped(s[m][n][i], scale, cap, inv_cap) : -INFINITY;
                    s[m][n][i] = v;
                    if (hi) t_hi = fmaxf(t_hi, v); else t_lo = fmaxf(t_lo, v);
                }
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 1));
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 2));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 1));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 2));
            const float n_lo = fmaxf(mx[m][0], t_lo), n_hi = fmaxf(mx[m][1], t_hi);
            const float c_lo = n_lo == -INFINITY ? 0.f : __expf(mx[m][0] - n_lo);  // (exp(-inf) = 0 on the first keys)
            const float c_hi = n_hi == -INFINITY ? 0.f : __expf(mx[m][1] - n_hi);
            float a_lo = 0.f, a_hi = 0.f;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                float pv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float v = s[m][n][i];
                    pv[i] = v == -INFINITY ? 0.f : __expf(v - (i >= 2 ? n_hi : n_lo));
                }
                a_lo += pv[0] + pv[1];
                a_hi += pv[2] + pv[3];
                w[m][n][0] = pack_bf16(pv[0], pv[1]);
                w[m][n][1] = pack_bf16(pv[2], pv[3]);
            }
            a_lo += __shfl_xor_sync(0xffffffffu, a_lo, 1);
            a_lo += __shfl_xor_sync(0xffffffffu, a_lo, 2);
            a_hi += __shfl_xor_sync(0xffffffffu, a_hi, 1);
            a_hi += __shfl_xor_sync(0xffffffffu, a_hi, 2);
            den[m][0] = den[m][0] * c_lo + a_lo;
            den[m][1] = den[m][1] * c_hi + a_hi;
            mx[m][0] = n_lo;
            mx[m][1] = n_hi;
#pragma unroll
            for (int n = 0; n < NT_W; ++n) {
                acc[m][n][0] *= c_lo;
                acc[m][n][1] *= c_lo;
                acc[m][n][2] *= c_hi;
                acc[m][n][3] *= c_hi;
            }
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            const unsigned a1[4] = {w[0][2 * kk][0], w[0][2 * kk][1], w[0][2 * kk + 1][0], w[0][2 * kk + 1][1]};
            const unsigned a2[4] = {w[1][2 * kk][0], w[1][2 * kk][1], w[1][2 * kk + 1][0], w[1][2 * kk + 1][1]};
#pragma unroll
            for (int pr = 0; pr < NT_W / 2; ++pr) {
                unsigned b0, b1, b2, b3;
                ldsm_x4_trans(b0, b1, b2, b3, vs + (kk * 16 + v_key) * VS + pr * 16 + v_col);
                mma_bf16(acc[0][2 * pr], a1, b0, b1);
                mma_bf16(acc[0][2 * pr + 1], a1, b2, b3);
                mma_bf16(acc[1][2 * pr], a2, b0, b1);
                mma_bf16(acc[1][2 * pr + 1], a2, b2, b3);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int p = h ? p_hi : p_lo;
        if (p >= n_packed) continue;
        const size_t item = ((size_t)sp * n_total_rows + row0 + p / R) * nh + g * R + p % R;
        if (warp == 0 && tq == 0) {
            float* dst = stats + item * 4;
            dst[0] = mx[0][h];
            dst[1] = den[0][h];
            dst[2] = mx[1][h];
            dst[3] = den[1][h];
        }
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float* dst = part + (item * 2 + m) * E + warp * (E / 4);
#pragma unroll
            for (int n = 0; n < NT_W; ++n)
                *reinterpret_cast<float2*>(dst + n * 8 + 2 * tq) = make_float2(acc[m][n][2 * h], acc[m][n][2 * h + 1]);
        }
    }
}

// The slices of the kernel above weighed by their maxima, the difference of the two maps, the norm: a CTA
// of four warps per (row, head); warp w adds the slices w, w + 4, ... and the four sums meet in shared
// memory in warp order.
__global__ void attention_diff_decode_merge_kernel(const float* __restrict__ stats, const float* __restrict__ part,
                                                   bf16* __restrict__ out, int splits, int n_rows, int nh, float lambda,
                                                   float eps, float out_scale) {
    pdl_trigger();
    pdl_wait();
    __shared__ float sh_o[4][2][E];
    __shared__ float sh_sum[4][2];
    __shared__ float sh_ss[4];
    const int item = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t step = (size_t)n_rows * nh;
    float best[2] = {-INFINITY, -INFINITY};
    for (int k = 0; k < splits; ++k) {
        best[0] = fmaxf(best[0], stats[(k * step + item) * 4]);
        best[1] = fmaxf(best[1], stats[(k * step + item) * 4 + 2]);
    }
    constexpr int PER = (E + 31) / 32;
    float o[2][PER], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int i = 0; i < PER; ++i) o[m][i] = 0.f;
    for (int k = warp; k < splits; k += 4) {
        const float* st = stats + (k * step + item) * 4;
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            const float mk = st[2 * m];
            const float f = mk == -INFINITY ? 0.f : expf(mk - best[m]);  // (-inf: the slice held no key of this row)
            sum[m] = fmaf(st[2 * m + 1], f, sum[m]);
            const float* src = part + ((k * step + item) * 2 + m) * E;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int c = lane + 32 * i;
                if (c < E) o[m][i] = fmaf(src[c], f, o[m][i]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        if (lane == 0) sh_sum[warp][m] = sum[m];
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = lane + 32 * i;
            if (c < E) sh_o[warp][m][c] = o[m][i];
        }
    }
    __syncthreads();
    const float s1 = ((sh_sum[0][0] + sh_sum[1][0]) + sh_sum[2][0]) + sh_sum[3][0];
    const float s2 = ((sh_sum[0][1] + sh_sum[1][1]) + sh_sum[2][1]) + sh_sum[3][1];
    const float i1 = s1 > 0.f ? 1.f / s1 : 0.f, i2 = s2 > 0.f ? -lambda / s2 : 0.f;
    constexpr int MINE = (E + 127) / 128;
    float v[MINE];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MINE; ++i) {
        const int c = threadIdx.x + 128 * i;
        v[i] = 0.f;
        if (c < E) {
            const float a1 = ((sh_o[0][0][c] + sh_o[1][0][c]) + sh_o[2][0][c]) + sh_o[3][0][c];
            const float a2 = ((sh_o[0][1][c] + sh_o[1][1][c]) + sh_o[2][1][c]) + sh_o[3][1][c];
            v[i] = a1 * i1 + a2 * i2;
        }
        ss = fmaf(v[i], v[i], ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) sh_ss[warp] = ss;
    __syncthreads();
    ss = ((sh_ss[0] + sh_ss[1]) + sh_ss[2]) + sh_ss[3];
    const float f = out_scale / sqrtf(ss / (float)E + eps);
#pragma unroll
    for (int i = 0; i < MINE; ++i) {
        const int c = threadIdx.x + 128 * i;
        if (c < E) out[(size_t)item * E + c] = __float2bfloat16_rn(v[i] * f);
    }
}
}  // namespace

IB_EXPORT int ib_attention_diff_mma_d() { return D; }
IB_EXPORT int ib_attention_diff_mma_e() { return E; }

// q: contiguous bf16 [n_rows, nh, 2 D]; out: contiguous bf16 [n_rows, nh, E]; pools [pages, nkv, page_size, 2 D | E];
// max_rows_per_entry: an upper bound on the rows of any entry (the grid's width).  splits > 1: the keys in
// slices of `slice_len` (a multiple of 32; splits * slice_len covers every key any row sees) over that many
// CTAs, through `scratch` (ib_attention_diff_mma_scratch_bytes); n_rows: all rows of the step.
IB_EXPORT long long ib_attention_diff_mma_scratch_bytes(int n_rows, int nh, int splits) {
    return (long long)splits * n_rows * nh * (4 + E) * (long long)sizeof(float);
}

IB_EXPORT int ib_attention_diff_mma(const void* q, const void* k_pool, const void* v_pool, void* out, const int* cu_rows,
                                    const int* positions, const int* block_tables, int max_blocks, int n_entries,
                                    int max_rows_per_entry, int nh, int nkv, int page_size, int num_pages, float scale,
                                    float cap, float lambda, float eps, float out_scale, unsigned* err, int n_rows,
                                    int splits, int slice_len, void* scratch, long long scratch_bytes, void* stream) {
    if (n_entries <= 0 || max_rows_per_entry <= 0) return IB_OK;
    if (!q || !k_pool || !v_pool || !out || !cu_rows || !positions || !block_tables || !err) return IB_ERR_BAD_ARG;
    if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || !(eps > 0.f))
        return IB_ERR_BAD_ARG;
    if (n_entries > 65535 || nkv > 65535) return IB_ERR_TOO_LARGE;
    const size_t smem = (size_t)(BM * QS + 2 * BN * KS + 2 * BN * VS) * sizeof(bf16);
    const size_t smem1 = (size_t)(BM * QS + 2 * BN * KS) * sizeof(bf16);  // the first walk alone fetches no values: a CTA more an SM
    static bool configured = false;
    if (!configured) {
        cudaError_t ce = cudaFuncSetAttribute(attention_diff_mma_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ce == cudaSuccess)
            ce = cudaFuncSetAttribute(attention_diff_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
        if (ce == cudaSuccess)
            ce = cudaFuncSetAttribute(attention_diff_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ce != cudaSuccess) return (int)ce;
        configured = true;
    }
    const int R = nh / nkv;
    const long long tiles = ((long long)max_rows_per_entry * R + BM - 1) / BM;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t le;
    if (splits <= 1) {
        le = launch_kernel(attention_diff_mma_kernel<0>, dim3((unsigned)tiles, n_entries, nkv), dim3(THREADS), smem, s,
                           (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, cu_rows, positions,
                           block_tables, max_blocks, nh, nkv, page_size, num_pages, scale, cap, lambda, eps, out_scale, err,
                           1, 0, n_rows, (float*)nullptr, (float*)nullptr);
        if (le != cudaSuccess) return (int)le;
        IB_LAUNCH_CHECK();
        return IB_OK;
    }
    if (!scratch || slice_len <= 0 || slice_len % BN || n_rows <= 0 || (long long)nkv * splits > 65535) return IB_ERR_BAD_ARG;
    if (scratch_bytes < ib_attention_diff_mma_scratch_bytes(n_rows, nh, splits)) return IB_ERR_BAD_ARG;
    float* stats = (float*)scratch;
    float* part = stats + (size_t)splits * n_rows * nh * 4;
    const dim3 grid((unsigned)tiles, n_entries, nkv * splits);
    le = launch_kernel(attention_diff_mma_kernel<1>, grid, dim3(THREADS), smem1, s, (const bf16*)q, (const bf16*)k_pool,
                       (const bf16*)v_pool, (bf16*)out, cu_rows, positions, block_tables, max_blocks, nh, nkv, page_size,
                       num_pages, scale, cap, lambda, eps, out_scale, err, splits, slice_len, n_rows, stats, part);
    if (le != cudaSuccess) return (int)le;
    le = launch_kernel(attention_diff_mma_kernel<2>, grid, dim3(THREADS), smem, s, (const bf16*)q, (const bf16*)k_pool,
                       (const bf16*)v_pool, (bf16*)out, cu_rows, positions, block_tables, max_blocks, nh, nkv, page_size,
                       num_pages, scale, cap, lambda, eps, out_scale, err, splits, slice_len, n_rows, stats, part);
    if (le != cudaSuccess) return (int)le;
    const long long warps = (long long)n_rows * nh;
    le = launch_kernel(attention_diff_merge_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, s, (const float*)part,
                       (bf16*)out, splits, n_rows, nh, eps, out_scale);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// Steps whose entries all have at most 16 packed rows (rows x heads of a group) and values a multiple of 64
// wide: the one-walk kernel over `splits` slices of `slice_len` keys (a multiple of 32) and its merge.
IB_EXPORT long long ib_attention_diff_decode_scratch_bytes(int n_rows, int nh, int splits) {
    return (long long)splits * n_rows * nh * (4 + 2 * E) * (long long)sizeof(float);
}

IB_EXPORT int ib_attention_diff_decode(const void* q, const void* k_pool, const void* v_pool, void* out, const int* cu_rows,
                                       const int* positions, const int* block_tables, int max_blocks, int n_entries,
                                       int nh, int nkv, int page_size, int num_pages, float scale, float cap, float lambda,
                                       float eps, float out_scale, unsigned* err, int n_rows, int splits, int slice_len,
                                       void* scratch, long long scratch_bytes, void* stream) {
    if (n_entries <= 0 || n_rows <= 0) return IB_OK;
    if (E % 64) return IB_ERR_UNSUPPORTED;
    if (!q || !k_pool || !v_pool || !out || !cu_rows || !positions || !block_tables || !err || !scratch)
        return IB_ERR_BAD_ARG;
    if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || !(eps > 0.f) ||
        splits <= 0 || slice_len <= 0 || slice_len % BN)
        return IB_ERR_BAD_ARG;
    if (n_entries > 65535 || (long long)nkv * splits > 65535) return IB_ERR_TOO_LARGE;
    if (scratch_bytes < ib_attention_diff_decode_scratch_bytes(n_rows, nh, splits)) return IB_ERR_BAD_ARG;
    const size_t smem = (size_t)(16 * QS + 2 * BN * KS + 2 * BN * VS) * sizeof(bf16);
    static bool configured = false;
    if (!configured) {
        cudaError_t ce = cudaFuncSetAttribute(attention_diff_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ce != cudaSuccess) return (int)ce;
        configured = true;
    }
    cudaStream_t s = (cudaStream_t)stream;
    float* stats = (float*)scratch;
    float* part = stats + (size_t)splits * n_rows * nh * 4;
    cudaError_t le = launch_kernel(attention_diff_decode_kernel, dim3(1, n_entries, nkv * splits), dim3(THREADS), smem, s,
                                   (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, cu_rows, positions, block_tables,
                                   max_blocks, nh, nkv, page_size, num_pages, scale, cap, err, splits, slice_len, n_rows, stats,
                                   part);
    if (le != cudaSuccess) return (int)le;
    le = launch_kernel(attention_diff_decode_merge_kernel, dim3((unsigned)((long long)n_rows * nh)), dim3(128), 0, s,
                       (const float*)stats, (const float*)part, (bf16*)out, splits, n_rows, nh, lambda, eps, out_scale);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
