// Routing of a mixture of experts.
//   z = router logits [N, E] (32-bit) + bias;  the `top` largest are chosen (the
//   lower index among equals), and their weights are the softmax over the chosen
//   logits only.  Written two ways: the lists ids[N, top] / weights[N, top] in
//   order of falling logit, and the dense row gate[N, E] that holds a chosen
//   expert's weight and 0 elsewhere.
// One warp per row; the row is kept in shared memory and a chosen logit is
// struck out there.
//
// A second way of scoring (ib_moe_route_scored): s_e = sigmoid(z_e); expert e belongs to
// group floor(e / (E / n_groups)); G_g = the sum of the `group_top` largest s_e of group g;
// the `keep` groups with the largest G_g stay open and the others' experts are struck out
// (n_groups <= 1: nothing is struck out); the `top` largest scores among those are
// chosen, the lower index among equals, and are the weights as they are - or,
// with `renorm`, divided by their sum.
#include "common.cuh"

using namespace ib;

// Router logits z[n, e] = sum_k x[n, k] w[e, k] in 32-bit: one warp per (row,
// expert), lanes stride over k, then a fixed tree over the lanes; a row's logits do
// not depend on the batch.  The product is skinny (a handful of experts, K in the
// thousands): a tiled product would leave one CTA walking all of K.
template <typename TX, typename TW>
__global__ void router_logits_kernel(const TX* __restrict__ x, int ldx, const TW* __restrict__ w, int ldw,
                                     float* __restrict__ z, int n_rows, int E, int K) {
    pdl_trigger();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_rows * E) return;
    const int n = warp / E, e = warp % E;
    const TX* xr = x + (size_t)n * ldx;
    const TW* wr = w + (size_t)e * ldw;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(to_f32(xr[k]), to_f32(wr[k]), acc);
    acc = warp_sum(acc);
    if (lane == 0) z[(size_t)n * E + e] = acc;
}

IB_EXPORT int ib_router_logits(const void* x, int x_dtype, int ldx, const void* w, int w_dtype, int ldw, float* z,
                               int n_rows, int E, int K, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x || !w || !z || E <= 0 || K <= 0 || ldx < K || ldw < K) return IB_ERR_BAD_ARG;
    const long long warps = (long long)n_rows * E;
    const unsigned blocks = (unsigned)((warps + 7) / 8);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t le;
    if (x_dtype == 0 && w_dtype == 0)
        le = launch_kernel(router_logits_kernel<float, float>, dim3(blocks), dim3(256), 0, s, (const float*)x, ldx,
                           (const float*)w, ldw, z, n_rows, E, K);
    else if (x_dtype == 1 && w_dtype == 1)
        le = launch_kernel(router_logits_kernel<bf16, bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)x, ldx,
                           (const bf16*)w, ldw, z, n_rows, E, K);
    else if (x_dtype == 1 && w_dtype == 0)
        le = launch_kernel(router_logits_kernel<bf16, float>, dim3(blocks), dim3(256), 0, s, (const bf16*)x, ldx,
                           (const float*)w, ldw, z, n_rows, E, K);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

__global__ void moe_route_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias, int E,
                                 int top, int* __restrict__ ids, float* __restrict__ weights,
                                 float* __restrict__ gate) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float z[];
    const int row = blockIdx.x, lane = threadIdx.x;
    const float* src = logits + (size_t)row * ld;
    for (int e = lane; e < E; e += 32) {
        z[e] = src[e] + (bias ? bias[e] : 0.f);
        if (gate) gate[(size_t)row * E + e] = 0.f;
    }
    __syncwarp();
    float zmax = 0.f, denom = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = E;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < at)) { best = v; at = e; }   // (NaN never wins)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= E) at = k < E ? k : 0;  // a row of NaN: any expert, weight NaN
        if (k == 0) zmax = best;
        const float p = expf(best - zmax);
        denom += p;
        if (lane == 0) {
            ids[(size_t)row * top + k] = at;
            weights[(size_t)row * top + k] = p;
            z[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0) {
        for (int k = 0; k < top; ++k) {
            const float w = weights[(size_t)row * top + k] / denom;
            weights[(size_t)row * top + k] = w;
            if (gate) gate[(size_t)row * E + ids[(size_t)row * top + k]] = w;
        }
    }
}

IB_EXPORT int ib_moe_route(const float* logits, int ld, const float* bias, int E, int top, int* ids,
                           float* weights, float* gate, int n_rows, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!logits || !ids || !weights || E <= 0 || top <= 0 || top > E || ld < E) return IB_ERR_BAD_ARG;
    if ((size_t)E * sizeof(float) > 48 * 1024) return IB_ERR_TOO_LARGE;
    cudaError_t le = launch_kernel(moe_route_kernel, dim3(n_rows), dim3(32), (size_t)E * sizeof(float),
                                   (cudaStream_t)stream, logits, ld, bias, E, top, ids, weights, gate);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

__global__ void moe_route_scored_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias,
                                        int E, int top, int n_groups, int keep, int group_top, int renorm,
                                        int* __restrict__ ids, float* __restrict__ weights,
                                        float* __restrict__ gate) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float z[];  // [E] scores, struck out as they are chosen; then [n_groups] group scores
    float* gs = z + E;
    const int row = blockIdx.x, lane = threadIdx.x;
    const float* src = logits + (size_t)row * ld;
    for (int e = lane; e < E; e += 32) {
        z[e] = 1.f / (1.f + expf(-(src[e] + (bias ? bias[e] : 0.f))));
        if (gate) gate[(size_t)row * E + e] = 0.f;
    }
    __syncwarp();
    if (n_groups > 1) {
        const int per = E / n_groups;
        // a lane a group: the sum of its group_top largest scores (lowest index among equals)
        for (int g = lane; g < n_groups; g += 32) {
            float sum = 0.f;
            unsigned long long taken = 0ull;  // (groups of more than 64 experts: see the host check)
            for (int k = 0; k < group_top && k < per; ++k) {
                float best = -INFINITY;
                int at = -1;
                for (int i = 0; i < per; ++i) {
                    if ((taken >> i) & 1ull) continue;
                    const float v = z[g * per + i];
                    if (v > best) { best = v; at = i; }
                }
                if (at < 0) break;
                taken |= 1ull << at;
                sum += best;
            }
            gs[g] = sum;
        }
        __syncwarp();
        // lane 0 picks the best groups and strikes out the experts of the others
        if (lane == 0) {
            for (int k = 0; k < keep; ++k) {
                float best = -INFINITY;
                int at = -1;
                for (int g = 0; g < n_groups; ++g)
                    if (gs[g] > best) { best = gs[g]; at = g; }
                if (at < 0) break;
                gs[at] = -INFINITY;  // chosen: marked by -inf, told apart from the rest below
            }
        }
        __syncwarp();
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != -INFINITY) z[e] = -INFINITY;
        __syncwarp();
    }
    float denom = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = E;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < at)) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= E) { at = k < E ? k : 0; best = 0.f; }  // nothing left to choose (a row of NaN): weight 0
        denom += best;
        if (lane == 0) {
            ids[(size_t)row * top + k] = at;
            weights[(size_t)row * top + k] = best;
            z[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0) {
        for (int k = 0; k < top; ++k) {
            float w = weights[(size_t)row * top + k];
            if (renorm) {
                w = w / denom;
                weights[(size_t)row * top + k] = w;
            }
            if (gate) gate[(size_t)row * E + ids[(size_t)row * top + k]] = w;
        }
    }
}

IB_EXPORT int ib_moe_route_scored(const float* logits, int ld, const float* bias, int E, int top, int n_groups,
                                  int keep, int group_top, int renorm, int* ids, float* weights, float* gate,
                                  int n_rows, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!logits || !ids || !weights || E <= 0 || top <= 0 || top > E || ld < E) return IB_ERR_BAD_ARG;
    if (n_groups > 1 && (E % n_groups || keep <= 0 || keep > n_groups || group_top <= 0 ||
                         (long long)keep * (E / n_groups) < top))
        return IB_ERR_BAD_ARG;
    if (n_groups > 1 && E / n_groups > 64) return IB_ERR_TOO_LARGE;
    const size_t smem = (size_t)(E + (n_groups > 1 ? n_groups : 0)) * sizeof(float);
    if (smem > 48 * 1024) return IB_ERR_TOO_LARGE;
    cudaError_t le = launch_kernel(moe_route_scored_kernel, dim3(n_rows), dim3(32), smem, (cudaStream_t)stream, logits,
                                   ld, bias, E, top, n_groups, keep, group_top, renorm, ids, weights, gate);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
