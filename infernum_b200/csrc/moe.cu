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

// A third way of scoring (ib_moe_route_softmax_all): s = softmax(z) over all E_all router
// outputs; the choice is made by s_e + correction_e (the lower index among equals), the
// weights are the chosen s_e (without the correction) over their sum + 1e-20.  The last
// E_all - E outputs have no expert behind them: choosing one hands the token's input on
// with that weight.  Written: ids / weights [N, top]; the dense row gate[N, E] for the
// experts that exist; extra[N, 2] = (the sum of the weights that fell on the outputs
// without an expert, sigmoid(z[E_all]) when the logits carry one more column - the gate of
// an expert that every token uses - else 1).  With gate_cols > E the dense row is that wide and its
// columns from E on hold extra[n, 1]: the expert that every token uses, run as further columns of the
// experts' products.
__global__ void moe_route_softmax_all_kernel(const float* __restrict__ logits, int ld,
                                             const float* __restrict__ correction, int E_all, int E, int top,
                                             int with_gate, int* __restrict__ ids, float* __restrict__ weights,
                                             float* __restrict__ gate, float* __restrict__ extra, int gate_cols) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    float* s = sm;          // [E_all] the scores
    float* c = sm + E_all;  // [E_all] the choice values, struck out as they are chosen
    const int row = blockIdx.x, lane = threadIdx.x;
    const float* src = logits + (size_t)row * ld;
    float zmax = -INFINITY;
    for (int e = lane; e < E_all; e += 32) zmax = fmaxf(zmax, src[e]);
    zmax = warp_max(zmax);
    float part = 0.f;
    for (int e = lane; e < E_all; e += 32) {
        const float p = expf(src[e] - zmax);
        s[e] = p;
        part += p;
    }
    const float denom = warp_sum(part);
    __syncwarp();
    for (int e = lane; e < E_all; e += 32) {
        const float v = s[e] / denom;
        s[e] = v;
        c[e] = v + (correction ? correction[e] : 0.f);
        if (gate && e < E) gate[(size_t)row * gate_cols + e] = 0.f;
    }
    __syncwarp();
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = E_all;
        for (int e = lane; e < E_all; e += 32) {
            const float v = c[e];
            if (v > best || (v == best && e < at)) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= E_all) at = k < E_all ? k : 0;  // a row of NaN: any output
        sum += s[at];
        if (lane == 0) {
            ids[(size_t)row * top + k] = at;
            c[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0) {
        const float inv = 1.f / (sum + 1e-20f);
        float passed = 0.f;
        for (int k = 0; k < top; ++k) {
            const int at = ids[(size_t)row * top + k];
            const float w = s[at] * inv;
            weights[(size_t)row * top + k] = w;
            if (at < E) {
                if (gate) gate[(size_t)row * gate_cols + at] = w;
            } else {
                passed += w;
            }
        }
        const float every = with_gate ? 1.f / (1.f + expf(-src[E_all])) : 1.f;
        if (extra) {
            extra[(size_t)row * 2] = passed;
            extra[(size_t)row * 2 + 1] = every;
        }
        if (gate)
            for (int e = E; e < gate_cols; ++e) gate[(size_t)row * gate_cols + e] = every;
    }
}

IB_EXPORT int ib_moe_route_softmax_all(const float* logits, int ld, const float* correction, int E_all, int E, int top,
                                       int with_gate, int* ids, float* weights, float* gate, float* extra,
                                       int gate_cols, int n_rows, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!logits || !ids || !weights || E_all <= 0 || E < 0 || E > E_all || top <= 0 || top > E_all ||
        ld < E_all + (with_gate ? 1 : 0) || (gate && gate_cols < E))
        return IB_ERR_BAD_ARG;
    const size_t smem = (size_t)E_all * 2 * sizeof(float);
    if (smem > 48 * 1024) return IB_ERR_TOO_LARGE;
    cudaError_t le = launch_kernel(moe_route_softmax_all_kernel, dim3(n_rows), dim3(32), smem, (cudaStream_t)stream,
                                   logits, ld, correction, E_all, E, top, with_gate, ids, weights, gate, extra, gate_cols);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// out[n, :] = routed[n, :] + extra[n, 0] * h[n, :] + extra[n, 1] * shared[n, :]: the experts' weighted
// sum, the input handed on by the outputs without an expert, and the expert that every token uses behind
// its gate; `routed` and `shared` may be absent.  32-bit arithmetic, one rounding at the store.
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ routed, const T* __restrict__ h, int h_stride,
                                   const T* __restrict__ shared, const float* __restrict__ extra,
                                   T* __restrict__ out, int n_rows, int W) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const float passed = extra[(size_t)row * 2], g = extra[(size_t)row * 2 + 1];
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < W; i += gridDim.y * blockDim.x) {
        float v = routed ? to_f32(routed[(size_t)row * W + i]) : 0.f;
        v = fmaf(passed, to_f32(h[(size_t)row * h_stride + i]), v);
        if (shared) v = fmaf(g, to_f32(shared[(size_t)row * W + i]), v);
        out[(size_t)row * W + i] = from_f32<T>(v);
    }
}

IB_EXPORT int ib_moe_combine(const void* routed, const void* h, int h_stride, const void* shared, const float* extra,
                             void* out, int dtype, int n_rows, int W, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!h || !extra || !out || W <= 0 || h_stride < W) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_rows, (W + 1023) / 1024), block(W >= 1024 ? 256 : 128);
    cudaError_t le;
    if (dtype == 0)
        le = launch_kernel(moe_combine_kernel<float>, grid, block, 0, s, (const float*)routed, (const float*)h, h_stride,
                           (const float*)shared, extra, (float*)out, n_rows, W);
    else if (dtype == 1)
        le = launch_kernel(moe_combine_kernel<bf16>, grid, block, 0, s, (const bf16*)routed, (const bf16*)h, h_stride,
                           (const bf16*)shared, extra, (bf16*)out, n_rows, W);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
