// A feed-forward of routed experts.
//
//   z = W_r h                                  router logits, 32-bit sums
//   s = sigmoid(z) (or softmax(z))             scores; the `top` largest choose the token's experts
//   w_j = s[e_j] (optionally divided by their sum)
//   expert e on input x:  g = W_gate x, u = W_up x (both clamped where the part gives limits),
//                         y = g * sigmoid(alpha g) * (u + up_shift),  result W_down y
//   out = sum_j expert_{e_j}(w_j h)   (weight on the input)    or    sum_j w_j expert_{e_j}(h)   (on the output)
//
// Kernels of this file (T: the activations' type, TW: the stored type of the experts' matrices):
//   moe_router_kernel      a block a token: logits, scores, the top experts and their weights
//   moe_gate_up_kernel     a block per (token, chosen expert, slice of the inner width): the token's row in shared
//                          memory, a warp per inner feature, 16-byte loads along the matrices' rows
//   moe_down_kernel        a block per (token, slice of the width): sums the chosen experts' down products in the order of
//                          the choice and writes or adds the 32-bit result
// They stream each chosen expert's matrices once per token: the form for steps of few tokens.  Steps of many tokens
// take the grouped tensor-core products of moe_grouped.cu.
#include "common.cuh"

namespace {
constexpr int MAX_TOP = 8;
constexpr int MAX_EXPERTS = 1024;

template <typename TW> __device__ __forceinline__ float dot8(const TW* w, const float* x);
template <> __device__ __forceinline__ float dot8<h16>(const h16* w, const float* x) {
    const uint4 raw = *(const uint4*)w;
    const h16x2* h = (const h16x2*)&raw;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = h16x2_to_float2(h[i]);
        s = fmaf(f.x, x[2 * i], s);
        s = fmaf(f.y, x[2 * i + 1], s);
    }
    return s;
}
template <> __device__ __forceinline__ float dot8<float>(const float* w, const float* x) {
    const float4 a = *(const float4*)w, b = *(const float4*)(w + 4);
    float s = 0.f;
    s = fmaf(a.x, x[0], s); s = fmaf(a.y, x[1], s); s = fmaf(a.z, x[2], s); s = fmaf(a.w, x[3], s);
    s = fmaf(b.x, x[4], s); s = fmaf(b.y, x[5], s); s = fmaf(b.z, x[6], s); s = fmaf(b.w, x[7], s);
    return s;
}
// <w, x> over K elements by one warp; every lane gets the sum.  The order of the additions depends on K alone.
template <typename TW>
__device__ __forceinline__ float warp_dot(const TW* __restrict__ w, const float* x, int K, int lane, bool vec) {
    float s = 0.f;
    if (vec) {
        for (int c = lane * 8; c < K; c += 256) s += dot8<TW>(w + c, x + c);
    } else {
        for (int c = lane; c < K; c += 32) s = fmaf(to_float(w[c]), x[c], s);
    }
    return warp_sum(s);
}

template <typename T, typename TW>
__global__ void __launch_bounds__(128)
moe_router_kernel(const T* __restrict__ h, int ld, const TW* __restrict__ wr, const int* __restrict__ token_request,
                  int* __restrict__ ids, float* __restrict__ weights, int W, int E, int top, int softmax_scores,
                  int renormalize) {
    extern __shared__ __align__(16) float sm[];            // [W] the row, [E] the scores
    float* x = sm;
    float* z = sm + ((W + 3) & ~3);
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (token_request[n] < 0) {                              // a padded row of a captured step: no expert
        if (threadIdx.x < top) { ids[(size_t)n * top + threadIdx.x] = -1; weights[(size_t)n * top + threadIdx.x] = 0.f; }
        return;
    }
    for (int c = threadIdx.x; c < W; c += blockDim.x) x[c] = to_float(h[(size_t)n * ld + c]);
    __syncthreads();
    const bool vec = W % 8 == 0 && ((uintptr_t)wr % 16) == 0;
    for (int e = warp; e < E; e += 4) {
        const float s = warp_dot<TW>(wr + (size_t)e * W, x, W, lane, vec);
        if (lane == 0) z[e] = s;
    }
    __syncthreads();
    if (warp != 0) return;
    // The choice is made on the logits: both scores grow with them, and a sigmoid that has run out of bits near 1
    // would tie experts that their logits still tell apart.
    float mx = -INFINITY, sum = 0.f;
    if (softmax_scores) {
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        for (int e = lane; e < E; e += 32) sum += expf(z[e] - mx);
        sum = warp_sum(sum);
    }
    float chosen_w[MAX_TOP];
    int chosen[MAX_TOP];
    float total = 0.f;
    for (int j = 0; j < top; ++j) {                         // the largest logit left; of equal ones the lowest index
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best) { best = v; arg = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        chosen[j] = arg;
        chosen_w[j] = softmax_scores ? expf(best - mx) / sum : 1.f / (1.f + expf(-best));
        total += chosen_w[j];
        if (lane == 0) z[arg] = -INFINITY;
        __syncwarp();
    }
    if (lane == 0)
        for (int j = 0; j < top; ++j) {
            ids[(size_t)n * top + j] = chosen[j];
            weights[(size_t)n * top + j] = renormalize ? chosen_w[j] / total : chosen_w[j];
        }
}

struct ExpertMath {
    float gate_max, up_min, up_max;     // clamps (infinite: none)
    float alpha, up_shift;              // y = g * sigmoid(alpha g) * (u + up_shift)
    int weight_on_input;
};

__device__ __forceinline__ float expert_act(float g, float u, const ExpertMath& m) {
    g = fminf(g, m.gate_max);
    u = fminf(fmaxf(u, m.up_min), m.up_max);
    return g / (1.f + expf(-m.alpha * g)) * (u + m.up_shift);
}

// gate_up: [E, 2F, W] (an expert's gate rows, then its up rows); y: [N * top, F] in the activations' type.
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
moe_gate_up_kernel(const T* __restrict__ h, int ld, const TW* __restrict__ gate_up, const int* __restrict__ ids,
                   const float* __restrict__ weights, T* __restrict__ y, int W, int F, int top, int per_block, ExpertMath m) {
    extern __shared__ __align__(16) float x[];             // [W]
    pdl_launch_dependents();
    pdl_wait();
    const int pair = blockIdx.x, n = pair / top, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = ids[pair];
    if (e < 0) return;
    const float wt = m.weight_on_input ? weights[pair] : 1.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) x[c] = wt * to_float(h[(size_t)n * ld + c]);
    __syncthreads();
    const TW* wg = gate_up + (size_t)e * 2 * F * W;
    const TW* wu = wg + (size_t)F * W;
    const bool vec = W % 8 == 0 && ((uintptr_t)gate_up % 16) == 0;
    const int f_end = min(F, (blockIdx.y + 1) * per_block);
    for (int f = blockIdx.y * per_block + warp; f < f_end; f += 4) {
        const float g = warp_dot<TW>(wg + (size_t)f * W, x, W, lane, vec);
        const float u = warp_dot<TW>(wu + (size_t)f * W, x, W, lane, vec);
        if (lane == 0) y[(size_t)pair * F + f] = from_float<T>(expert_act(g, u, m));
    }
}

// down: [E, W, F]; out: 32-bit [N, W], written (accumulate 0) or added to.
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
moe_down_kernel(const T* __restrict__ y, const TW* __restrict__ down, const int* __restrict__ ids,
                const float* __restrict__ weights, float* out, int W, int F, int top, int per_block, int accumulate,
                int weight_on_input) {
    extern __shared__ __align__(16) float ys[];            // [top][F]
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (ids[(size_t)n * top] < 0) return;
    const int Fp = (F + 3) & ~3;
    for (int i = threadIdx.x; i < top * F; i += blockDim.x) {
        const int j = i / F, f = i % F;
        const float wt = weight_on_input ? 1.f : weights[(size_t)n * top + j];
        ys[j * Fp + f] = wt * to_float(y[((size_t)n * top + j) * F + f]);
    }
    __syncthreads();
    const bool vec = F % 8 == 0 && ((uintptr_t)down % 16) == 0;
    const int o_end = min(W, (blockIdx.y + 1) * per_block);
    for (int o = blockIdx.y * per_block + warp; o < o_end; o += 4) {
        float s = 0.f;
        for (int j = 0; j < top; ++j) {
            const int e = ids[(size_t)n * top + j];
            s += warp_dot<TW>(down + ((size_t)e * W + o) * F, ys + j * Fp, F, lane, vec);
        }
        if (lane == 0) {
            float* dst = out + (size_t)n * W + o;
            *dst = accumulate ? *dst + s : s;
        }
    }
}
}  // namespace

TNX_EXPORT int tnx_moe_route(const void* h, int ld, const void* router, const int* token_request, int* ids, float* weights,
                             int N, int W, int E, int top, int softmax_scores, int renormalize, int h_h16, int w_h16,
                             cudaStream_t stream) {
    if (N <= 0) return 0;
    if (W <= 0 || E <= 0 || E > MAX_EXPERTS || top <= 0 || top > MAX_TOP || top > E) return TNX_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(((W + 3) & ~3) + E) * sizeof(float);
    if (smem > 160 * 1024) return TNX_ERR_UNSUPPORTED;
#define GO(T, TW)                                                                                                       \
    do {                                                                                                                \
        if (smem > 48 * 1024) cudaFuncSetAttribute(moe_router_kernel<T, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return tnx_launch_in_order(moe_router_kernel<T, TW>, dim3(N), dim3(128), smem, stream, (const T*)h, ld,         \
                                   (const TW*)router, token_request, ids, weights, W, E, top, softmax_scores, renormalize); \
    } while (0)
    if (h_h16 && w_h16) GO(h16, h16);
    if (h_h16) GO(h16, float);
    if (w_h16) GO(float, h16);
    GO(float, float);
#undef GO
}

TNX_EXPORT int tnx_moe_experts(const void* h, int ld, const void* gate_up, const void* down, const int* ids,
                               const float* weights, void* y, float* out, int N, int W, int F, int top, float gate_max,
                               float up_min, float up_max, float alpha, float up_shift, int weight_on_input, int accumulate,
                               int h_h16, int w_h16, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (W <= 0 || F <= 0 || top <= 0 || top > MAX_TOP) return TNX_ERR_UNSUPPORTED;
    const size_t smem1 = (size_t)W * sizeof(float), smem2 = (size_t)top * ((F + 3) & ~3) * sizeof(float);
    if (smem1 > 160 * 1024 || smem2 > 160 * 1024) return TNX_ERR_UNSUPPORTED;
    ExpertMath m{gate_max, up_min, up_max, alpha, up_shift, weight_on_input};
    // enough blocks to fill the GPU when the tokens are few, whole rows of work per warp when they are many
    const int pairs = N * top;
    int per1 = 4; while (per1 < F && (long long)pairs * ((F + per1 - 1) / per1) > 2048) per1 *= 2;
    int per2 = 4; while (per2 < W && (long long)N * ((W + per2 - 1) / per2) > 2048) per2 *= 2;
    const dim3 g1(pairs, (F + per1 - 1) / per1), g2(N, (W + per2 - 1) / per2);
#define GO(T, TW)                                                                                                       \
    do {                                                                                                                \
        if (smem1 > 48 * 1024) cudaFuncSetAttribute(moe_gate_up_kernel<T, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1); \
        if (smem2 > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel<T, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);    \
        int rc = tnx_launch_in_order(moe_gate_up_kernel<T, TW>, g1, dim3(128), smem1, stream, (const T*)h, ld,          \
                                     (const TW*)gate_up, ids, weights, (T*)y, W, F, top, per1, m);                      \
        if (rc != 0) return rc;                                                                                         \
        return tnx_launch_in_order(moe_down_kernel<T, TW>, g2, dim3(128), smem2, stream, (const T*)y, (const TW*)down,  \
                                   ids, weights, out, W, F, top, per2, accumulate, weight_on_input);                    \
    } while (0)
    if (h_h16 && w_h16) GO(h16, h16);
    if (h_h16) GO(h16, float);
    if (w_h16) GO(float, h16);
    GO(float, float);
#undef GO
}
