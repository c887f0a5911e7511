// The elementwise step of a gated feed-forward: out = act(gate) * up, where gate and up are the two halves
// (columns [0, F) and [F, 2F)) of one product's output; the activation is named by its code (common.cuh).
// Computed in 32-bit from the stored values, rounded once.
#include "common.cuh"

namespace {
template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ gu, int ld, T* __restrict__ out, int out_ld,
                                        long long total, int F, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const long long n = e / F;
        const int c = (int)(e % F);
        const T* row = gu + n * ld;
        const float g = to_float(row[c]), u = to_float(row[F + c]);
        out[n * out_ld + c] = from_float<T>(apply_activation(g, act) * u);
    }
}

// The same, eight 16-bit values a thread (one 16-byte piece of the gate, one of the up half, one stored).
__global__ void gated_activation_h16x8_kernel(const h16* __restrict__ gu, int ld, h16* __restrict__ out, int out_ld,
                                              long long total8, int F8, int F, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total8; e += stride) {
        const long long n = e / F8;
        const int c = (int)(e % F8) * 8;
        const h16* row = gu + n * ld;
        const uint4 g4 = *(const uint4*)(row + c), u4 = *(const uint4*)(row + F + c);
        const h16x2* gp = (const h16x2*)&g4;
        const h16x2* up = (const h16x2*)&u4;
        uint4 o4;
        h16x2* op = (h16x2*)&o4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 g = h16x2_to_float2(gp[i]), u = h16x2_to_float2(up[i]);
            op[i] = floats_to_h16x2(apply_activation(g.x, act) * u.x, apply_activation(g.y, act) * u.y);
        }
        *(uint4*)(out + n * out_ld + c) = o4;
    }
}
}  // namespace

TNX_EXPORT int tnx_gated_activation(const void* gu, int ld, void* out, int out_ld, int n_rows, int F, int act,
                                    int is_h16, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (F <= 0 || ld < 2 * F || out_ld < F || act < 0 || act >= TNX_ACT_COUNT) return TNX_ERR_BAD_ARG;
    const long long total = (long long)n_rows * F;
    const int threads = 256;
    if (is_h16 && F % 8 == 0 && ld % 8 == 0 && out_ld % 8 == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        const long long total8 = total / 8;
        const int blocks8 = (int)((total8 + threads - 1) / threads < 148 * 16 ? (total8 + threads - 1) / threads : 148 * 16);
        return tnx_launch_in_order(gated_activation_h16x8_kernel, dim3(blocks8), dim3(threads), 0, stream, (const h16*)gu, ld,
                                   (h16*)out, out_ld, total8, F / 8, F, act);
    }
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (is_h16)
        return tnx_launch_in_order(gated_activation_kernel<h16>, dim3(blocks), dim3(threads), 0, stream, (const h16*)gu, ld,
                                   (h16*)out, out_ld, total, F, act);
    return tnx_launch_in_order(gated_activation_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)gu, ld,
                               (float*)out, out_ld, total, F, act);
}
