// minGRU: a gated recurrence whose gates read only the current token.  Per channel c, from the projection's
// raw outputs a (update gate), u (candidate) and, when given, g (output gate):
//     z = sigmoid(a);   cand = u + 1/2 where u >= 0, sigmoid(u) where u < 0
//     S_t = (1 - z) S_(t-1) + z cand                       (S: 32-bit, kept per request between steps)
//     out_t = S_t * silu(g) * out_scale                      (out_t = S_t * out_scale without g), in the activation type
// Gates, candidate and state are computed in 32-bit from the projection's output.
// One thread per (request, channel) walks the request's tokens of this step in order; the loads of the next
// tokens do not depend on the state and are issued ahead (the loop is unrolled by four).
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }

template <typename T>
__global__ void mingru_scan_kernel(const T* __restrict__ proj, int ld, int z_off, int x_off, int g_off,
                                   float* __restrict__ state, const int* __restrict__ q_start,
                                   const int* __restrict__ q_len, const int* __restrict__ state_slots,
                                   T* __restrict__ out, int out_ld, float out_scale, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int req = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int len = q_len[req];
    if (c >= width || len <= 0) return;              // len 0: a padded request of a captured batch
    const int slot = state_slots[req];
    if (slot < 0) return;
    const int t0 = q_start[req];
    float S = state[(size_t)slot * width + c];
    const T* p = proj + (size_t)t0 * ld + c;
    T* o = out + (size_t)t0 * out_ld + c;
    int t = 0;
    for (; t + 4 <= len; t += 4) {
        float a[4], u[4], g[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const T* row = p + (size_t)(t + i) * ld;
            a[i] = to_float(row[z_off]);
            u[i] = to_float(row[x_off]);
            g[i] = g_off >= 0 ? to_float(row[g_off]) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float z = sigmoidf_(a[i]);
            const float cand = u[i] >= 0.f ? u[i] + 0.5f : sigmoidf_(u[i]);
            S = (1.f - z) * S + z * cand;
            const float y = g_off >= 0 ? S * (g[i] * sigmoidf_(g[i])) : S;
            o[(size_t)(t + i) * out_ld] = from_float<T>(y * out_scale);
        }
    }
    for (; t < len; ++t) {
        const T* row = p + (size_t)t * ld;
        const float a = to_float(row[z_off]), u = to_float(row[x_off]);
        const float z = sigmoidf_(a);
        const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
        S = (1.f - z) * S + z * cand;
        float y = S;
        if (g_off >= 0) { const float g = to_float(row[g_off]); y = S * (g * sigmoidf_(g)); }
        o[(size_t)t * out_ld] = from_float<T>(y * out_scale);
    }
    state[(size_t)slot * width + c] = S;
}

}  // namespace

// proj: [tokens, ld] with the update gate's raw values at column z_off, the candidate's at x_off and the output
// gate's at g_off (g_off < 0: no output gate), `width` columns each; state: [slots, width] 32-bit.
TNX_EXPORT int tnx_mingru_scan(const void* proj, int ld, int z_off, int x_off, int g_off, float* state,
                               const int* q_start, const int* q_len, const int* state_slots, void* out, int out_ld,
                               float out_scale, int n_requests, int width, int is_h16, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (width <= 0 || n_requests > 65535 || out_ld < width) return TNX_ERR_BAD_ARG;
    const int threads = 128;
    const dim3 grid((width + threads - 1) / threads, n_requests);
    if (is_h16)
        return tnx_launch_in_order(mingru_scan_kernel<h16>, grid, dim3(threads), 0, stream, (const h16*)proj, ld, z_off, x_off,
                                   g_off, state, q_start, q_len, state_slots, (h16*)out, out_ld, out_scale, width);
    return tnx_launch_in_order(mingru_scan_kernel<float>, grid, dim3(threads), 0, stream, (const float*)proj, ld, z_off,
                               x_off, g_off, state, q_start, q_len, state_slots, (float*)out, out_ld, out_scale, width);
}
