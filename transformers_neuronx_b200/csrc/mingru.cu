// minGRU: a gated recurrence whose gates read only the current token.  Per channel c, from the projection's
// raw outputs a (update gate), u (candidate) and, when given, g (output gate):
//     z = sigmoid(a);   cand = u + 1/2 where u >= 0, sigmoid(u) where u < 0
//     S_t = (1 - z) S_(t-1) + z cand                       (S: 32-bit, kept per request between steps)
//     out_t = S_t * silu(g) * out_scale                      (out_t = S_t * out_scale without g), in the activation type
// Gates, candidate and state are computed in 32-bit from the projection's output.
// The loads of the next tokens do not depend on the state and are issued ahead (the loops are unrolled by eight).
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }

// One token of the recurrence: the new state from the raw gate value a and the raw candidate value u.
__device__ __forceinline__ float mingru_step(float S, float a, float u) {
    const float z = sigmoidf_(a);
    const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
    return (1.f - z) * S + z * cand;
}

// A thread block owns 32 channels (the lanes) of one request; its warps own consecutive segments of the request's
// tokens of this step.  The recurrence is linear in the state, S_t = (1 - z_t) S_(t-1) + z_t cand_t, so a segment
// is first run from a zero state, which gives its own contribution B and the product A of its (1 - z_t); the state
// a segment starts from is then folded from the segments before it (S <- A S + B), and the segment is run again
// from that state, now writing its outputs.  With one segment (a step of single tokens) the first run is skipped.
template <typename T>
__global__ void mingru_scan_kernel(const T* __restrict__ proj, int ld, int z_off, int x_off, int g_off,
                                   float* __restrict__ state, const int* __restrict__ q_start,
                                   const int* __restrict__ q_len, const int* __restrict__ state_slots,
                                   T* __restrict__ out, int out_ld, float out_scale, int width) {
    __shared__ float As[32][33], Bs[32][33];          // [segment][channel]
    pdl_launch_dependents();
    pdl_wait();
    const int req = blockIdx.y;
    const int lane = threadIdx.x & 31, seg = threadIdx.x >> 5, n_seg = blockDim.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    const int len = q_len[req];
    if (len <= 0) return;                             // a padded request of a captured batch
    const int slot = state_slots[req];
    if (slot < 0) return;
    const bool live = c < width;
    const int per = (len + n_seg - 1) / n_seg;
    const int lo = min(len, seg * per), hi = min(len, lo + per);
    const T* p = proj + (size_t)q_start[req] * ld + (live ? c : 0);
    if (n_seg > 1) {
        float A = 1.f, B = 0.f;
        int t = lo;
        for (; t + 8 <= hi; t += 8) {
            float a[8], u[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { const T* row = p + (size_t)(t + i) * ld; a[i] = to_float(row[z_off]); u[i] = to_float(row[x_off]); }
#pragma unroll
            for (int i = 0; i < 8; ++i) { B = mingru_step(B, a[i], u[i]); A *= 1.f - sigmoidf_(a[i]); }
        }
        for (; t < hi; ++t) {
            const T* row = p + (size_t)t * ld;
            const float a = to_float(row[z_off]), u = to_float(row[x_off]);
            B = mingru_step(B, a, u);
            A *= 1.f - sigmoidf_(a);
        }
        As[seg][lane] = A;
        Bs[seg][lane] = B;
        __syncthreads();
    }
    float S = live ? state[(size_t)slot * width + c] : 0.f;
    for (int s = 0; s < seg; ++s) S = As[s][lane] * S + Bs[s][lane];
    T* o = out + (size_t)q_start[req] * out_ld + (live ? c : 0);
    int t = lo;
    for (; t + 8 <= hi; t += 8) {
        float a[8], u[8], g[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const T* row = p + (size_t)(t + i) * ld;
            a[i] = to_float(row[z_off]);
            u[i] = to_float(row[x_off]);
            g[i] = g_off >= 0 ? to_float(row[g_off]) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            S = mingru_step(S, a[i], u[i]);
            const float y = g_off >= 0 ? S * (g[i] * sigmoidf_(g[i])) : S;
            if (live) o[(size_t)(t + i) * out_ld] = from_float<T>(y * out_scale);
        }
    }
    for (; t < hi; ++t) {
        const T* row = p + (size_t)t * ld;
        S = mingru_step(S, to_float(row[z_off]), to_float(row[x_off]));
        float y = S;
        if (g_off >= 0) { const float g = to_float(row[g_off]); y = S * (g * sigmoidf_(g)); }
        if (live) o[(size_t)t * out_ld] = from_float<T>(y * out_scale);
    }
    if (live && hi == len && lo < len) state[(size_t)slot * width + c] = S;      // the segment that holds the last token
}

}  // namespace

// proj: [tokens, ld] with the update gate's raw values at column z_off, the candidate's at x_off and the output
// gate's at g_off (g_off < 0: no output gate), `width` columns each; state: [slots, width] 32-bit.
TNX_EXPORT int tnx_mingru_scan(const void* proj, int ld, int z_off, int x_off, int g_off, float* state,
                               const int* q_start, const int* q_len, const int* state_slots, void* out, int out_ld,
                               float out_scale, int n_requests, int width, int most_tokens, int is_h16,
                               cudaStream_t stream) {
    // most_tokens: an upper bound of any request's rows (1 for a step of single tokens): a segment gets 32 tokens or more
    if (n_requests <= 0) return 0;
    if (width <= 0 || n_requests > 65535 || out_ld < width || most_tokens <= 0) return TNX_ERR_BAD_ARG;
    int segments = 1;
    while (segments < 16 && segments * 32 < most_tokens) segments *= 2;
    const int threads = 32 * segments;
    const dim3 grid((width + 31) / 32, n_requests);
    if (is_h16)
        return tnx_launch_in_order(mingru_scan_kernel<h16>, grid, dim3(threads), 0, stream, (const h16*)proj, ld, z_off, x_off,
                                   g_off, state, q_start, q_len, state_slots, (h16*)out, out_ld, out_scale, width);
    return tnx_launch_in_order(mingru_scan_kernel<float>, grid, dim3(threads), 0, stream, (const float*)proj, ld, z_off,
                               x_off, g_off, state, q_start, q_len, state_slots, (float*)out, out_ld, out_scale, width);
}
