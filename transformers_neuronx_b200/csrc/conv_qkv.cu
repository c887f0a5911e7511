// What lies between an attention mixer's projections and its attention kernel when the projections pass through
// a short causal convolution over time:
//
//   u_t[c]   the projection's output (bias included) of channel c at position t of the request; zero before position 0
//   y_t[c] = sum_j w[c, j] * u_(t - taps + 1 + j)[c]                     j = 0 .. taps - 1   (no convolution: y = u)
//   queries and keys, per head of `dk` channels:  y / sqrt(mean(y^2) + eps) * g[c]   (g: one weight vector for all heads)
//   then the first rot_dims channels of each head turned by the position: pairs (2i, 2i + 1) (interleaved) or
//   (i, i + rot_dims / 2) (halves), (a, b) -> (a cos - b sin, b cos + a sin) * magnitude, angle = t * inv_freq[i]
//   values: y only.
//
// Everything after the loads is 32-bit (the angle is position x frequency in 32-bit, sincosf); the results are
// written in the activation type with `D` channels a head, the rest zero, as the attention kernels and the pages want
// them.  The last taps - 1 projected values of every channel are the request's state ([slots, taps - 1, channels], in
// the projection's type, oldest first): a token whose predecessors are not among this step's rows reads them from
// there, so the result does not depend on how the request was cut into steps.  A request with one row updates its
// state in the same kernel (no other row reads it); requests with several rows are brought up to date by
// conv_state_update_kernel, launched after every row has read the old state.
//
// One thread block per token, one warp per head (of queries, keys or values) at a time; a lane owns the pairs
// (2 lane, 2 lane + 1) + 64 r of the head, so that an interleaved rotation stays inside the lane.
#include "common.cuh"

namespace {
constexpr int MAX_R = 4;            // a head has at most 64 * MAX_R channels
constexpr int MAX_TAPS = 8;

template <typename T>
struct ConvPrep {
    const T* proj; int ld; int col0;             // the mixer's projections begin at column col0: queries, keys, values
    const float* conv_w; int taps;              // [channels, taps] or null (no convolution; taps is 1 then)
    T* state;                                   // [slots, taps - 1, channels]
    const int* token_request; const int* positions; const int* q_start; const int* q_len; const int* state_slots;
    const float* q_norm; const float* k_norm; float eps;      // [dk] each, or null
    const float* inv_freq; int rot_dims; int interleaved; float magnitude;
    T* q_out; T* k_out; T* v_out;
    int H, G, dk, dv, D;                        // G = 0: the mixer has no keys and values of its own
    int channels;
};

template <typename T>
__global__ void __launch_bounds__(128) conv_norm_rotate_kernel(const ConvPrep<T> p) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int req = p.token_request[n];
    if (req < 0) return;                                    // a padded row of a captured step
    const int pos = p.positions[n], idx = n - p.q_start[req], slot = p.state_slots[req];
    const bool alone = p.q_len[req] == 1;
    const int taps = p.taps, keep = taps - 1;
    const T* row = p.proj + (size_t)n * p.ld + p.col0;
    T* st = (keep > 0 && slot >= 0) ? p.state + (size_t)slot * keep * p.channels : nullptr;
    const int units = p.H + 2 * p.G;
    for (int u = warp; u < units; u += 4) {
        const int kind = u < p.H ? 0 : (u < p.H + p.G ? 1 : 2);
        const int head = kind == 0 ? u : (kind == 1 ? u - p.H : u - p.H - p.G);
        const int dims = kind == 2 ? p.dv : p.dk;
        const int base = kind == 0 ? head * p.dk : (kind == 1 ? p.H * p.dk + head * p.dk : (p.H + p.G) * p.dk + head * p.dv);
        float val[MAX_R][2];
        float ssq = 0.f;
#pragma unroll
        for (int r = 0; r < MAX_R; ++r)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = 2 * lane + 64 * r + e;
                float y = 0.f;
                if (c < dims) {
                    const int ch = base + c;
                    const float cur = to_float(row[ch]);
                    if (p.conv_w == nullptr) {
                        y = cur;
                    } else {
                        const float* w = p.conv_w + (size_t)ch * taps;
                        float past[MAX_TAPS];                   // past[b]: the projected value b positions back
                        past[0] = cur;
                        for (int b = 1; b < taps; ++b) {
                            float v = 0.f;
                            if (pos - b >= 0) {
                                if (idx - b >= 0) v = to_float(row[ch - (ptrdiff_t)b * p.ld]);
                                else if (st) v = to_float(st[(size_t)(keep + idx - b) * p.channels + ch]);
                            }
                            past[b] = v;
                        }
                        for (int j = 0; j < taps; ++j) y = fmaf(w[j], past[taps - 1 - j], y);
                        if (alone && st) {                      // oldest first: what was one back is now two back
                            for (int s = 0; s < keep; ++s)
                                st[(size_t)s * p.channels + ch] = from_float<T>(past[keep - 1 - s]);
                        }
                    }
                }
                val[r][e] = y;
                ssq = fmaf(y, y, ssq);
            }
        T* out = (kind == 0 ? p.q_out + (size_t)n * p.H * p.D : (kind == 1 ? p.k_out : p.v_out) + (size_t)n * p.G * p.D) +
                 (size_t)head * p.D;
        const float* g = kind == 0 ? p.q_norm : (kind == 1 ? p.k_norm : nullptr);
        if (kind != 2) {
            if (g != nullptr) {
                const float rinv = 1.0f / sqrtf(warp_sum(ssq) / (float)dims + p.eps);
#pragma unroll
                for (int r = 0; r < MAX_R; ++r)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int c = 2 * lane + 64 * r + e;
                        if (c < dims) val[r][e] *= rinv * g[c];
                    }
            }
            if (p.rot_dims > 0 && p.interleaved) {
#pragma unroll
                for (int r = 0; r < MAX_R; ++r) {
                    const int c = 2 * lane + 64 * r;
                    if (c + 1 < p.rot_dims) {
                        float sn, cs;
                        sincosf((float)pos * p.inv_freq[c >> 1], &sn, &cs);
                        sn *= p.magnitude; cs *= p.magnitude;
                        const float a = val[r][0], b = val[r][1];
                        val[r][0] = a * cs - b * sn;
                        val[r][1] = b * cs + a * sn;
                    }
                }
            }
        }
        if (kind != 2 && p.rot_dims > 0 && !p.interleaved) {
            // halves: channel i turns with channel i + rot_dims / 2, which another lane may own: through shared memory
            __shared__ float sh[4][64 * MAX_R];
            float* mine = sh[warp];
#pragma unroll
            for (int r = 0; r < MAX_R; ++r)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = 2 * lane + 64 * r + e;
                    if (c < dims) mine[c] = val[r][e];
                }
            __syncwarp();
            const int half = p.rot_dims / 2;
#pragma unroll
            for (int r = 0; r < MAX_R; ++r)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = 2 * lane + 64 * r + e;
                    if (c < p.rot_dims && c < dims) {
                        const int i = c < half ? c : c - half;
                        float sn, cs;
                        sincosf((float)pos * p.inv_freq[i], &sn, &cs);
                        sn *= p.magnitude; cs *= p.magnitude;
                        const float a = mine[i], b = mine[i + half];
                        val[r][e] = c < half ? a * cs - b * sn : b * cs + a * sn;
                    }
                }
            __syncwarp();
        }
#pragma unroll
        for (int r = 0; r < MAX_R; ++r)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = 2 * lane + 64 * r + e;
                if (c < p.D) out[c] = from_float<T>(c < dims ? val[r][e] : 0.f);
            }
    }
}

// After a step: the state of every request with more than one row (q_len 1: the kernel above did it) becomes its last
// taps - 1 projected values.  A thread owns a channel and walks the state from the oldest entry on: what it reads
// (further on in the old state, or this step's rows) it has not yet overwritten.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ proj, int ld, int col0, T* state, int keep, int channels,
                                         const int* __restrict__ q_start, const int* __restrict__ q_len,
                                         const int* __restrict__ state_slots) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.y;
    const int len = q_len[r], slot = state_slots[r];
    if (len <= 1 || slot < 0) return;
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= channels) return;
    T* st = state + (size_t)slot * keep * channels + ch;
    const T* rows = proj + (size_t)q_start[r] * ld + col0 + ch;
    for (int s = 0; s < keep; ++s) {
        const int rel = len - keep + s;                     // which of this step's rows it is; negative: still the old state's
        st[(size_t)s * channels] = rel >= 0 ? rows[(size_t)rel * ld] : st[(size_t)(s + len) * channels];
    }
}

template <typename T>
int launch(const void* proj, int ld, int col0, const float* conv_w, int taps, void* state, const int* token_request,
           const int* positions, const int* q_start, const int* q_len, const int* state_slots, int n_requests,
           int update_state, const float* q_norm, const float* k_norm, float eps, const float* inv_freq, int rot_dims,
           int interleaved, float magnitude, void* q_out, void* k_out, void* v_out, int N, int H, int G, int dk, int dv,
           int D, cudaStream_t stream) {
    ConvPrep<T> p;
    p.proj = (const T*)proj; p.ld = ld; p.col0 = col0; p.conv_w = conv_w; p.taps = conv_w ? taps : 1; p.state = (T*)state;
    p.token_request = token_request; p.positions = positions; p.q_start = q_start; p.q_len = q_len;
    p.state_slots = state_slots; p.q_norm = q_norm; p.k_norm = k_norm; p.eps = eps; p.inv_freq = inv_freq;
    p.rot_dims = inv_freq ? rot_dims : 0; p.interleaved = interleaved; p.magnitude = magnitude;
    p.q_out = (T*)q_out; p.k_out = (T*)k_out; p.v_out = (T*)v_out; p.H = H; p.G = G; p.dk = dk; p.dv = dv; p.D = D;
    p.channels = H * dk + G * (dk + dv);
    int rc = tnx_launch_in_order(conv_norm_rotate_kernel<T>, dim3(N), dim3(128), 0, stream, p);
    if (rc != 0 || !update_state || p.taps <= 1 || n_requests <= 0) return rc;
    return tnx_launch_in_order(conv_state_update_kernel<T>, dim3((p.channels + 127) / 128, n_requests), dim3(128), 0, stream,
                               (const T*)proj, ld, col0, (T*)state, p.taps - 1, p.channels, q_start, q_len, state_slots);
}
}  // namespace

// update_state: 0 when every request of the step has one row (nothing is left for the second kernel).
TNX_EXPORT int tnx_conv_qkv_prep(const void* proj, int ld, int col0, const float* conv_w, int taps, void* state,
                                 const int* token_request, const int* positions, const int* q_start, const int* q_len,
                                 const int* state_slots, int n_requests, int update_state, const float* q_norm,
                                 const float* k_norm, float eps, const float* inv_freq, int rot_dims, int interleaved,
                                 float magnitude, void* q_out, void* k_out, void* v_out, int N, int H, int G, int dk, int dv,
                                 int D, int is_h16, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || G < 0 || dk <= 0 || dv <= 0 || D < dk || D < dv || D > 64 * MAX_R || taps < 1 || taps > MAX_TAPS ||
        rot_dims < 0 || rot_dims % 2 || rot_dims > dk)
        return TNX_ERR_UNSUPPORTED;
    if (conv_w && taps > 1 && !state) return TNX_ERR_BAD_ARG;
    if (is_h16)
        return launch<h16>(proj, ld, col0, conv_w, taps, state, token_request, positions, q_start, q_len, state_slots,
                           n_requests, update_state, q_norm, k_norm, eps, inv_freq, rot_dims, interleaved, magnitude, q_out,
                           k_out, v_out, N, H, G, dk, dv, D, stream);
    return launch<float>(proj, ld, col0, conv_w, taps, state, token_request, positions, q_start, q_len, state_slots,
                         n_requests, update_state, q_norm, k_norm, eps, inv_freq, rot_dims, interleaved, magnitude, q_out,
                         k_out, v_out, N, H, G, dk, dv, D, stream);
}
