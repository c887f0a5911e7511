// Retention: linear attention with a fixed decay per head, no softmax and no denominator.  Per head, with
// q_t, k_t of k_dim numbers and v_t of v_dim numbers:
//     S_t = decay * S_(t-1) + k_t v_t^T          (S: k_dim x v_dim, 32-bit, kept per request between steps)
//     o_t = S_t^T q_t
// Everything that enters the recurrence is 32-bit: queries and keys are rotated by position in 32-bit from the
// projection's output (tnx_retention_prep) and are not rounded again; the state lives in 32-bit.
//
// tnx_retention_prep: on the first rot_dims dims of each head, dim i paired with i + rot_dims/2, the pair
//   (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * inv_freq[i]; keys are then
//   multiplied by k_scale.  Output: 32-bit q and k, [tokens, heads * k_dim].
// tnx_retention_scan: a thread block owns C columns (value dims) of one head of one request and walks the
//   request's tokens of this step in order, the state's columns in registers: a column's k_dim rows are spread
//   over R adjacent lanes, which add their partial sums of o_t with shuffles.  The state is stored
//   [slot, head, v_dim, k_dim] (a column's rows side by side), so that the R lanes of a column read one
//   contiguous piece.  A step of one token per request streams the state through once; a portion of a prompt
//   keeps it in registers for all its tokens.  Queries and keys of a few tokens at a time are staged in shared memory.
// tnx_headwise_gated_rms_norm: o of each (token, head) divided by its root mean square (eps inside the root,
//   an optional weight over the head's dims), multiplied by silu(gate) and by out_scale, written in the
//   activation type.
#include "common.cuh"

namespace {

template <typename T>
__global__ void retention_prep_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off,
                                      const int* __restrict__ token_request, const int* __restrict__ positions,
                                      const float* __restrict__ inv_freq, int rot_dims, float k_scale,
                                      float* __restrict__ q_out, float* __restrict__ k_out, int H, int dk) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    if (token_request[n] < 0) return;
    const float pos = (float)positions[n];
    const T* row = proj + (size_t)n * ld;
    const int half = rot_dims / 2;
    float* qd = q_out + (size_t)n * H * dk;
    float* kd = k_out + (size_t)n * H * dk;
    for (int e = threadIdx.x; e < H * half; e += blockDim.x) {
        const int h = e / half, i = e % half;
        const int c0 = h * dk + i, c1 = c0 + half;
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        const float qu = to_float(row[q_off + c0]), qv = to_float(row[q_off + c1]);
        const float ku = to_float(row[k_off + c0]), kv = to_float(row[k_off + c1]);
        qd[c0] = qu * cs - qv * sn;
        qd[c1] = qv * cs + qu * sn;
        kd[c0] = (ku * cs - kv * sn) * k_scale;
        kd[c1] = (kv * cs + ku * sn) * k_scale;
    }
    const int rest = dk - rot_dims;
    for (int e = threadIdx.x; e < H * rest; e += blockDim.x) {
        const int c = (e / rest) * dk + rot_dims + e % rest;
        qd[c] = to_float(row[q_off + c]);
        kd[c] = to_float(row[k_off + c]) * k_scale;
    }
}

constexpr int SCAN_TOKENS = 8;        // tokens whose queries and keys are staged in shared memory at a time

// KPT: rows of a column one thread keeps; R: lanes a column's rows are spread over (KPT * R >= k_dim).
// VEC: a thread's rows come in runs of four (rows 4 (r + R m) .. + 3), read as one 16-byte piece.
template <typename T, int KPT, int R, bool VEC>
__global__ void __launch_bounds__(256)
retention_scan_kernel(const float* __restrict__ qr, const float* __restrict__ kr, const T* __restrict__ v, int v_ld,
                      const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ q_start,
                      const int* __restrict__ q_len, const int* __restrict__ state_slots, float* __restrict__ out,
                      int H, int dk, int dv, int C) {
    constexpr int DKP = KPT * R;
    extern __shared__ __align__(16) float sm[];       // q [SCAN_TOKENS][DKP], k [SCAN_TOKENS][DKP], v [SCAN_TOKENS][C]
    pdl_launch_dependents();
    pdl_wait();
    const int req = blockIdx.z, h = blockIdx.y;
    const int len = q_len[req];
    if (len <= 0) return;                            // a padded request of a captured batch
    const int slot = state_slots[req];
    if (slot < 0) return;
    const int t_first = q_start[req];
    float* qs = sm;
    float* ks = qs + SCAN_TOKENS * DKP;
    float* vs = ks + SCAN_TOKENS * DKP;
    const int jl = threadIdx.x / R, r = threadIdx.x % R;
    const int j = blockIdx.x * C + jl;
    const bool col = j < dv;
    const float dec = decay[h];
    float* st = state + (((size_t)slot * H + h) * dv + (col ? j : 0)) * dk;

    float S[KPT];
#pragma unroll
    for (int m = 0; m < KPT; ++m) {
        const int i = VEC ? 4 * (r + R * (m / 4)) + (m % 4) : r + R * m;
        S[m] = (col && i < dk) ? st[i] : 0.f;
    }
    for (int t0 = 0; t0 < len; t0 += SCAN_TOKENS) {
        const int nt = min(SCAN_TOKENS, len - t0);
        __syncthreads();
        for (int e = threadIdx.x; e < nt * DKP; e += blockDim.x) {
            const int tt = e / DKP, i = e % DKP;
            const size_t g = (size_t)(t_first + t0 + tt) * H * dk + (size_t)h * dk + i;
            qs[e] = i < dk ? qr[g] : 0.f;
            ks[e] = i < dk ? kr[g] : 0.f;
        }
        for (int e = threadIdx.x; e < nt * C; e += blockDim.x) {
            const int tt = e / C, c = blockIdx.x * C + e % C;
            vs[e] = c < dv ? to_float(v[(size_t)(t_first + t0 + tt) * v_ld + (size_t)h * dv + c]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float vj = vs[tt * C + jl];
            const float* kt = ks + tt * DKP;
            const float* qt = qs + tt * DKP;
            float acc = 0.f;
            if (VEC) {
#pragma unroll
                for (int m4 = 0; m4 < KPT / 4; ++m4) {
                    const float4 k4 = ((const float4*)kt)[r + R * m4];
                    const float4 q4 = ((const float4*)qt)[r + R * m4];
                    S[4 * m4 + 0] = fmaf(dec, S[4 * m4 + 0], k4.x * vj); acc = fmaf(S[4 * m4 + 0], q4.x, acc);
                    S[4 * m4 + 1] = fmaf(dec, S[4 * m4 + 1], k4.y * vj); acc = fmaf(S[4 * m4 + 1], q4.y, acc);
                    S[4 * m4 + 2] = fmaf(dec, S[4 * m4 + 2], k4.z * vj); acc = fmaf(S[4 * m4 + 2], q4.z, acc);
                    S[4 * m4 + 3] = fmaf(dec, S[4 * m4 + 3], k4.w * vj); acc = fmaf(S[4 * m4 + 3], q4.w, acc);
                }
            } else {
#pragma unroll
                for (int m = 0; m < KPT; ++m) {
                    S[m] = fmaf(dec, S[m], kt[r + R * m] * vj);
                    acc = fmaf(S[m], qt[r + R * m], acc);
                }
            }
#pragma unroll
            for (int o = R / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (r == 0 && col) out[(size_t)(t_first + t0 + tt) * H * dv + (size_t)h * dv + j] = acc;
        }
    }
    if (col) {
#pragma unroll
        for (int m = 0; m < KPT; ++m) {
            const int i = VEC ? 4 * (r + R * (m / 4)) + (m % 4) : r + R * m;
            if (i < dk) st[i] = S[m];
        }
    }
}

template <typename T>
__global__ void headwise_gated_rms_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_ld,
                                               const int* __restrict__ token_request, const float* __restrict__ w,
                                               float eps, float out_scale, T* __restrict__ out, int out_ld,
                                               int n_tokens, int H, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (pair >= (long long)n_tokens * H) return;
    const int n = (int)(pair / H), h = (int)(pair % H);
    if (token_request[n] < 0) return;
    const float* src = o + ((size_t)n * H + h) * dv;
    float s = 0.f;
    for (int c = lane; c < dv; c += 32) { const float v = src[c]; s += v * v; }
    s = warp_sum(s);
    const float rinv = 1.0f / sqrtf(s / (float)dv + eps);
    const T* g = gate ? gate + (size_t)n * gate_ld + (size_t)h * dv : nullptr;
    T* dst = out + (size_t)n * out_ld + (size_t)h * dv;
    for (int c = lane; c < dv; c += 32) {
        float y = src[c] * rinv;
        if (w) y *= w[c];
        if (g) { const float z = to_float(g[c]); y *= z / (1.f + expf(-z)); }
        dst[c] = from_float<T>(y * out_scale);
    }
}

}  // namespace

TNX_EXPORT int tnx_retention_prep(const void* proj, int ld, int q_off, int k_off, const int* token_request,
                                  const int* positions, const float* inv_freq, int rot_dims, float k_scale, float* q_out,
                                  float* k_out, int n_tokens, int H, int dk, int is_h16, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || dk <= 0 || rot_dims < 0 || rot_dims > dk || rot_dims % 2 || (rot_dims && !inv_freq)) return TNX_ERR_BAD_ARG;
    const int threads = H * dk >= 2048 ? 256 : 128;
    if (is_h16)
        return tnx_launch_in_order(retention_prep_kernel<h16>, dim3(n_tokens), dim3(threads), 0, stream, (const h16*)proj, ld,
                                   q_off, k_off, token_request, positions, inv_freq, rot_dims, k_scale, q_out, k_out, H, dk);
    return tnx_launch_in_order(retention_prep_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)proj, ld,
                               q_off, k_off, token_request, positions, inv_freq, rot_dims, k_scale, q_out, k_out, H, dk);
}

// The columns a thread block of the scan owns: 16 (8 where the head has fewer; columns beyond the head are
// idle lanes), so that even one request of a few heads spreads over many SMs and every block is whole warps.
TNX_EXPORT int tnx_retention_scan_columns(int dv) { return dv >= 16 ? 16 : 8; }

template <typename T>
static int retention_scan_launch(const float* qr, const float* kr, const T* v, int v_ld, const float* decay, float* state,
                                 const int* q_start, const int* q_len, const int* state_slots, float* out, int n_requests,
                                 int H, int dk, int dv, cudaStream_t stream) {
    const int C = tnx_retention_scan_columns(dv);
    const dim3 grid((dv + C - 1) / C, H, n_requests);
    const bool vec = dk % 4 == 0;
#define SCAN(KPT, R)                                                                                                    \
    do {                                                                                                                \
        const size_t smem = (size_t)SCAN_TOKENS * (2 * (KPT) * (R) + C) * sizeof(float);                                \
        if (vec && (KPT) % 4 == 0)                                                                                      \
            return tnx_launch_in_order(retention_scan_kernel<T, KPT, R, ((KPT) % 4 == 0)>, grid, dim3(C * (R)), smem,   \
                                       stream, qr, kr, v, v_ld, decay, state, q_start, q_len, state_slots, out, H, dk,  \
                                       dv, C);                                                                          \
        return tnx_launch_in_order(retention_scan_kernel<T, KPT, R, false>, grid, dim3(C * (R)), smem, stream, qr, kr,  \
                                   v, v_ld, decay, state, q_start, q_len, state_slots, out, H, dk, dv, C);              \
    } while (0)
    if (dk <= 16) SCAN(4, 4);
    if (dk <= 32) SCAN(4, 8);
    if (dk <= 64) SCAN(8, 8);
    if (dk <= 128) SCAN(16, 8);
    if (dk <= 256) SCAN(32, 8);
    return TNX_ERR_UNSUPPORTED;
#undef SCAN
}

TNX_EXPORT int tnx_retention_scan(const float* qr, const float* kr, const void* v, int v_ld, const float* decay,
                                  float* state, const int* q_start, const int* q_len, const int* state_slots, float* out,
                                  int n_requests, int H, int dk, int dv, int v_h16, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (H <= 0 || dk <= 0 || dv <= 0 || H > 65535 || n_requests > 65535) return TNX_ERR_BAD_ARG;
    if (v_h16)
        return retention_scan_launch<h16>(qr, kr, (const h16*)v, v_ld, decay, state, q_start, q_len, state_slots, out,
                                          n_requests, H, dk, dv, stream);
    return retention_scan_launch<float>(qr, kr, (const float*)v, v_ld, decay, state, q_start, q_len, state_slots, out,
                                        n_requests, H, dk, dv, stream);
}

TNX_EXPORT int tnx_headwise_gated_rms_norm(const float* o, const void* gate, int gate_ld, const int* token_request,
                                           const float* w, float eps, float out_scale, void* out, int out_ld,
                                           int n_tokens, int H, int dv, int is_h16, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || dv <= 0 || out_ld < H * dv) return TNX_ERR_BAD_ARG;
    const int warps = 4;
    const long long pairs = (long long)n_tokens * H;
    const int blocks = (int)((pairs + warps - 1) / warps);
    if (is_h16)
        return tnx_launch_in_order(headwise_gated_rms_norm_kernel<h16>, dim3(blocks), dim3(warps * 32), 0, stream, o,
                                   (const h16*)gate, gate_ld, token_request, w, eps, out_scale, (h16*)out, out_ld, n_tokens,
                                   H, dv);
    return tnx_launch_in_order(headwise_gated_rms_norm_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, o,
                               (const float*)gate, gate_ld, token_request, w, eps, out_scale, (float*)out, out_ld, n_tokens,
                               H, dv);
}
