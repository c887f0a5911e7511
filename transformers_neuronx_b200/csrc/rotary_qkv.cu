// What lies between the q/k/v projection and the paged attention kernels for an attention whose queries and
// keys are normalised over the whole projection, rotated by position (and whose values are rotated too), and
// what lies behind them.  Everything here is computed in 32-bit from the projection's output and rounded once.
//
// tnx_rotary_qkv_prep, one thread block per token at position p:
//   q <- q / sqrt(mean_all(q^2) + eps) * wq        (over all heads at once; skipped without wq)
//   k <- k / sqrt(mean_all(k^2) + eps) * wk
//   on the first `rot_dims` dims of each head of q and k, dim i paired with dim i + rot_dims/2:
//       (u, v) <- (u cos a - v sin a, v cos a + u sin a),  a = p * inv_freq_qk[i]
//   q of head h <- q * head_scale[h]                (skipped without head_scale)
//   values, when inv_freq_v is given: over all v_dim dims, dim m paired with m + v_dim/2, a = p * inv_freq_v[m]
//   q, k and v are written with `D` dims a head (D >= k_dim, v_dim; the rest zero), the layout the paged
//   attention kernels take: zeros in q and k leave the scores alone, zeros in v give zero output columns.
//
// tnx_rotary_unrotate, one thread block per token at position p: each head's first v_dim output dims of the
// attention (D a head) are turned back, pair m by -p * inv_freq_v[m], multiplied by out_scale and written
// v_dim a head into a (possibly wider) activation buffer.
#include "common.cuh"
#pragma nv_diag_suppress 128      // the plain loops behind a vectorised branch that returns are unreachable in that instantiation

namespace {

// eight 16-bit values <-> eight floats (one 16-byte piece)
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
    const h16x2* p = (const h16x2*)&raw;
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = h16x2_to_float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 raw;
    h16x2* p = (h16x2*)&raw;
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = floats_to_h16x2(f[2 * i], f[2 * i + 1]);
    return raw;
}

// VEC8 (16-bit types; every size a multiple of 8 and every row 16-byte aligned): rows are read and written in
// 16-byte pieces, a thread turning eight neighbouring pairs at a time.
template <typename T, bool VEC8>
__global__ void rotary_qkv_prep_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
                                       const int* __restrict__ token_request, const int* __restrict__ positions,
                                       const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                       const float* __restrict__ head_scale, const float* __restrict__ inv_freq_qk,
                                       int rot_dims, const float* __restrict__ inv_freq_v, T* __restrict__ q_out,
                                       T* __restrict__ k_out, T* __restrict__ v_out, int H, int G, int dk, int dv, int D) {
    extern __shared__ float sm[];                   // q [H * dk], k [G * dk], v [G * dv], then cos/sin of the token's angles
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    if (token_request[n] < 0) return;               // a padded row of a captured batch
    const float pos = (float)positions[n];
    const T* row = proj + (size_t)n * ld;
    float* qs = sm;
    float* ks = qs + H * dk;
    float* vs = ks + G * dk;
    const int nq = H * dk, nk = G * dk, nv = G * dv;
    // every head turns by the same angles: their sines and cosines are computed once per token
    const int half = rot_dims / 2, hv = inv_freq_v ? dv / 2 : 0;
    float* cs_qk = vs + nv;
    float* sn_qk = cs_qk + half;
    float* cs_v = sn_qk + half;
    float* sn_v = cs_v + hv;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq_qk[i], &sn_qk[i], &cs_qk[i]);
    for (int i = threadIdx.x; i < hv; i += blockDim.x) sincosf(pos * inv_freq_v[i], &sn_v[i], &cs_v[i]);
    float sq = 0.f, sk = 0.f;
    if constexpr (VEC8) {
        for (int c = threadIdx.x; c < (nq + nk + nv) / 8; c += blockDim.x) {
            const int e = 8 * c;                       // q, k and v follow one another in shared memory
            const int col = e < nq ? q_off + e : (e < nq + nk ? k_off + e - nq : v_off + e - nq - nk);
            float f[8];
            unpack8(*(const uint4*)(row + col), f);
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) { qs[e + i] = f[i]; ss += f[i] * f[i]; }
            if (e < nq) sq += ss; else if (e < nq + nk) sk += ss;
        }
    } else {
        for (int c = threadIdx.x; c < nq; c += blockDim.x) { const float v = to_float(row[q_off + c]); qs[c] = v; sq += v * v; }
        for (int c = threadIdx.x; c < nk; c += blockDim.x) { const float v = to_float(row[k_off + c]); ks[c] = v; sk += v * v; }
        for (int c = threadIdx.x; c < nv; c += blockDim.x) vs[c] = to_float(row[v_off + c]);
    }
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);                    // block_sum synchronises: the rows are in shared memory now
    const float rq = wq ? 1.0f / sqrtf(sq / (float)nq + eps) : 1.f;
    const float rk = wk ? 1.0f / sqrtf(sk / (float)nk + eps) : 1.f;

    // queries and keys: pairs of the rotated part, then the dims that pass unchanged, then the padding
    for (int which = 0; which < 2; ++which) {
        const int heads = which ? G : H;
        const float* src = which ? ks : qs;
        const float* w = which ? wk : wq;
        const float rinv = which ? rk : rq;
        T* dst = (which ? k_out : q_out) + (size_t)n * heads * D;
        if constexpr (VEC8) {
            const int h8 = half / 8;
            for (int e = threadIdx.x; e < heads * h8; e += blockDim.x) {
                const int h = e / h8, i0 = (e % h8) * 8;
                const int c0 = h * dk + i0, c1 = c0 + half;
                const float hs = (!which && head_scale) ? head_scale[h] : 1.f;
                float a[8], b[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float u = src[c0 + i] * rinv, v = src[c1 + i] * rinv;
                    if (w) { u *= w[c0 + i]; v *= w[c1 + i]; }
                    const float sn = sn_qk[i0 + i], cs = cs_qk[i0 + i];
                    a[i] = (u * cs - v * sn) * hs;
                    b[i] = (v * cs + u * sn) * hs;
                }
                *(uint4*)(dst + h * D + i0) = pack8(a);
                *(uint4*)(dst + h * D + i0 + half) = pack8(b);
            }
            const int rest8 = (D - rot_dims) / 8;
            for (int e = threadIdx.x; e < heads * rest8; e += blockDim.x) {
                const int h = e / rest8, c = rot_dims + (e % rest8) * 8;
                const float hs = (!which && head_scale) ? head_scale[h] : 1.f;
                float y[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    y[i] = 0.f;
                    if (c + i < dk) { y[i] = src[h * dk + c + i] * rinv * hs; if (w) y[i] *= w[h * dk + c + i]; }
                }
                *(uint4*)(dst + h * D + c) = pack8(y);
            }
            continue;
        }
        for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
            const int h = e / half, i = e % half;
            const int c0 = h * dk + i, c1 = c0 + half;
            float u = src[c0] * rinv, v = src[c1] * rinv;
            if (w) { u *= w[c0]; v *= w[c1]; }
            const float sn = sn_qk[i], cs = cs_qk[i];
            float a = u * cs - v * sn, b = v * cs + u * sn;
            if (!which && head_scale) { a *= head_scale[h]; b *= head_scale[h]; }
            dst[h * D + i] = from_float<T>(a);
            dst[h * D + i + half] = from_float<T>(b);
        }
        const int rest = D - rot_dims;
        for (int e = threadIdx.x; e < heads * rest; e += blockDim.x) {
            const int h = e / rest, c = rot_dims + e % rest;
            float y = 0.f;
            if (c < dk) {
                y = src[h * dk + c] * rinv;
                if (w) y *= w[h * dk + c];
                if (!which && head_scale) y *= head_scale[h];
            }
            dst[h * D + c] = from_float<T>(y);
        }
    }
    // values
    T* vd = v_out + (size_t)n * G * D;
    if constexpr (VEC8) {
        if (inv_freq_v) {
            const int h8 = hv / 8;
            for (int e = threadIdx.x; e < G * h8; e += blockDim.x) {
                const int h = e / h8, m0 = (e % h8) * 8;
                float a[8], b[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float u = vs[h * dv + m0 + i], v = vs[h * dv + m0 + hv + i];
                    a[i] = u * cs_v[m0 + i] - v * sn_v[m0 + i];
                    b[i] = v * cs_v[m0 + i] + u * sn_v[m0 + i];
                }
                *(uint4*)(vd + h * D + m0) = pack8(a);
                *(uint4*)(vd + h * D + m0 + hv) = pack8(b);
            }
        } else {
            for (int e = threadIdx.x; e < nv / 8; e += blockDim.x) {
                float y[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) y[i] = vs[8 * e + i];
                *(uint4*)(vd + ((8 * e) / dv) * D + (8 * e) % dv) = pack8(y);
            }
        }
        const int vrest8 = (D - dv) / 8;
        const float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int e = threadIdx.x; e < G * vrest8; e += blockDim.x) *(uint4*)(vd + (e / vrest8) * D + dv + (e % vrest8) * 8) = pack8(zero);
        return;
    }
    if (inv_freq_v) {
        for (int e = threadIdx.x; e < G * hv; e += blockDim.x) {
            const int h = e / hv, m = e % hv;
            const float u = vs[h * dv + m], v = vs[h * dv + m + hv];
            const float sn = sn_v[m], cs = cs_v[m];
            vd[h * D + m] = from_float<T>(u * cs - v * sn);
            vd[h * D + m + hv] = from_float<T>(v * cs + u * sn);
        }
    } else {
        for (int e = threadIdx.x; e < nv; e += blockDim.x) vd[(e / dv) * D + e % dv] = from_float<T>(vs[e]);
    }
    const int vrest = D - dv;
    for (int e = threadIdx.x; e < G * vrest; e += blockDim.x) vd[(e / vrest) * D + dv + e % vrest] = from_float<T>(0.f);
}

template <typename T, bool VEC8>
__global__ void rotary_unrotate_kernel(const T* __restrict__ att, const int* __restrict__ token_request,
                                       const int* __restrict__ positions, const float* __restrict__ inv_freq_v,
                                       float out_scale, T* __restrict__ out, int out_ld, int H, int dv, int D) {
    extern __shared__ float sm[];                   // cos and sin of the token's angles, the same for every head
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    if (token_request[n] < 0) return;
    const float pos = (float)positions[n];
    const T* src = att + (size_t)n * H * D;
    T* dst = out + (size_t)n * out_ld;
    if (inv_freq_v) {
        const int hv = dv / 2;
        float* cs_v = sm;
        float* sn_v = sm + hv;
        for (int i = threadIdx.x; i < hv; i += blockDim.x) sincosf(pos * inv_freq_v[i], &sn_v[i], &cs_v[i]);
        __syncthreads();
        if constexpr (VEC8) {
            const int h8 = hv / 8;
            for (int e = threadIdx.x; e < H * h8; e += blockDim.x) {
                const int h = e / h8, m0 = (e % h8) * 8;
                float u[8], v[8], a[8], b[8];
                unpack8(*(const uint4*)(src + h * D + m0), u);
                unpack8(*(const uint4*)(src + h * D + m0 + hv), v);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    a[i] = (u[i] * cs_v[m0 + i] + v[i] * sn_v[m0 + i]) * out_scale;
                    b[i] = (v[i] * cs_v[m0 + i] - u[i] * sn_v[m0 + i]) * out_scale;
                }
                *(uint4*)(dst + h * dv + m0) = pack8(a);
                *(uint4*)(dst + h * dv + m0 + hv) = pack8(b);
            }
            return;
        }
        for (int e = threadIdx.x; e < H * hv; e += blockDim.x) {
            const int h = e / hv, m = e % hv;
            const float u = to_float(src[h * D + m]), v = to_float(src[h * D + m + hv]);
            const float sn = sn_v[m], cs = cs_v[m];                 // the turn by -a: (u cos a + v sin a, v cos a - u sin a)
            dst[h * dv + m] = from_float<T>((u * cs + v * sn) * out_scale);
            dst[h * dv + m + hv] = from_float<T>((v * cs - u * sn) * out_scale);
        }
    } else {
        for (int e = threadIdx.x; e < H * dv; e += blockDim.x)
            dst[e] = from_float<T>(to_float(src[(e / dv) * D + e % dv]) * out_scale);
    }
}

}  // namespace

TNX_EXPORT int tnx_rotary_qkv_prep(const void* proj, int ld, int q_off, int k_off, int v_off, const int* token_request,
                                   const int* positions, const float* wq, const float* wk, float eps,
                                   const float* head_scale, const float* inv_freq_qk, int rot_dims,
                                   const float* inv_freq_v, void* q_out, void* k_out, void* v_out, int n_tokens, int H,
                                   int G, int dk, int dv, int D, int is_h16, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || D < dk || D < dv || rot_dims < 0 || rot_dims > dk || rot_dims % 2 ||
        (rot_dims && !inv_freq_qk) || (inv_freq_v && dv % 2))
        return TNX_ERR_BAD_ARG;
    const size_t smem = (size_t)(H * dk + G * dk + G * dv + rot_dims + dv) * sizeof(float);
    if (smem > 200 * 1024) return TNX_ERR_UNSUPPORTED;
    const int threads = 256;
#define PREP_LAUNCH(T, V8)                                                                                              \
    do {                                                                                                                \
        if (smem + 1024 > 48 * 1024)                                                                                    \
            cudaFuncSetAttribute(rotary_qkv_prep_kernel<T, V8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return tnx_launch_in_order(rotary_qkv_prep_kernel<T, V8>, dim3(n_tokens), dim3(threads), smem, stream,          \
                                   (const T*)proj, ld, q_off, k_off, v_off, token_request, positions, wq, wk, eps,      \
                                   head_scale, inv_freq_qk, rot_dims, inv_freq_v, (T*)q_out, (T*)k_out, (T*)v_out, H,   \
                                   G, dk, dv, D);                                                                       \
    } while (0)
    const bool v8 = is_h16 && dk % 8 == 0 && dv % 8 == 0 && D % 8 == 0 && rot_dims % 16 == 0 && (!inv_freq_v || dv % 16 == 0) &&
                    ld % 8 == 0 && q_off % 8 == 0 && k_off % 8 == 0 && v_off % 8 == 0 && ((uintptr_t)proj % 16) == 0 &&
                    ((uintptr_t)q_out % 16) == 0 && ((uintptr_t)k_out % 16) == 0 && ((uintptr_t)v_out % 16) == 0;
    if (is_h16 && v8) PREP_LAUNCH(h16, true);
    if (is_h16) PREP_LAUNCH(h16, false);
    PREP_LAUNCH(float, false);
#undef PREP_LAUNCH
}

TNX_EXPORT int tnx_rotary_unrotate(const void* att, const int* token_request, const int* positions,
                                   const float* inv_freq_v, float out_scale, void* out, int out_ld, int n_tokens, int H,
                                   int dv, int D, int is_h16, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || dv <= 0 || D < dv || (inv_freq_v && dv % 2) || out_ld < H * dv) return TNX_ERR_BAD_ARG;
    const int threads = H * dv >= 2048 ? 256 : 128;
    const size_t smem = (size_t)dv * sizeof(float);
    if (smem > 48 * 1024) return TNX_ERR_UNSUPPORTED;
    const bool v8 = is_h16 && inv_freq_v && dv % 16 == 0 && D % 8 == 0 && out_ld % 8 == 0 && ((uintptr_t)att % 16) == 0 &&
                    ((uintptr_t)out % 16) == 0;
    if (is_h16 && v8)
        return tnx_launch_in_order(rotary_unrotate_kernel<h16, true>, dim3(n_tokens), dim3(threads), smem, stream, (const h16*)att,
                                   token_request, positions, inv_freq_v, out_scale, (h16*)out, out_ld, H, dv, D);
    if (is_h16)
        return tnx_launch_in_order(rotary_unrotate_kernel<h16, false>, dim3(n_tokens), dim3(threads), smem, stream, (const h16*)att,
                                   token_request, positions, inv_freq_v, out_scale, (h16*)out, out_ld, H, dv, D);
    return tnx_launch_in_order(rotary_unrotate_kernel<float, false>, dim3(n_tokens), dim3(threads), smem, stream, (const float*)att,
                               token_request, positions, inv_freq_v, out_scale, (float*)out, out_ld, H, dv, D);
}
