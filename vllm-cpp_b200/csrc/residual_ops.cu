// Kernels around the residual stream for layers that are not "norm, sublayer, add":
//
//   embedding_sinusoid_kernel   x[t] = table[id] * scale + sinusoidal position vector
//   token_shift_kernel          s[t] = x[t] + (x[t-1] - x[t]) * mu, the row before a request's first row of
//                               this step taken from (and the step's last row left in) the request's state slot
//   gated_norm_residual_kernel  z = y * sigmoid(a + b);  x += mult * z / sqrt(mean(z^2) + eps) * gain
//                               (a norm on the sublayer's result, with one gain for all coordinates)
//
// The residual stream x, the state, sigmoids, sums of squares and angles are float whatever the storage
// type T of the activations is.  The reference has none of these (its layers are pre-norm blocks without
// gates, src/model/qwen.cpp:300-318).
#include "common.cuh"

// ------------------------------------------------- embedding with scale and sinusoidal positions
// Entry 2i of the position vector is sin(p * f_i), entry 2i+1 is cos(p * f_i); f_i (inv_freq, float,
// (hidden + 1) / 2 values) comes from the host.  The angle is the float product of the position and f_i;
// sincosf is the accurate one (no fast-math build).
template <typename T>
__global__ void embedding_sinusoid_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                          const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                          float* __restrict__ residual, int hidden, int vocab, float scale, int* status) {
    pdl_start();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = (unsigned)id < (unsigned)vocab;
    if (!ok && status && threadIdx.x == 0 && blockIdx.y == 0) atomicCAS(status, 0, VCB_STATUS_BAD_TOKEN);
    const T* row = table + (size_t)(ok ? id : 0) * hidden;
    const float p = (float)positions[t];
    float* out = residual + (size_t)t * hidden;
    // one thread per pair of entries: a sine and a cosine of the same angle
    const int pair = blockIdx.y * blockDim.x + threadIdx.x, i = 2 * pair;
    if (i >= hidden) return;
    float sn, cs;
    sincosf(p * inv_freq[pair], &sn, &cs);
    out[i] = ok ? to_f32<T>(row[i]) * scale + sn : 0.0f;
    if (i + 1 < hidden) out[i + 1] = ok ? to_f32<T>(row[i + 1]) * scale + cs : 0.0f;
}

VCB_EXPORT int vcb_embedding_sinusoid(const void* table, const int* ids, const int* positions, const float* inv_freq,
                                      float* residual, int n_tokens, int hidden, int vocab, float scale, int* status,
                                      int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (vocab <= 0 || hidden <= 0) return VCB_ERR_BAD_ARG;
    const int threads = 128, pairs = (hidden + 1) / 2;
    dim3 grid(n_tokens, (pairs + threads - 1) / threads);
    if (grid.y > 65535) return VCB_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32)
        vcb_launch(embedding_sinusoid_kernel<float>, grid, threads, 0, s, (const float*)table, ids, positions, inv_freq,
                   residual, hidden, vocab, scale, status);
    else if (dtype == VCB_BF16)
        vcb_launch(embedding_sinusoid_kernel<__nv_bfloat16>, grid, threads, 0, s, (const __nv_bfloat16*)table, ids,
                   positions, inv_freq, residual, hidden, vocab, scale, status);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ---------------------------------------------------------------- token shift
// One CTA per token row.  The row before row t is row t - 1 of the step unless t is its request's first
// row of the step: then it is zero at position 0 and the request's state slot otherwise.  The CTA of a
// request's first row also leaves the request's last row of this step in the slot, each thread after it
// has read the slot's old value for the same elements, so no other CTA touches the slot.
// Outputs: shifted (T, always) and plain (T, the unshifted row in the activations' type; may be null).
template <typename T>
__global__ void token_shift_kernel(const float* __restrict__ x, const float* __restrict__ mu, float* __restrict__ state,
                                   T* __restrict__ shifted, T* __restrict__ plain, const int* __restrict__ q_start,
                                   const int* __restrict__ req_of_token, const int* __restrict__ positions,
                                   const int* __restrict__ state_slots, int hidden) {
    pdl_start();
    const int t = blockIdx.x;
    const int r = req_of_token[t];
    const int first_row = q_start[r], last_row = q_start[r + 1] - 1;
    const bool first = t == first_row;
    const bool zero_prev = first && positions[t] == 0;
    float* slot = state + (size_t)state_slots[r] * hidden;
    const float* cur = x + (size_t)t * hidden;
    const float* prev = first ? slot : cur - hidden;
    const float* last = x + (size_t)last_row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float c = cur[i];
        const float p = zero_prev ? 0.0f : prev[i];
        if (first) slot[i] = last[i];
        shifted[(size_t)t * hidden + i] = from_f32<T>(c + (p - c) * mu[i]);
        if (plain) plain[(size_t)t * hidden + i] = from_f32<T>(c);
    }
}

// The same for bfloat16 rows of a multiple of 8 elements: one thread per 8 elements (two 16-byte loads of x and of
// the row before, 16-byte stores), any number of rows a CTA.
__global__ void token_shift_bf16x8_kernel(const float* __restrict__ x, const float* __restrict__ mu, float* __restrict__ state,
                                          __nv_bfloat16* __restrict__ shifted, __nv_bfloat16* __restrict__ plain,
                                          const int* __restrict__ q_start, const int* __restrict__ req_of_token,
                                          const int* __restrict__ positions, const int* __restrict__ state_slots,
                                          int n_tokens, int hidden) {
    pdl_start();
    const int nvec = hidden >> 3;
    const long long total = (long long)n_tokens * nvec;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(idx / nvec), i = (int)(idx - (long long)t * nvec) * 8;
        const int r = req_of_token[t];
        const int first_row = q_start[r];
        const bool first = t == first_row;
        float* slot = state + (size_t)state_slots[r] * hidden + i;
        const float* cur = x + (size_t)t * hidden + i;
        const float4 c0 = *reinterpret_cast<const float4*>(cur), c1 = *reinterpret_cast<const float4*>(cur + 4);
        float4 p0 = make_float4(0.f, 0.f, 0.f, 0.f), p1 = p0;
        if (!(first && positions[t] == 0)) {
            const float* prev = first ? slot : cur - hidden;
            p0 = *reinterpret_cast<const float4*>(prev);
            p1 = *reinterpret_cast<const float4*>(prev + 4);
        }
        if (first) {
            const float* last = x + (size_t)(q_start[r + 1] - 1) * hidden + i;
            const float4 l0 = *reinterpret_cast<const float4*>(last), l1 = *reinterpret_cast<const float4*>(last + 4);
            *reinterpret_cast<float4*>(slot) = l0;
            *reinterpret_cast<float4*>(slot + 4) = l1;
        }
        const float4 m0 = *reinterpret_cast<const float4*>(mu + i), m1 = *reinterpret_cast<const float4*>(mu + i + 4);
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        const float m[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        uint4 sv, pv;
        __nv_bfloat162* s2 = reinterpret_cast<__nv_bfloat162*>(&sv);
        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            s2[e] = __floats2bfloat162_rn(c[2 * e] + (p[2 * e] - c[2 * e]) * m[2 * e], c[2 * e + 1] + (p[2 * e + 1] - c[2 * e + 1]) * m[2 * e + 1]);
            p2[e] = __floats2bfloat162_rn(c[2 * e], c[2 * e + 1]);
        }
        *reinterpret_cast<uint4*>(shifted + (size_t)t * hidden + i) = sv;
        if (plain) *reinterpret_cast<uint4*>(plain + (size_t)t * hidden + i) = pv;
    }
}

VCB_EXPORT int vcb_token_shift(const float* x, const float* mu, float* state, void* shifted, void* plain,
                               const int* q_start, const int* req_of_token, const int* positions,
                               const int* state_slots, int n_tokens, int hidden, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || !state || !shifted) return VCB_ERR_BAD_ARG;
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    const uintptr_t addrs = (uintptr_t)x | (uintptr_t)mu | (uintptr_t)state | (uintptr_t)shifted | (uintptr_t)plain;
    if (dtype == VCB_BF16 && hidden % 8 == 0 && !(addrs & 15)) {
        const long long total = (long long)n_tokens * (hidden / 8);
        const long long want = (total + 255) / 256, cap = (long long)vcb_sm_count() * 16;
        vcb_launch(token_shift_bf16x8_kernel, (int)(want < cap ? want : cap), 256, 0, s, x, mu, state, (__nv_bfloat16*)shifted,
                   (__nv_bfloat16*)plain, q_start, req_of_token, positions, state_slots, n_tokens, hidden);
        return vcb_last_error();
    }
    if (dtype == VCB_F32)
        vcb_launch(token_shift_kernel<float>, n_tokens, threads, 0, s, x, mu, state, (float*)shifted, (float*)plain, q_start,
                   req_of_token, positions, state_slots, hidden);
    else if (dtype == VCB_BF16)
        vcb_launch(token_shift_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, x, mu, state, (__nv_bfloat16*)shifted,
                   (__nv_bfloat16*)plain, q_start, req_of_token, positions, state_slots, hidden);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------- gate, norm on the result, residual addition
// One CTA per row.  y: the sublayer's result; a: the gate's pre-activation (null: no gate), b: its bias
// (float, may be null).  z = y * sigmoid(a + b);  x += mult * (z / sqrt(mean(z^2) + eps)) * gain[0 or i].
// gain_stride 0: one gain for all coordinates, 1: a vector.  The new row is also written in the
// activations' type to `plain` when given (the next sublayer's input).  z is computed twice rather than
// kept, so no row length is too long.
template <typename T>
__device__ __forceinline__ float gated_value(const T* y, const T* a, const float* b, int i) {
    float z = to_f32<T>(y[i]);
    if (a) {
        const float pre = to_f32<T>(a[i]) + (b ? b[i] : 0.0f);
        z *= 1.0f / (1.0f + expf(-pre));
    }
    return z;
}

template <typename T>
__global__ void gated_norm_residual_kernel(const T* __restrict__ y, const T* __restrict__ a, const float* __restrict__ b,
                                           const float* __restrict__ gain, int gain_stride, float* __restrict__ x,
                                           T* __restrict__ plain, int hidden, float mult, float eps) {
    __shared__ float scratch[33];
    pdl_start();
    const size_t row = (size_t)blockIdx.x * hidden;
    const T* yr = y + row;
    const T* ar = a ? a + row : nullptr;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float z = gated_value<T>(yr, ar, b, i);
        ss += z * z;
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float z = gated_value<T>(yr, ar, b, i);
        const float v = x[row + i] + mult * ((z * r) * gain[(size_t)i * gain_stride]);
        x[row + i] = v;
        if (plain) plain[row + i] = from_f32<T>(v);
    }
}

// The same for bfloat16 rows of a multiple of 8 elements that fit the CTA's registers: NCH vectors of 8 elements a
// thread, 16-byte accesses, z kept between the two passes.
template <int NCH>
__global__ void gated_norm_residual_bf16x8_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ a,
                                                  const float* __restrict__ b, const float* __restrict__ gain, int gain_stride,
                                                  float* __restrict__ x, __nv_bfloat16* __restrict__ plain, int hidden,
                                                  float mult, float eps) {
    __shared__ float scratch[33];
    pdl_start();
    const size_t row = (size_t)blockIdx.x * hidden;
    const int nvec = hidden >> 3;
    float z[NCH][8];
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec) {
            const uint4 yv = *reinterpret_cast<const uint4*>(y + row + (size_t)i * 8);
            const __nv_bfloat162* y2 = reinterpret_cast<const __nv_bfloat162*>(&yv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(y2[e]);
                z[c][2 * e] = f.x;
                z[c][2 * e + 1] = f.y;
            }
            if (a) {
                const uint4 av = *reinterpret_cast<const uint4*>(a + row + (size_t)i * 8);
                const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
                float bb[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (b) {
                    const float4 b0 = *reinterpret_cast<const float4*>(b + i * 8), b1 = *reinterpret_cast<const float4*>(b + i * 8 + 4);
                    bb[0] = b0.x; bb[1] = b0.y; bb[2] = b0.z; bb[3] = b0.w; bb[4] = b1.x; bb[5] = b1.y; bb[6] = b1.z; bb[7] = b1.w;
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(a2[e]);
                    z[c][2 * e] *= 1.0f / (1.0f + expf(-(f.x + bb[2 * e])));
                    z[c][2 * e + 1] *= 1.0f / (1.0f + expf(-(f.y + bb[2 * e + 1])));
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += z[c][e] * z[c][e];
        }
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)hidden + eps);
    const float g0 = gain[0];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec) {
            float* xr = x + row + (size_t)i * 8;
            const float4 x0 = *reinterpret_cast<const float4*>(xr), x1 = *reinterpret_cast<const float4*>(xr + 4);
            float v[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] += mult * ((z[c][e] * r) * (gain_stride ? gain[i * 8 + e] : g0));
            *reinterpret_cast<float4*>(xr) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(xr + 4) = make_float4(v[4], v[5], v[6], v[7]);
            if (plain) {
                uint4 pv;
                __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pv);
#pragma unroll
                for (int e = 0; e < 4; ++e) p2[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
                *reinterpret_cast<uint4*>(plain + row + (size_t)i * 8) = pv;
            }
        }
    }
}

VCB_EXPORT int vcb_gated_norm_residual(const void* y, const void* a, const float* b, const float* gain, int gain_stride,
                                       float* x, void* plain, int n_tokens, int hidden, float mult, float eps,
                                       int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || !y || !gain || !x || (gain_stride != 0 && gain_stride != 1)) return VCB_ERR_BAD_ARG;
    const int threads = hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    const uintptr_t addrs = (uintptr_t)y | (uintptr_t)a | (uintptr_t)b | (uintptr_t)x | (uintptr_t)plain | (gain_stride ? (uintptr_t)gain : 0);
    if (dtype == VCB_BF16 && hidden % 8 == 0 && hidden / 8 <= 4 * 256 && !(addrs & 15)) {
        const int nvec = hidden / 8;
        const int vt = nvec >= 256 ? 256 : (nvec + 31) / 32 * 32;
        const int nch = (nvec + vt - 1) / vt;
        const __nv_bfloat16 *yb = (const __nv_bfloat16*)y, *ab = (const __nv_bfloat16*)a;
        __nv_bfloat16* pb = (__nv_bfloat16*)plain;
        if (nch == 1) vcb_launch(gated_norm_residual_bf16x8_kernel<1>, n_tokens, vt, 0, s, yb, ab, b, gain, gain_stride, x, pb, hidden, mult, eps);
        else if (nch == 2) vcb_launch(gated_norm_residual_bf16x8_kernel<2>, n_tokens, vt, 0, s, yb, ab, b, gain, gain_stride, x, pb, hidden, mult, eps);
        else vcb_launch(gated_norm_residual_bf16x8_kernel<4>, n_tokens, vt, 0, s, yb, ab, b, gain, gain_stride, x, pb, hidden, mult, eps);
        return vcb_last_error();
    }
    if (dtype == VCB_F32)
        vcb_launch(gated_norm_residual_kernel<float>, n_tokens, threads, 0, s, (const float*)y, (const float*)a, b, gain,
                   gain_stride, x, (float*)plain, hidden, mult, eps);
    else if (dtype == VCB_BF16)
        vcb_launch(gated_norm_residual_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, (const __nv_bfloat16*)y,
                   (const __nv_bfloat16*)a, b, gain, gain_stride, x, (__nv_bfloat16*)plain, hidden, mult, eps);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------- norm on a result, residual addition, and the norm before the next sublayer
// One CTA per row:  x += (y / sqrt(mean(y^2) + eps)) * gain;  next = (x / sqrt(mean(x^2) + eps_next)) * next_gain
// (next may be null: then only the addition).  gain holds whatever multiplies the normed result coordinate by
// coordinate (a norm's gain times a layer scale).  The new row stays in registers between the two reductions
// when it fits (up to PER values a thread), else x is read again.
template <typename T, int PER>
__global__ void norm_residual_norm_kernel(const T* __restrict__ y, const float* __restrict__ gain, float* __restrict__ x,
                                          const float* __restrict__ next_gain, T* __restrict__ next, int hidden,
                                          float eps, float eps_next) {
    __shared__ float scratch[33];
    pdl_start();
    const size_t row = (size_t)blockIdx.x * hidden;
    const bool kept = hidden <= PER * (int)blockDim.x;
    float v[PER];
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float z = to_f32<T>(y[row + i]);
        ss += z * z;
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)hidden + eps);
    float sx = 0.0f;
#pragma unroll
    for (int c = 0; c < PER; ++c) v[c] = 0.0f;
    if (kept) {
#pragma unroll
        for (int c = 0; c < PER; ++c) {
            const int i = threadIdx.x + c * blockDim.x;
            if (i < hidden) {
                v[c] = x[row + i] + (to_f32<T>(y[row + i]) * r) * gain[i];
                x[row + i] = v[c];
                sx += v[c] * v[c];
            }
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float nv = x[row + i] + (to_f32<T>(y[row + i]) * r) * gain[i];
            x[row + i] = nv;
            sx += nv * nv;
        }
    }
    if (!next) return;
    sx = block_sum(sx, scratch);
    const float rn = 1.0f / sqrtf(sx / (float)hidden + eps_next);
    if (kept) {
#pragma unroll
        for (int c = 0; c < PER; ++c) {
            const int i = threadIdx.x + c * blockDim.x;
            if (i < hidden) next[row + i] = from_f32<T>(v[c] * rn * next_gain[i]);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) next[row + i] = from_f32<T>(x[row + i] * rn * next_gain[i]);
    }
}

// The same for bfloat16 rows of a multiple of 8 elements that fit the CTA's registers: NCH vectors of 8 elements a
// thread, 16-byte accesses, the row kept between the passes.
template <int NCH>
__global__ void norm_residual_norm_bf16x8_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ gain, float* __restrict__ x,
                                                 const float* __restrict__ next_gain, __nv_bfloat16* __restrict__ next, int hidden,
                                                 float eps, float eps_next) {
    __shared__ float scratch[33];
    pdl_start();
    const size_t row = (size_t)blockIdx.x * hidden;
    const int nvec = hidden >> 3;
    float v[NCH][8];
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec) {
            const uint4 yv = *reinterpret_cast<const uint4*>(y + row + (size_t)i * 8);
            const __nv_bfloat162* y2 = reinterpret_cast<const __nv_bfloat162*>(&yv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(y2[e]);
                v[c][2 * e] = f.x;
                v[c][2 * e + 1] = f.y;
                ss += f.x * f.x + f.y * f.y;
            }
        }
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)hidden + eps);
    float sx = 0.0f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec) {
            float* xr = x + row + (size_t)i * 8;
            const float4 x0 = *reinterpret_cast<const float4*>(xr), x1 = *reinterpret_cast<const float4*>(xr + 4);
            const float4 g0 = *reinterpret_cast<const float4*>(gain + i * 8), g1 = *reinterpret_cast<const float4*>(gain + i * 8 + 4);
            const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            const float gs[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[c][e] = xs[e] + (v[c][e] * r) * gs[e];
                sx += v[c][e] * v[c][e];
            }
            *reinterpret_cast<float4*>(xr) = make_float4(v[c][0], v[c][1], v[c][2], v[c][3]);
            *reinterpret_cast<float4*>(xr + 4) = make_float4(v[c][4], v[c][5], v[c][6], v[c][7]);
        }
    }
    if (!next) return;
    sx = block_sum(sx, scratch);
    const float rn = 1.0f / sqrtf(sx / (float)hidden + eps_next);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec) {
            const float4 g0 = *reinterpret_cast<const float4*>(next_gain + i * 8), g1 = *reinterpret_cast<const float4*>(next_gain + i * 8 + 4);
            const float gs[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            uint4 pv;
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pv);
#pragma unroll
            for (int e = 0; e < 4; ++e) p2[e] = __floats2bfloat162_rn(v[c][2 * e] * rn * gs[2 * e], v[c][2 * e + 1] * rn * gs[2 * e + 1]);
            *reinterpret_cast<uint4*>(next + row + (size_t)i * 8) = pv;
        }
    }
}

VCB_EXPORT int vcb_norm_residual_norm(const void* y, const float* gain, float* x, const float* next_gain, void* next,
                                      int n_tokens, int hidden, float eps, float eps_next, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || !y || !gain || !x || (next && !next_gain)) return VCB_ERR_BAD_ARG;
    const int threads = hidden >= 4096 ? 512 : hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    const uintptr_t addrs = (uintptr_t)y | (uintptr_t)gain | (uintptr_t)x | (uintptr_t)next_gain | (uintptr_t)next;
    if (dtype == VCB_BF16 && hidden % 8 == 0 && hidden / 8 <= 4 * 256 && !(addrs & 15)) {
        const int nvec = hidden / 8;
        const int vt = nvec >= 256 ? 256 : (nvec + 31) / 32 * 32;
        const int nch = (nvec + vt - 1) / vt;
        const __nv_bfloat16* yb = (const __nv_bfloat16*)y;
        __nv_bfloat16* nb = (__nv_bfloat16*)next;
        if (nch == 1) vcb_launch(norm_residual_norm_bf16x8_kernel<1>, n_tokens, vt, 0, s, yb, gain, x, next_gain, nb, hidden, eps, eps_next);
        else if (nch == 2) vcb_launch(norm_residual_norm_bf16x8_kernel<2>, n_tokens, vt, 0, s, yb, gain, x, next_gain, nb, hidden, eps, eps_next);
        else vcb_launch(norm_residual_norm_bf16x8_kernel<4>, n_tokens, vt, 0, s, yb, gain, x, next_gain, nb, hidden, eps, eps_next);
        return vcb_last_error();
    }
    if (dtype == VCB_F32)
        vcb_launch(norm_residual_norm_kernel<float, 16>, n_tokens, threads, 0, s, (const float*)y, gain, x, next_gain, (float*)next,
                   hidden, eps, eps_next);
    else if (dtype == VCB_BF16)
        vcb_launch(norm_residual_norm_kernel<__nv_bfloat16, 16>, n_tokens, threads, 0, s, (const __nv_bfloat16*)y, gain, x, next_gain,
                   (__nv_bfloat16*)next, hidden, eps, eps_next);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}
