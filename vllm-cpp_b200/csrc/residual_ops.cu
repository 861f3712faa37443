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
// sinf and cosf are the accurate ones (no fast-math build).
template <typename T>
__global__ void embedding_sinusoid_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                          const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                          float* __restrict__ residual, int hidden, int vocab, float scale, int* status) {
    pdl_start();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = (unsigned)id < (unsigned)vocab;
    if (!ok && status && threadIdx.x == 0) atomicCAS(status, 0, VCB_STATUS_BAD_TOKEN);
    const T* row = table + (size_t)(ok ? id : 0) * hidden;
    const float p = (float)positions[t];
    float* out = residual + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float angle = p * inv_freq[i >> 1];
        const float pe = (i & 1) ? cosf(angle) : sinf(angle);
        out[i] = ok ? to_f32<T>(row[i]) * scale + pe : 0.0f;
    }
}

VCB_EXPORT int vcb_embedding_sinusoid(const void* table, const int* ids, const int* positions, const float* inv_freq,
                                      float* residual, int n_tokens, int hidden, int vocab, float scale, int* status,
                                      int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (vocab <= 0 || hidden <= 0) return VCB_ERR_BAD_ARG;
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32)
        vcb_launch(embedding_sinusoid_kernel<float>, n_tokens, threads, 0, s, (const float*)table, ids, positions, inv_freq,
                   residual, hidden, vocab, scale, status);
    else if (dtype == VCB_BF16)
        vcb_launch(embedding_sinusoid_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, (const __nv_bfloat16*)table, ids,
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

VCB_EXPORT int vcb_token_shift(const float* x, const float* mu, float* state, void* shifted, void* plain,
                               const int* q_start, const int* req_of_token, const int* positions,
                               const int* state_slots, int n_tokens, int hidden, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || !state || !shifted) return VCB_ERR_BAD_ARG;
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
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

VCB_EXPORT int vcb_gated_norm_residual(const void* y, const void* a, const float* b, const float* gain, int gain_stride,
                                       float* x, void* plain, int n_tokens, int hidden, float mult, float eps,
                                       int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || !y || !gain || !x || (gain_stride != 0 && gain_stride != 1)) return VCB_ERR_BAD_ARG;
    const int threads = hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
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
