// Mixers whose memory is a matrix per head that decays and takes up an outer product at every token:
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T        S: [dk, dv] float, one per (request, head), zero at admission
//     o_t = S_t^T q_t
//
//   decayed_state_scan_kernel   runs the recurrence over a step's tokens, request by request, from the state the
//                               request's slot holds, and leaves the new state there.  The decay a_t is either one
//                               number per head (constant over tokens and key channels) or one per key channel and
//                               token, sigmoid(z + b)^(1/tau) of a projection z, computed here through its logarithm.
//                               q, k and v may pass through silu on the way in, q through a constant factor.
//   gated_group_norm_kernel     RMS norm of the result over groups of channels (a head, or all heads together)
//                               times silu or sigmoid of a gate, rounded to the activations' type for the output product.
//
// The state, the decays and their logarithms, the activations, the sums and the norm are float whatever the
// storage type T of the projections is.  The reference has no recurrent mixer (its one mixer is
// src/layers/attention.cpp).
#include "common.cuh"

struct ScanArgs {
    const void* q;              // [n, H * dk] rows of the step's tokens, row stride ldq (elements)
    const void* k;
    const void* v;              // [n, H * dv]
    const void* decay_pre;      // [n, H * dk] or null: pre-activation of the per-channel decay
    long long ldq, ldk, ldv, ldd;
    const float* decay_bias;    // [H * dk] or null
    const float* decay_const;   // [H] or null: the decay of a head when decay_pre is null (1 if both are null)
    float inv_tau, q_scale;
    int act;                    // 1: silu on q, k and v
    float* state;               // [slots][H][dk][dv]
    float* out;                 // [n, H * dv], row stride ldo
    long long ldo;
    const int* q_start;
    const int* state_slots;
    int H, dk, dv, chunk;       // chunk: tokens staged in shared memory at a time
    // For long portions cut into pieces that run side by side (see decayed_state_carry_kernel): every piece is a
    // "request" of its own here.  fresh: S starts from zero and the slot is only written.  qp (may be null): float
    // [n, H * dk], row stride ldqp, receives q_t (activated, scaled) times the product of the decays from the piece's
    // first token through t; dtot (may be null): float [pieces, H, dk], the product over the whole piece.
    int fresh;
    float* qp;
    long long ldqp;
    float* dtot;
};

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
// ln(sigmoid(z)) without cancellation on either side
__device__ __forceinline__ float log_sigmoid_f(float z) { return z < 0.0f ? z - log1pf(expf(z)) : -log1pf(expf(-z)); }

// Grid (request, head, tile of value channels); block (DVT value channels, parts): thread (x, y) keeps rows
// y * DKP .. y * DKP + DKP - 1 of column x of S in registers.  Key channels beyond dk are padded with k = q = 0.
template <typename T, int DKP>
__global__ void decayed_state_scan_kernel(ScanArgs a) {
    extern __shared__ __align__(16) float sm[];
    pdl_start();
    const int r = blockIdx.x, h = blockIdx.y, dvt = blockDim.x, col0 = blockIdx.z * dvt;
    const int tx = threadIdx.x, part = threadIdx.y, parts = blockDim.y;
    const int dkpad = parts * DKP, TC = a.chunk;
    float* qs = sm;
    float* ks = qs + TC * dkpad;
    float* as = ks + TC * dkpad;
    float* vs = as + TC * dkpad;
    float* ps = vs + TC * dvt;
    float* carry = ps + parts * TC * dvt;         // [dkpad]: product of the decays so far, per key channel
    const int row0 = a.q_start[r], row1 = a.q_start[r + 1];
    const int col = col0 + tx;
    const bool col_ok = col < a.dv;
    float* st = a.state + (((size_t)a.state_slots[r] * a.H + h) * a.dk) * a.dv;
    float S[DKP];
#pragma unroll
    for (int i = 0; i < DKP; ++i) {
        const int kr = part * DKP + i;
        S[i] = (col_ok && kr < a.dk && !a.fresh) ? st[(size_t)kr * a.dv + col] : 0.0f;
    }
    const int tid = part * dvt + tx, nthreads = dvt * parts;
    const bool tracks = (a.qp || a.dtot) && blockIdx.z == 0;      // one block per (piece, head) follows the decays' product
    if (tracks) for (int i = tid; i < dkpad; i += nthreads) carry[i] = 1.0f;
    const float dconst = a.decay_const ? a.decay_const[h] : 1.0f;
    const T* q = (const T*)a.q;
    const T* k = (const T*)a.k;
    const T* v = (const T*)a.v;
    const T* dp = (const T*)a.decay_pre;
    for (int c0 = row0; c0 < row1; c0 += TC) {
        const int tc = min(TC, row1 - c0);
        __syncthreads();                          // the chunk before has been read
        // four elements a thread at a time: all their loads are issued before the first is used
        for (int base = tid; base < tc * dkpad; base += 4 * nthreads) {
            float rq[4], rk[4], rz[4];
            bool in[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int idx = base + j * nthreads;
                const int tt = idx / dkpad, i = idx - tt * dkpad;
                in[j] = idx < tc * dkpad && i < a.dk;
                rq[j] = rk[j] = rz[j] = 0.0f;
                if (in[j]) {
                    const size_t row = (size_t)(c0 + tt);
                    const int c = h * a.dk + i;
                    rq[j] = to_f32<T>(q[row * a.ldq + c]);
                    rk[j] = to_f32<T>(k[row * a.ldk + c]);
                    if (dp) rz[j] = to_f32<T>(dp[row * a.ldd + c]) + (a.decay_bias ? a.decay_bias[c] : 0.0f);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int idx = base + j * nthreads;
                if (idx >= tc * dkpad) continue;
                float qv = 0.0f, kv = 0.0f, av = 1.0f;
                if (in[j]) {
                    qv = rq[j];
                    kv = rk[j];
                    if (a.act) { qv = silu_f(qv); kv = silu_f(kv); }
                    qv *= a.q_scale;
                    av = dp ? expf(log_sigmoid_f(rz[j]) * a.inv_tau) : dconst;
                }
                qs[idx] = qv;
                ks[idx] = kv;
                as[idx] = av;
            }
        }
        for (int idx = tid; idx < tc * dvt; idx += nthreads) {
            const int tt = idx / dvt, j = idx - tt * dvt, c = col0 + j;
            float vv = c < a.dv ? to_f32<T>(v[(size_t)(c0 + tt) * a.ldv + h * a.dv + c]) : 0.0f;
            if (a.act) vv = silu_f(vv);
            vs[idx] = vv;
        }
        __syncthreads();
        if (tracks) {
            for (int i = tid; i < a.dk; i += nthreads) {
                float run = carry[i];
                for (int tt = 0; tt < tc; ++tt) {
                    run *= as[tt * dkpad + i];
                    if (a.qp) a.qp[(size_t)(c0 + tt) * a.ldqp + h * a.dk + i] = qs[tt * dkpad + i] * run;
                }
                carry[i] = run;
            }
        }
        for (int tt = 0; tt < tc; ++tt) {
            const float vv = vs[tt * dvt + tx];
            // 16-byte reads of the token's q, k and decays (the same addresses for the whole warp); four sums in flight
            const float4* qq = reinterpret_cast<const float4*>(qs + tt * dkpad + part * DKP);
            const float4* kk = reinterpret_cast<const float4*>(ks + tt * dkpad + part * DKP);
            const float4* aa = reinterpret_cast<const float4*>(as + tt * dkpad + part * DKP);
            float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
#pragma unroll
            for (int i = 0; i < DKP / 4; ++i) {
                const float4 a4 = aa[i], k4 = kk[i], q4 = qq[i];
                S[4 * i] = fmaf(a4.x, S[4 * i], k4.x * vv);
                S[4 * i + 1] = fmaf(a4.y, S[4 * i + 1], k4.y * vv);
                S[4 * i + 2] = fmaf(a4.z, S[4 * i + 2], k4.z * vv);
                S[4 * i + 3] = fmaf(a4.w, S[4 * i + 3], k4.w * vv);
                acc0 = fmaf(S[4 * i], q4.x, acc0);
                acc1 = fmaf(S[4 * i + 1], q4.y, acc1);
                acc2 = fmaf(S[4 * i + 2], q4.z, acc2);
                acc3 = fmaf(S[4 * i + 3], q4.w, acc3);
            }
            ps[(part * TC + tt) * dvt + tx] = (acc0 + acc1) + (acc2 + acc3);
        }
        __syncthreads();
        for (int idx = tid; idx < tc * dvt; idx += nthreads) {
            const int tt = idx / dvt, j = idx - tt * dvt, c = col0 + j;
            if (c >= a.dv) continue;
            float s = 0.0f;
            for (int p = 0; p < parts; ++p) s += ps[(p * TC + tt) * dvt + j];
            a.out[(size_t)(c0 + tt) * a.ldo + h * a.dv + c] = s;
        }
    }
#pragma unroll
    for (int i = 0; i < DKP; ++i) {
        const int kr = part * DKP + i;
        if (col_ok && kr < a.dk) st[(size_t)kr * a.dv + col] = S[i];
    }
    if (tracks && a.dtot) {
        __syncthreads();
        for (int i = tid; i < a.dk; i += nthreads) a.dtot[((size_t)r * a.H + h) * a.dk + i] = carry[i];
    }
}

template <typename T>
static int launch_scan(const ScanArgs& a, int n_reqs, cudaStream_t s) {
    // rows of S a thread keeps: few for small heads, so that the threads of a block stay many
    const int dkp = a.dk <= 64 ? 16 : a.dk <= 256 ? 32 : 64;
    const int parts = (a.dk + dkp - 1) / dkp;
    if (parts > 8) return VCB_ERR_UNSUPPORTED;
    // a narrow tile of value channels when the grid would otherwise leave most SMs without a block
    const long long wide_blocks = (long long)n_reqs * a.H * ((a.dv + 63) / 64);
    const int dvt = (a.dv <= 32 || wide_blocks < 2LL * vcb_sm_count()) ? 32 : 64;
    const int dkpad = parts * dkp;
    int chunk = 16;
    auto bytes = [&](int tc) { return ((size_t)tc * (3 * dkpad + dvt + parts * dvt) + dkpad) * sizeof(float); };
    while (chunk > 1 && bytes(chunk) > 48 * 1024) chunk >>= 1;
    ScanArgs b = a;
    b.chunk = chunk;
    dim3 grid(n_reqs, a.H, (a.dv + dvt - 1) / dvt), block(dvt, parts);
    if (dkp == 16) vcb_launch(decayed_state_scan_kernel<T, 16>, grid, block, bytes(chunk), s, b);
    else if (dkp == 32) vcb_launch(decayed_state_scan_kernel<T, 32>, grid, block, bytes(chunk), s, b);
    else vcb_launch(decayed_state_scan_kernel<T, 64>, grid, block, bytes(chunk), s, b);
    return vcb_last_error();
}

VCB_EXPORT int vcb_decayed_state_scan(const void* q, const void* k, const void* v, const void* decay_pre,
                                      long long ldq, long long ldk, long long ldv, long long ldd,
                                      const float* decay_bias, const float* decay_const, float inv_tau, float q_scale,
                                      int act, float* state, float* out, long long ldo, const int* q_start,
                                      const int* state_slots, int n_reqs, int H, int dk, int dv, int fresh, float* qp,
                                      long long ldqp, float* dtot, int dtype, void* stream) {
    if (n_reqs <= 0) return 0;
    if (!q || !k || !v || !state || !out || H <= 0 || dk <= 0 || dv <= 0 || H > 65535) return VCB_ERR_BAD_ARG;
    if ((dv + 31) / 32 > 65535) return VCB_ERR_UNSUPPORTED;
    ScanArgs a{q, k, v, decay_pre, ldq, ldk, ldv, ldd, decay_bias, decay_const, inv_tau, q_scale, act, state, out, ldo,
               q_start, state_slots, H, dk, dv, 0, fresh, qp, ldqp, dtot};
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32) return launch_scan<float>(a, n_reqs, s);
    if (dtype == VCB_BF16) return launch_scan<__nv_bfloat16>(a, n_reqs, s);
    return VCB_ERR_BAD_ARG;
}

// ------------------------------------------------------------- long portions: pieces side by side
// A long portion is cut into pieces.  decayed_state_scan_kernel runs every piece as if it were a request that starts from
// a zero state: its outputs are then right but for what the state before the piece adds, and its end state is the
// piece's own contribution.  With P_t the product of the decays from the piece's first token through t:
//     S_before(next piece) = diag(P_last) S_before(piece) + S_end(piece)            (decayed_state_carry_kernel)
//     o_t += (q_t * P_t)^T S_before(piece)                                          (decayed_state_inter_kernel)
// Every factor is a product of decays (at most 1): nothing is ever divided by a decay.
//
// One thread per element of S: walks the pieces of its request in order, leaves in piece_state the state before each
// piece and in the request's slot the state after the last.
__global__ void decayed_state_carry_kernel(float* __restrict__ piece_state, const float* __restrict__ dtot, float* __restrict__ state,
                                           const int* __restrict__ req_pieces, const int* __restrict__ state_slots, int H, int dk, int dv) {
    pdl_start();
    const int r = blockIdx.y;
    const size_t per = (size_t)H * dk * dv;
    const int p0 = req_pieces[r], p1 = req_pieces[r + 1];
    float* slot = state + (size_t)state_slots[r] * per;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < per; e += (size_t)gridDim.x * blockDim.x) {
        const size_t hi = e / dv;                     // (head, key channel)
        float S = slot[e];
        for (int p = p0; p < p1; ++p) {
            const float own = piece_state[(size_t)p * per + e];
            piece_state[(size_t)p * per + e] = S;
            S = fmaf(dtot[(size_t)p * H * dk + hi], S, own);
        }
        slot[e] = S;
    }
}

// Grid (piece, head, tile of 64 value channels), 256 threads: thread (x, y) of 16 x 16 owns columns 4x .. 4x + 3 for
// the piece's tokens 8y .. 8y + 7 (32 sums in registers); key channels pass through shared memory in slabs of 32.
#define INTER_MAX_TOKENS 128
__global__ void __launch_bounds__(256)
decayed_state_inter_kernel(const float* __restrict__ qp, long long ldqp, const float* __restrict__ piece_state, float* __restrict__ out,
                           long long ldo, const int* __restrict__ piece_start, int H, int dk, int dv) {
    __shared__ float qs[INTER_MAX_TOKENS][33];
    __shared__ __align__(16) float ss[32][64];
    pdl_start();
    const int p = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int col0 = blockIdx.z * 64;
    const int row0 = piece_start[p], rows = min(piece_start[p + 1] - row0, INTER_MAX_TOKENS);
    const float* S = piece_state + (((size_t)p * H + h) * dk) * dv;
    float acc[8][4];
#pragma unroll
    for (int t = 0; t < 8; ++t)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[t][c] = 0.0f;
    for (int i0 = 0; i0 < dk; i0 += 32) {
        __syncthreads();
        for (int idx = tid; idx < INTER_MAX_TOKENS * 32; idx += 256) {
            const int t = idx >> 5, i = idx & 31;
            qs[t][i] = (t < rows && i0 + i < dk) ? qp[(size_t)(row0 + t) * ldqp + h * dk + i0 + i] : 0.0f;
        }
        for (int idx = tid; idx < 32 * 64; idx += 256) {
            const int i = idx >> 6, c = col0 + (idx & 63);
            ss[i][idx & 63] = (i0 + i < dk && c < dv) ? S[(size_t)(i0 + i) * dv + c] : 0.0f;
        }
        __syncthreads();
        if (ty * 8 < rows) {
#pragma unroll 8
            for (int i = 0; i < 32; ++i) {
                const float4 sv = *reinterpret_cast<const float4*>(&ss[i][tx * 4]);
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    const float qv = qs[ty * 8 + t][i];
                    acc[t][0] = fmaf(qv, sv.x, acc[t][0]);
                    acc[t][1] = fmaf(qv, sv.y, acc[t][1]);
                    acc[t][2] = fmaf(qv, sv.z, acc[t][2]);
                    acc[t][3] = fmaf(qv, sv.w, acc[t][3]);
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        const int tok = ty * 8 + t;
        if (tok >= rows) continue;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int col = col0 + tx * 4 + c;
            if (col < dv) out[(size_t)(row0 + tok) * ldo + h * dv + col] += acc[t][c];
        }
    }
}

// piece_state: [pieces, H, dk, dv] as decayed_state_scan left it (fresh, slots 0 .. pieces - 1); req_pieces [n_reqs + 1]:
// the pieces of request r are req_pieces[r] .. req_pieces[r + 1] - 1; piece_start [pieces + 1]: their first rows.  No piece
// is longer than 128 tokens.
VCB_EXPORT int vcb_decayed_state_join(const float* qp, long long ldqp, float* piece_state, const float* dtot, float* state,
                                      float* out, long long ldo, const int* piece_start, const int* req_pieces,
                                      const int* state_slots, int n_pieces, int n_reqs, int H, int dk, int dv, void* stream) {
    if (n_pieces <= 0 || n_reqs <= 0) return 0;
    if (!qp || !piece_state || !dtot || !state || !out || H <= 0 || dk <= 0 || dv <= 0 || H > 65535 || n_reqs > 65535) return VCB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t per = (size_t)H * dk * dv;
    const int blocks = (int)((per + 255) / 256 < 1024 ? (per + 255) / 256 : 1024);
    vcb_launch(decayed_state_carry_kernel, dim3(blocks, n_reqs), 256, 0, s, piece_state, dtot, state, req_pieces, state_slots, H, dk, dv);
    vcb_launch(decayed_state_inter_kernel, dim3(n_pieces, H, (dv + 63) / 64), 256, 0, s, qp, ldqp, (const float*)piece_state, out, ldo,
               piece_start, H, dk, dv);
    return vcb_last_error();
}

// ------------------------------------------------------------- norm over groups of channels, times a gate
// One CTA per token.  o: float [n, C]; groups of `group` consecutive channels are normed apart,
// out = o / sqrt(mean_group(o^2) + eps) * w[channel % wlen] * act(gate), act 0: sigmoid, 1: silu.
// One group (group == C): the CTA reduces together; several: a warp per group.
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ o, long long ldo, const T* __restrict__ gate, long long ldg,
                                        const float* __restrict__ w, int wlen, T* __restrict__ out, long long ldout,
                                        int C, int group, int act, float eps) {
    __shared__ float scratch[33];
    pdl_start();
    const float* orow = o + (size_t)blockIdx.x * ldo;
    const T* grow = gate ? gate + (size_t)blockIdx.x * ldg : nullptr;
    T* dst = out + (size_t)blockIdx.x * ldout;
    if (group >= C) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < C; i += blockDim.x) ss += orow[i] * orow[i];
        ss = block_sum(ss, scratch);
        const float r = 1.0f / sqrtf(ss / (float)C + eps);
        for (int i = threadIdx.x; i < C; i += blockDim.x) {
            float y = orow[i] * r * w[i % wlen];
            if (grow) { const float g = to_f32<T>(grow[i]); y *= act ? silu_f(g) : sigmoid_f(g); }
            dst[i] = from_f32<T>(y);
        }
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int g0 = warp * group; g0 < C; g0 += nwarps * group) {
        const int len = min(group, C - g0);
        float ss = 0.0f;
        for (int i = lane; i < len; i += 32) ss += orow[g0 + i] * orow[g0 + i];
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)len + eps);
        for (int i = lane; i < len; i += 32) {
            float y = orow[g0 + i] * r * w[(g0 + i) % wlen];
            if (grow) { const float g = to_f32<T>(grow[g0 + i]); y *= act ? silu_f(g) : sigmoid_f(g); }
            dst[g0 + i] = from_f32<T>(y);
        }
    }
}

// The same for bfloat16 gates and results with groups, strides and widths that are multiples of 4: four channels a
// thread at a time (16-byte loads of o and the gain, 8-byte loads and stores of the gate and the result).
__global__ void gated_group_norm_bf16x4_kernel(const float* __restrict__ o, long long ldo, const __nv_bfloat16* __restrict__ gate, long long ldg,
                                               const float* __restrict__ w, int wlen, __nv_bfloat16* __restrict__ out, long long ldout,
                                               int C, int group, int act, float eps) {
    __shared__ float scratch[33];
    pdl_start();
    const float* orow = o + (size_t)blockIdx.x * ldo;
    const __nv_bfloat16* grow = gate ? gate + (size_t)blockIdx.x * ldg : nullptr;
    __nv_bfloat16* dst = out + (size_t)blockIdx.x * ldout;
    auto finish = [&](int i, float r, const float4& v) {          // channels i .. i + 3, whose values are v
        const float4 g = *reinterpret_cast<const float4*>(w + i % wlen);
        float y[4] = {v.x * r * g.x, v.y * r * g.y, v.z * r * g.z, v.w * r * g.w};
        if (grow) {
            const uint2 raw = *reinterpret_cast<const uint2*>(grow + i);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float2 a0 = __bfloat1622float2(p[0]), a1 = __bfloat1622float2(p[1]);
            const float gs[4] = {a0.x, a0.y, a1.x, a1.y};
#pragma unroll
            for (int e = 0; e < 4; ++e) y[e] *= act ? silu_f(gs[e]) : sigmoid_f(gs[e]);
        }
        uint2 packed;
        __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&packed);
        q[0] = __floats2bfloat162_rn(y[0], y[1]);
        q[1] = __floats2bfloat162_rn(y[2], y[3]);
        *reinterpret_cast<uint2*>(dst + i) = packed;
    };
    if (group >= C) {
        float ss = 0.0f;
        for (int i = threadIdx.x * 4; i < C; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(orow + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = block_sum(ss, scratch);
        const float r = 1.0f / sqrtf(ss / (float)C + eps);
        for (int i = threadIdx.x * 4; i < C; i += blockDim.x * 4) finish(i, r, *reinterpret_cast<const float4*>(orow + i));
        return;
    }
    // with few tokens a row's groups are dealt to gridDim.y blocks, so that every warp has one round of work
    const int lane = threadIdx.x & 31, nwarps = (blockDim.x >> 5) * gridDim.y, warp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (group <= 128) {
        // a group is at most one vector a lane: read once.  Two groups of a warp are in flight together.
        for (int g0 = warp * group; g0 < C; g0 += 2 * nwarps * group) {
            const int g1 = g0 + nwarps * group;
            const bool in0 = lane * 4 < group, in1 = in0 && g1 < C;
            const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const float4 v0 = in0 ? *reinterpret_cast<const float4*>(orow + g0 + lane * 4) : zero;
            const float4 v1 = in1 ? *reinterpret_cast<const float4*>(orow + g1 + lane * 4) : zero;
            const float s0 = warp_sum(v0.x * v0.x + v0.y * v0.y + v0.z * v0.z + v0.w * v0.w);
            const float s1 = warp_sum(v1.x * v1.x + v1.y * v1.y + v1.z * v1.z + v1.w * v1.w);
            if (in0) finish(g0 + lane * 4, 1.0f / sqrtf(s0 / (float)group + eps), v0);
            if (in1) finish(g1 + lane * 4, 1.0f / sqrtf(s1 / (float)group + eps), v1);
        }
        return;
    }
    for (int g0 = warp * group; g0 < C; g0 += nwarps * group) {
        float ss = 0.0f;
        for (int i = lane * 4; i < group; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(orow + g0 + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)group + eps);
        for (int i = lane * 4; i < group; i += 128) finish(g0 + i, r, *reinterpret_cast<const float4*>(orow + g0 + i));
    }
}

VCB_EXPORT int vcb_gated_group_norm(const float* o, long long ldo, const void* gate, long long ldg, const float* w, int wlen,
                                    void* out, long long ldout, int n_tokens, int C, int group, int act, float eps,
                                    int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (!o || !w || !out || C <= 0 || group <= 0 || wlen <= 0) return VCB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = C >= 2048 ? 512 : C >= 512 ? 256 : 128;
    const uintptr_t addrs = (uintptr_t)o | (uintptr_t)w;
    if (dtype == VCB_BF16 && !((C | group | wlen) & 3) && C % group == 0 && !((ldo | ldg | ldout) & 3) && !(addrs & 15) &&
        !(((uintptr_t)gate | (uintptr_t)out) & 7)) {
        const int groups = group >= C ? 1 : C / group;
        const int th = group >= C ? (C >= 4096 ? 512 : C >= 1024 ? 256 : 128) : (groups >= 8 ? 256 : 128);
        int split = 1;
        if (groups > 1 && n_tokens <= 256) {
            split = (groups + 2 * (th / 32) - 1) / (2 * (th / 32));
            if (split > 8) split = 8;
        }
        vcb_launch(gated_group_norm_bf16x4_kernel, dim3(n_tokens, split), th, 0, s, o, ldo, (const __nv_bfloat16*)gate, ldg, w, wlen, (__nv_bfloat16*)out,
                   ldout, C, group, act, eps);
        return vcb_last_error();
    }
    if (dtype == VCB_F32)
        vcb_launch(gated_group_norm_kernel<float>, n_tokens, threads, 0, s, o, ldo, (const float*)gate, ldg, w, wlen, (float*)out,
                   ldout, C, group, act, eps);
    else if (dtype == VCB_BF16)
        vcb_launch(gated_group_norm_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, o, ldo, (const __nv_bfloat16*)gate, ldg, w, wlen,
                   (__nv_bfloat16*)out, ldout, C, group, act, eps);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------------------------- two mixers side by side
// out = a * x + b * y, in float, rounded once.
template <typename T>
__global__ void scaled_sum_kernel(const T* __restrict__ x, const T* __restrict__ y, T* __restrict__ out, long long n, float a, float b) {
    pdl_start();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(a * to_f32<T>(x[i]) + b * to_f32<T>(y[i]));
}

VCB_EXPORT int vcb_scaled_sum(const void* x, const void* y, void* out, long long n, float a, float b, int dtype, void* stream) {
    if (n <= 0) return 0;
    const long long want = (n + 255) / 256, cap = (long long)vcb_sm_count() * 16;
    const int blocks = (int)(want < cap ? want : cap);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32) vcb_launch(scaled_sum_kernel<float>, blocks, 256, 0, s, (const float*)x, (const float*)y, (float*)out, n, a, b);
    else if (dtype == VCB_BF16)
        vcb_launch(scaled_sum_kernel<__nv_bfloat16>, blocks, 256, 0, s, (const __nv_bfloat16*)x, (const __nv_bfloat16*)y,
                   (__nv_bfloat16*)out, n, a, b);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}
