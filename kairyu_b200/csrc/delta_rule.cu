// The gated delta rule: a linear-attention mixer whose memory is one matrix S [D, V] per head and
// request, kept in 32-bit and rewritten by every token:
//
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
//
// q, k (KH heads of D) and v (H heads of V) come from a packed projection through a short causal
// convolution over time per channel and silu; q and k are made unit vectors per head (q also times
// D^-1/2); beta = sigmoid(b), g = exp(-exp(A_log) * softplus(a + dt_bias)) per head.  Head h uses
// q/k head h / (H / KH).  The output is o / rms(o) * w * silu(gate) per head.
//
// With a decay a head AND key channel (g a row of D numbers, from a projection of its own) g scales the rows of S.
// The gate of the output is silu or sigmoid of columns of the packed projection or of a tensor of its own.
//
// Kernels:
//   delta_prepare     per token and head (a warp each): convolution (reaching into the request's kept
//                     inputs for the taps that lie before the step's first token), silu, unit norms;
//                     beta and g per token (g a head, or a head and key channel); all results 32-bit
//   conv_state        (linear_recurrence.cuh) per request: the last (taps - 1) inputs of the step become the kept inputs
//   the recurrence    linear_recurrence.cuh, with the delta and either kind of decay: per (request, head, 16 columns
//                     of S) it walks the request's tokens in order
//   delta_gated_norm  per token and head: o / sqrt(mean(o^2) + eps) * w * act(gate)
//
// Every sum runs in an order that depends on the sizes alone, never on the batch or on how a
// prompt was cut.
#include "common.cuh"
#include "linear_recurrence.cuh"

#define DELTA_MAX_TAPS LR_MAX_TAPS

// NT: the number of taps where it is one of the usual few (the taps' loop unrolls, the rows of the last
// tokens are looked up once a token, a channel's taps come in one load); 0: any number, taken at run time.
template <typename TA, int NT>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const TA* __restrict__ proj, int stride, const float* __restrict__ gates, int gate_stride,
                     const float* __restrict__ channel_a, const float* __restrict__ taps,
                     int n, const float* __restrict__ conv_state, const int* __restrict__ row_ids,
                     const int* __restrict__ qo_indptr, const int* __restrict__ state_slots,
                     const float* __restrict__ A_log, const float* __restrict__ dt_bias, int KH, int D, int H, int V,
                     float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vv, float* __restrict__ beta,
                     float* __restrict__ decay, int num_rows, int* flag) {
    const int t = blockIdx.x;
    const int row = row_ids[t];
    pdl_wait();
    if (row < 0 || row >= num_rows) {
        if (threadIdx.x == 0 && flag) atomicOr(flag, KB_FLAG_BAD_ROW);
        return;
    }
    const int o = t - qo_indptr[row];
    const int C = 2 * KH * D + H * V;
    const float* kept = conv_state + (size_t)state_slots[row] * (n - 1) * C;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    // where the inputs `back` tokens before this one lie: in the step's rows, or among the request's kept inputs
    constexpr int ROWS = NT ? NT : 1;
    const TA* step_row[ROWS];
    const float* kept_row[ROWS];
#pragma unroll
    for (int back = 0; back < ROWS; ++back) {
        step_row[back] = o - back >= 0 ? proj + (size_t)(t - back) * stride : nullptr;
        kept_row[back] = o - back >= 0 ? nullptr : kept + (size_t)((n - 1) + (o - back)) * C;
    }
    auto convolve = [&](int c) -> float {
        float z = 0.0f;
        if constexpr (NT == 0) {
            for (int back = 0; back < n; ++back) z += taps[(size_t)c * n + (n - 1 - back)] * conv_input(proj, stride, kept, C, n, t, o, back, c);
        } else {
            float w[NT];
            if constexpr (NT == 4) {
                const float4 all = *reinterpret_cast<const float4*>(taps + (size_t)c * 4);
                w[0] = all.x; w[1] = all.y; w[2] = all.z; w[3] = all.w;
            } else {
#pragma unroll
                for (int j = 0; j < NT; ++j) w[j] = taps[(size_t)c * NT + j];
            }
#pragma unroll
            for (int back = 0; back < NT; ++back) {
                const float x = step_row[back] ? to_float(step_row[back][c]) : kept_row[back][c];
                z = fmaf(w[NT - 1 - back], x, z);
            }
        }
        return z;
    };
    // A warp takes one head: of q, of k (with the unit norm) or of v; blockIdx.y spreads a token's heads over
    // blocks, so that a step of few tokens still fills the device and no thread walks many channels in turn.
    const int unit = blockIdx.y * warps + warp;
    if (unit < 2 * KH) {
        float vals[16];
        float ss = 0.0f;
#pragma unroll
        for (int m = 0; m < 16; ++m) {
            const int e = lane + 32 * m;
            float z = 0.0f;
            if (e < D) z = silu_f(convolve(unit * D + e));
            vals[m] = z;
            ss += z * z;
        }
        ss = warp_sum(ss);
        float scale = rsqrtf(ss + 1e-6f);
        float* dst;
        if (unit < KH) {
            scale *= rsqrtf((float)D);
            dst = qn + ((size_t)t * KH + unit) * D;
        } else {
            dst = kn + ((size_t)t * KH + (unit - KH)) * D;
        }
#pragma unroll
        for (int m = 0; m < 16; ++m) {
            const int e = lane + 32 * m;
            if (e < D) dst[e] = vals[m] * scale;
        }
    } else if (unit < 2 * KH + H) {
        const int first = (unit - 2 * KH) * V;
        for (int e = lane; e < V; e += 32) vv[(size_t)t * H * V + first + e] = silu_f(convolve(2 * KH * D + first + e));
    }
    if (channel_a) {
        // one decay a head and key channel: a comes as [tokens, H * D], dt_bias has H * D entries; beta alone in `gates`
        for (int h = threadIdx.x; blockIdx.y == 0 && h < H; h += blockDim.x)
            beta[(size_t)t * H + h] = 1.0f / (1.0f + expf(-gates[(size_t)t * gate_stride + h]));
        for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H * D; i += gridDim.y * blockDim.x) {
            const float a = channel_a[(size_t)t * H * D + i] + dt_bias[i];
            decay[(size_t)t * H * D + i] = expf(-expf(A_log[i / D]) * softplus_f(a));
        }
        return;
    }
    for (int h = threadIdx.x; blockIdx.y == 0 && h < H; h += blockDim.x) {
        const float b = gates[(size_t)t * gate_stride + h];
        const float a = gates[(size_t)t * gate_stride + H + h] + dt_bias[h];
        beta[(size_t)t * H + h] = 1.0f / (1.0f + expf(-b));
        decay[(size_t)t * H + h] = expf(-expf(A_log[h]) * softplus_f(a));
    }
}

// gate: [tokens, H * V] columns of a row of `gate_stride` entries; sigmoid_gate: sigmoid(gate), else silu(gate)
template <typename TA>
__global__ void __launch_bounds__(128)
delta_gated_norm_kernel(const float* __restrict__ o, const TA* __restrict__ gate, int gate_stride, int sigmoid_gate,
                        const float* __restrict__ w, float eps, int H, int V, TA* __restrict__ out) {
    // a warp a (token, head); blockIdx.y spreads a token's heads over blocks, so that a step of few tokens still fills the device
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    pdl_wait();
    for (int h = blockIdx.y * warps + warp; h < H; h += gridDim.y * warps) {
        const float* oh = o + ((size_t)t * H + h) * V;
        float ss = 0.0f;
        for (int e = lane; e < V; e += 32) ss += oh[e] * oh[e];
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)V + eps);
        for (int e = lane; e < V; e += 32) {
            const float z = to_float(gate[(size_t)t * gate_stride + h * V + e]);
            const float factor = sigmoid_gate ? 1.0f / (1.0f + expf(-z)) : silu_f(z);
            out[(size_t)t * H * V + h * V + e] = from_float<TA>(oh[e] * inv * w[e] * factor);
        }
    }
}

// channel_a null: `gates` is [tokens, 2H] (beta's logits, then a) and the decay one number a head ([tokens, H]);
// else `gates` is [tokens, H], channel_a [tokens, H * D], dt_bias [H * D] and the decay [tokens, H, D].
KB_EXPORT int kb_delta_prepare(const void* proj, int stride, int is_bf16, const float* gates, const float* channel_a, const float* taps, int n,
                               float* conv_state, const int* row_ids, const int* qo_indptr, const int* state_slots,
                               const float* A_log, const float* dt_bias, int KH, int D, int H, int V, float* qn, float* kn,
                               float* vv, float* beta, float* decay, int num_rows, int T, int* flag, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!proj || !gates || !taps || !row_ids || !qo_indptr || !state_slots || !A_log || !dt_bias || !qn || !kn || !vv || !beta || !decay)
        return KB_ERR_NULL;
    if (n < 1 || n > DELTA_MAX_TAPS + 1 || D < 1 || D > 512 || KH < 1 || H % KH != 0 || V < 1) return KB_ERR_UNSUPPORTED_SIZE;
    if (n > 1 && !conv_state) return KB_ERR_NULL;
    const int C = 2 * KH * D + H * V;
    const int gate_stride = channel_a ? H : 2 * H;
#define LAUNCH(TA, NT)                                                                                                        \
    kb_launch(delta_prepare_kernel<TA, NT>, dim3(T, (2 * KH + H + 3) / 4), dim3(128), 0, stream, (const TA*)proj, stride, gates, gate_stride, channel_a, taps, n, \
              (const float*)conv_state, row_ids, qo_indptr, state_slots, A_log, dt_bias, KH, D, H, V, qn, kn, vv, beta, decay, num_rows, flag)
#define PICK(TA)                                                                                                              \
    do {                                                                                                                      \
        if (n == 1) LAUNCH(TA, 1); else if (n == 2) LAUNCH(TA, 2); else if (n == 3) LAUNCH(TA, 3); else if (n == 4) LAUNCH(TA, 4); \
        else LAUNCH(TA, 0);                                                                                                   \
    } while (0)
    if (is_bf16) PICK(__nv_bfloat16); else PICK(float);
#undef PICK
#undef LAUNCH
    int code = kb_launch_result();
    if (code != 0 || n == 1) return code;
    return launch_conv_state(proj, stride, is_bf16, conv_state, n, C, qo_indptr, state_slots, num_rows, stream);
}

// channel_decay: decay is [tokens, H, D], else [tokens, H]
KB_EXPORT int kb_delta_recurrence(const float* qn, const float* kn, const float* vv, const float* beta, const float* decay,
                                  float* states, const int* qo_indptr, const int* state_slots, int KH, int D, int H, int V,
                                  float* out, int num_rows, int single_tokens, int channel_decay, cudaStream_t stream) {
    if (channel_decay)
        return launch_linear_recurrence<true, true>(qn, kn, vv, beta, decay, states, qo_indptr, state_slots, KH, D, H, V, out, num_rows, single_tokens, stream);
    return launch_linear_recurrence<true, false>(qn, kn, vv, beta, decay, states, qo_indptr, state_slots, KH, D, H, V, out, num_rows, single_tokens, stream);
}

KB_EXPORT int kb_delta_gated_norm(const float* o, const void* gate, int gate_stride, int sigmoid_gate, int is_bf16, const float* w,
                                  float eps, int H, int V, void* out, int T, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!o || !gate || !w || !out) return KB_ERR_NULL;
    if (H < 1 || H > 4 * 65535) return KB_ERR_UNSUPPORTED_SIZE;
    if (is_bf16)
        kb_launch(delta_gated_norm_kernel<__nv_bfloat16>, dim3(T, (H + 3) / 4), dim3(128), 0, stream, o, (const __nv_bfloat16*)gate, gate_stride, sigmoid_gate, w, eps, H, V, (__nv_bfloat16*)out);
    else
        kb_launch(delta_gated_norm_kernel<float>, dim3(T, (H + 3) / 4), dim3(128), 0, stream, o, (const float*)gate, gate_stride, sigmoid_gate, w, eps, H, V, (float*)out);
    return kb_launch_result();
}
