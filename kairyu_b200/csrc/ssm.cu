// A selective state-space mixer in its state-space-duality form: per head and request a state S [N, V]
// (N state channels, V columns of the head), kept in 32-bit and rewritten by every token:
//
//     S <- exp(-exp(A_log) dt) S + dt B x^T,     y = S^T C + D x
//
// x (H heads of V), B and C (G groups of N; head h uses group h / (H / G)) come from a packed projection
// through a short causal convolution over time per channel (with a bias) and silu; dt = softplus(raw + dt_bias),
// one number a head.  The result is multiplied by silu(z), then normed in `norm_groups` equal parts (each by
// its own root mean square), times a weight a column.
//
// Kernels:
//   ssm_prepare      per token: convolution (reaching into the request's kept inputs for the taps that lie
//                    before the step's first token), bias, silu -> x, B, C in 32-bit; dt and the decay a head
//   conv_state       (linear_recurrence.cuh) the step's last inputs become the kept ones
//   the recurrence   linear_recurrence.cuh with k = B, q = C, v = x, beta = dt, one decay a head and no delta
//   ssm_gated_norm   per token: (y + D x) silu(z), the grouped norm, the weight; one rounding at the store
//
// Every sum runs in an order that depends on the sizes alone.
#include "common.cuh"
#include "linear_recurrence.cuh"

template <typename TA>
__global__ void __launch_bounds__(128)
ssm_prepare_kernel(const TA* __restrict__ proj, int stride, const float* __restrict__ dt_raw, const float* __restrict__ taps,
                   const float* __restrict__ conv_bias, int n, const float* __restrict__ conv_state, const int* __restrict__ row_ids,
                   const int* __restrict__ qo_indptr, const int* __restrict__ state_slots, const float* __restrict__ A_log,
                   const float* __restrict__ dt_bias, int G, int N, int H, int V, float* __restrict__ xo, float* __restrict__ Bo,
                   float* __restrict__ Co, float* __restrict__ dt, float* __restrict__ decay, int num_rows, int* flag) {
    const int t = blockIdx.x;
    const int row = row_ids[t];
    pdl_wait();
    if (row < 0 || row >= num_rows) {
        if (threadIdx.x == 0 && blockIdx.y == 0 && flag) atomicOr(flag, KB_FLAG_BAD_ROW);
        return;
    }
    const int o = t - qo_indptr[row];
    const int inner = H * V, GN = G * N;
    const int C = inner + 2 * GN;
    const float* kept = n > 1 ? conv_state + (size_t)state_slots[row] * (n - 1) * C : nullptr;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float z = conv_bias ? conv_bias[c] : 0.0f;
        for (int back = n - 1; back >= 0; --back)  // oldest input first: the order of the taps
            z = fmaf(taps[(size_t)c * n + (n - 1 - back)], conv_input(proj, stride, kept, C, n, t, o, back, c), z);
        z = silu_f(z);
        if (c < inner) xo[(size_t)t * inner + c] = z;
        else if (c < inner + GN) Bo[(size_t)t * GN + (c - inner)] = z;
        else Co[(size_t)t * GN + (c - inner - GN)] = z;
    }
    for (int h = threadIdx.x; blockIdx.y == 0 && h < H; h += blockDim.x) {
        const float step = softplus_f(dt_raw[(size_t)t * H + h] + dt_bias[h]);
        dt[(size_t)t * H + h] = step;
        decay[(size_t)t * H + h] = expf(-expf(A_log[h]) * step);
    }
}

// y: [tokens, H * V] fp32 (the recurrence's read-out); x: the same shape (the convolved inputs); z: the gate's
// columns of the packed projection; parts: the norm's equal parts of (H * V) / parts columns
template <typename TA>
__global__ void __launch_bounds__(128)
ssm_gated_norm_kernel(const float* __restrict__ y, const float* __restrict__ x, const float* __restrict__ skip,
                      const TA* __restrict__ z, int z_stride, const float* __restrict__ w, float eps, int H, int V, int parts,
                      TA* __restrict__ out) {
    // one block per (token, part of the norm): the part's columns spread over the block's threads
    __shared__ float scratch[32];
    const int t = blockIdx.x, part = blockIdx.y;
    const int inner = H * V, size = inner / parts;
    pdl_wait();
    auto gated = [&](int e) -> float {
        const float value = y[(size_t)t * inner + e] + skip[e / V] * x[(size_t)t * inner + e];
        return value * silu_f(to_float(z[(size_t)t * z_stride + e]));
    };
    float ss = 0.0f;
    for (int e = threadIdx.x; e < size; e += blockDim.x) {
        const float v = gated(part * size + e);
        ss += v * v;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)size + eps);
    for (int e = threadIdx.x; e < size; e += blockDim.x) {
        const int c = part * size + e;
        out[(size_t)t * inner + c] = from_float<TA>(gated(c) * inv * w[c]);
    }
}

KB_EXPORT int kb_ssm_prepare(const void* proj, int stride, int is_bf16, const float* dt_raw, const float* taps, const float* conv_bias, int n,
                             float* conv_state, const int* row_ids, const int* qo_indptr, const int* state_slots, const float* A_log,
                             const float* dt_bias, int G, int N, int H, int V, float* xo, float* Bo, float* Co, float* dt, float* decay,
                             int num_rows, int T, int* flag, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!proj || !dt_raw || !taps || !row_ids || !qo_indptr || !state_slots || !A_log || !dt_bias || !xo || !Bo || !Co || !dt || !decay)
        return KB_ERR_NULL;
    if (n < 1 || n > LR_MAX_TAPS + 1 || N < 1 || N > 512 || G < 1 || H % G != 0 || V < 1) return KB_ERR_UNSUPPORTED_SIZE;
    if (n > 1 && !conv_state) return KB_ERR_NULL;
    const int C = H * V + 2 * G * N;
    int blocks = (C + 127) / 128;
    if (blocks > 64) blocks = 64;
    if (is_bf16)
        kb_launch(ssm_prepare_kernel<__nv_bfloat16>, dim3(T, blocks), dim3(128), 0, stream, (const __nv_bfloat16*)proj, stride, dt_raw, taps,
                  conv_bias, n, (const float*)conv_state, row_ids, qo_indptr, state_slots, A_log, dt_bias, G, N, H, V, xo, Bo, Co, dt, decay,
                  num_rows, flag);
    else
        kb_launch(ssm_prepare_kernel<float>, dim3(T, blocks), dim3(128), 0, stream, (const float*)proj, stride, dt_raw, taps, conv_bias, n,
                  (const float*)conv_state, row_ids, qo_indptr, state_slots, A_log, dt_bias, G, N, H, V, xo, Bo, Co, dt, decay, num_rows, flag);
    int code = kb_launch_result();
    if (code != 0 || n == 1) return code;
    return launch_conv_state(proj, stride, is_bf16, conv_state, n, C, qo_indptr, state_slots, num_rows, stream);
}

// states: [slots, H, V, N] fp32 (S column by column)
KB_EXPORT int kb_ssm_recurrence(const float* Cq, const float* Bk, const float* x, const float* dt, const float* decay, float* states,
                                const int* qo_indptr, const int* state_slots, int G, int N, int H, int V, float* out, int num_rows,
                                int single_tokens, cudaStream_t stream) {
    return launch_linear_recurrence<false, false>(Cq, Bk, x, dt, decay, states, qo_indptr, state_slots, G, N, H, V, out, num_rows,
                                                  single_tokens, stream);
}

KB_EXPORT int kb_ssm_gated_norm(const float* y, const float* x, const float* skip, const void* z, int z_stride, int is_bf16, const float* w,
                                float eps, int H, int V, int parts, void* out, int T, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!y || !x || !skip || !z || !w || !out) return KB_ERR_NULL;
    if (parts < 1 || parts > 65535 || (H * V) % parts != 0) return KB_ERR_BAD_ARG;
    if (is_bf16)
        kb_launch(ssm_gated_norm_kernel<__nv_bfloat16>, dim3(T, parts), dim3(128), 0, stream, y, x, skip, (const __nv_bfloat16*)z, z_stride, w, eps,
                  H, V, parts, (__nv_bfloat16*)out);
    else
        kb_launch(ssm_gated_norm_kernel<float>, dim3(T, parts), dim3(128), 0, stream, y, x, skip, (const float*)z, z_stride, w, eps, H, V, parts,
                  (float*)out);
    return kb_launch_result();
}
