// A norm on a sub-layer's OUTPUT, with the residual sum behind it:
//
//     y[t]  = sum_k mix[t, k] * parts[at(t * K + k)]      (K = 1 and no mix: y = parts; at: an optional
//                                                          index of where each of the K rows lies)
//     x[t] += y[t] * rsqrt(mean(y[t]^2) + eps) * w         (x: the fp32 residual stream)
//     copy[t] = x[t] in the activation dtype               (what the next sub-layer's products read)
//
// The K-fold sum is how a mixture of experts hands its output over: one row per (token, chosen
// expert) and the router's weights, added here in the order of k, so no kernel of its own
// combines them and the order of the sum never depends on the batch.
// Statistics, the weighted sum and the residual sum are 32-bit.  One block per token; the row
// of y is kept in shared memory between the two passes.
#include "common.cuh"

template <typename TY, typename TW, typename TC>
__global__ void __launch_bounds__(256)
output_norm_add_kernel(float* __restrict__ x, const TY* __restrict__ parts, const float* __restrict__ mix,
                       const int* __restrict__ at, int K, const TW* __restrict__ w, TC* __restrict__ copy, int H, float eps) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_wait();
    const int t = blockIdx.x;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v;
        if (mix) {
            v = 0.0f;
            for (int k = 0; k < K; ++k) {
                const size_t p = (size_t)t * K + k;
                v += mix[p] * to_float(parts[(at ? (size_t)at[p] : p) * H + i]);
            }
        } else {
            v = to_float(parts[(size_t)t * H + i]);
        }
        row[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)H + eps);
    float* xr = x + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = xr[i] + row[i] * inv * to_float(w[i]);
        xr[i] = v;
        if (copy) copy[(size_t)t * H + i] = from_float<TC>(v);
    }
}

template <typename TY, typename TW>
static int launch_output_norm(float* x, const void* parts, const float* mix, const int* at, int K, const void* w, void* copy,
                              int copy_is_bf16, int T, int H, float eps, cudaStream_t stream) {
    const size_t smem = (size_t)H * sizeof(float);
    if (copy_is_bf16)
        kb_launch(output_norm_add_kernel<TY, TW, __nv_bfloat16>, dim3(T), dim3(256), smem, stream, x, (const TY*)parts, mix, at, K,
                  (const TW*)w, (__nv_bfloat16*)copy, H, eps);
    else
        kb_launch(output_norm_add_kernel<TY, TW, float>, dim3(T), dim3(256), smem, stream, x, (const TY*)parts, mix, at, K,
                  (const TW*)w, (float*)copy, H, eps);
    return kb_launch_result();
}

KB_EXPORT int kb_output_norm_add(float* x, const void* parts, int parts_is_bf16, const float* mix, const int* at, int K, const void* w,
                                 int w_is_bf16, void* copy, int copy_is_bf16, int T, int H, float eps, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!x || !parts || !w) return KB_ERR_NULL;
    if (H < 1 || H > 12000 || K < 1) return KB_ERR_UNSUPPORTED_SIZE;  // the row lives in 48 KB of shared memory
    if (parts_is_bf16) {
        if (w_is_bf16) return launch_output_norm<__nv_bfloat16, __nv_bfloat16>(x, parts, mix, at, K, w, copy, copy_is_bf16, T, H, eps, stream);
        return launch_output_norm<__nv_bfloat16, float>(x, parts, mix, at, K, w, copy, copy_is_bf16, T, H, eps, stream);
    }
    if (w_is_bf16) return launch_output_norm<float, __nv_bfloat16>(x, parts, mix, at, K, w, copy, copy_is_bf16, T, H, eps, stream);
    return launch_output_norm<float, float>(x, parts, mix, at, K, w, copy, copy_is_bf16, T, H, eps, stream);
}

// copy[t] = x[t] in bfloat16: the first sub-layer of a model reads the embedding's rows.
__global__ void residual_copy_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ copy, size_t n) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) copy[i] = __float2bfloat16_rn(x[i]);
}

KB_EXPORT int kb_residual_copy(const float* x, void* copy, long long n, cudaStream_t stream) {
    if (n == 0) return 0;
    if (!x || !copy) return KB_ERR_NULL;
    kb_launch(residual_copy_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, (__nv_bfloat16*)copy, (size_t)n);
    return kb_launch_result();
}

// A norm on a sub-layer's output and the norm that reads the stream next, as one kernel:
//
//     x[t] += y[t] * rsqrt(mean(y[t]^2) + eps_y) * wy       (y null: nothing is added)
//     out[r] = x[t] * rsqrt(mean(x[t]^2) + eps_x) * wx      (out null: the sum alone)
//
// for t = rows[r] (rows null: every row, and x is left updated; with rows x is not written: the listed rows'
// results are all that is wanted).  Statistics, both weights and the sum are 32-bit; y and out have the
// activation dtype.  One block per row; the row is kept in shared memory between the passes.
template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
sandwich_norm_kernel(float* __restrict__ x, const TA* __restrict__ y, const TW* __restrict__ wy, float eps_y, const TW* __restrict__ wx,
                     float eps_x, TA* __restrict__ out, const int* __restrict__ rows, int H) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_trigger();
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    pdl_wait();
    float* xr = x + (size_t)t * H;
    float inv_y = 0.0f;
    if (y) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = to_float(y[(size_t)t * H + i]);
            row[i] = v;
            ss += v * v;
        }
        inv_y = rsqrtf(block_sum(ss, scratch) / (float)H + eps_y);
    }
    float sx = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (y) {
            v += row[i] * inv_y * to_float(wy[i]);
            if (!rows) xr[i] = v;
        }
        row[i] = v;
        sx += v * v;
    }
    if (!out) return;
    const float inv_x = rsqrtf(block_sum(sx, scratch) / (float)H + eps_x);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)r * H + i] = from_float<TA>(row[i] * inv_x * to_float(wx[i]));
}

// The same, four columns a thread a turn (16-byte accesses of the 32-bit rows, 8-byte ones of bfloat16 rows), for rows of a
// multiple of four columns with fp32 weights.  A thread owns other columns than in the kernel above, so the sums' order
// differs between the two; which one runs depends on the width and the weights' type alone, never on the batch.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&lo);
    raw.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// two_rows: shared memory holds the stream's row beside the output's, and both are fetched in the first pass, so that the
// stream's row is not waited for behind the first reduction (a step of few rows is the latency of these passes).
template <typename TA>
__global__ void __launch_bounds__(256)
sandwich_norm_vec_kernel(float* __restrict__ x, const TA* __restrict__ y, const float* __restrict__ wy, float eps_y,
                         const float* __restrict__ wx, float eps_x, TA* __restrict__ out, const int* __restrict__ rows, int H,
                         int two_rows) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    pdl_trigger();
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    pdl_wait();
    float* xr = x + (size_t)t * H;
    float* kept = row + H;  // two_rows: the stream's row
    float inv_y = 0.0f;
    if (y) {
        float ss = 0.0f;
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 v = load4(y + (size_t)t * H + i);
            if (two_rows) store4(kept + i, load4(xr + i));
            store4(row + i, v);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        inv_y = rsqrtf(block_sum(ss, scratch) / (float)H + eps_y);
    }
    float sx = 0.0f;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
        float4 v = (y && two_rows) ? load4(kept + i) : load4(xr + i);
        if (y) {
            const float4 p = load4(row + i), w = load4(wy + i);
            v.x += p.x * inv_y * w.x; v.y += p.y * inv_y * w.y; v.z += p.z * inv_y * w.z; v.w += p.w * inv_y * w.w;
            if (!rows) store4(xr + i, v);
        }
        store4(row + i, v);
        sx += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    if (!out) return;
    const float inv_x = rsqrtf(block_sum(sx, scratch) / (float)H + eps_x);
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
        const float4 v = load4(row + i), w = load4(wx + i);
        store4(out + (size_t)r * H + i, make_float4(v.x * inv_x * w.x, v.y * inv_x * w.y, v.z * inv_x * w.z, v.w * inv_x * w.w));
    }
}

KB_EXPORT int kb_sandwich_norm(float* x, const void* y, const void* wy, float eps_y, const void* wx, float eps_x, void* out, int act_bf16,
                               int w_bf16, const int* rows, int R, int H, cudaStream_t stream) {
    if (R == 0) return 0;
    if (!x || (y && !wy) || (out && !wx) || (!y && !out)) return KB_ERR_NULL;
    if (H < 1 || H > 12000) return KB_ERR_UNSUPPORTED_SIZE;  // the row lives in 48 KB of shared memory
    const size_t smem = (size_t)H * sizeof(float);
    const bool aligned = ((uintptr_t)x | (uintptr_t)y | (uintptr_t)wy | (uintptr_t)wx | (uintptr_t)out) % 16 == 0;
    if (H % 4 == 0 && !w_bf16 && aligned) {
        const int two_rows = y && 2 * smem <= 48 * 1024;  // both rows fit the shared memory a block gets without asking
        const size_t held = two_rows ? 2 * smem : smem;
        if (act_bf16)
            kb_launch(sandwich_norm_vec_kernel<__nv_bfloat16>, dim3(R), dim3(256), held, stream, x, (const __nv_bfloat16*)y, (const float*)wy, eps_y,
                      (const float*)wx, eps_x, (__nv_bfloat16*)out, rows, H, two_rows);
        else
            kb_launch(sandwich_norm_vec_kernel<float>, dim3(R), dim3(256), held, stream, x, (const float*)y, (const float*)wy, eps_y, (const float*)wx,
                      eps_x, (float*)out, rows, H, two_rows);
        return kb_launch_result();
    }
#define LAUNCH(TA, TW)                                                                                                                  \
    kb_launch(sandwich_norm_kernel<TA, TW>, dim3(R), dim3(256), smem, stream, x, (const TA*)y, (const TW*)wy, eps_y, (const TW*)wx, eps_x, \
              (TA*)out, rows, H)
    if (act_bf16) {
        if (w_bf16) LAUNCH(__nv_bfloat16, __nv_bfloat16); else LAUNCH(__nv_bfloat16, float);
    } else {
        if (w_bf16) LAUNCH(float, __nv_bfloat16); else LAUNCH(float, float);
    }
#undef LAUNCH
    return kb_launch_result();
}
