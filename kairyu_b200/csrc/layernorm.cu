// Layer norm with weight and bias over the fp32 residual, with the residual sum fused in.
//
// One block per output row r; source row s = rows ? rows[r] : r.
//   v = x[s] (+ d1[s]) (+ d2[s])          two pending sums: a layer whose sub-layers run side by side
//                                          leaves the mixer's and the feed-forward's output, and both
//                                          are added here, in 32-bit, in that order
//   if write_back: x[s] = v
//   out[r] = (v - mean(v)) * rsqrt(mean((v - mean(v))^2) + eps) * w + b
// Statistics are 32-bit and two-pass (the variance is the mean of the squared deviations); the
// order of every sum depends on H alone.
#include "common.cuh"

#define LN_THREADS 256
#define LN_CHUNKS 8  // float4 chunks a thread keeps: rows up to 4 * 8 * 256 = 8,192 wide stay in registers

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = raw;
}

// H % 4 == 0, H <= 4 * LN_CHUNKS * LN_THREADS, 16-byte aligned rows: the row is read once.
template <typename TA, typename TW>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_vec_kernel(float* __restrict__ x, const TA* __restrict__ d1, const TA* __restrict__ d2, const TW* __restrict__ w,
                     const TW* __restrict__ b, TA* __restrict__ out, const int* __restrict__ rows, int H, float eps,
                     int write_back) {
    __shared__ float scratch[32];
    pdl_trigger();
    const int r = blockIdx.x;
    const int chunks = H >> 2;
    pdl_wait();
    const int s = rows ? rows[r] : r;
    float* xr = x + (size_t)s * H;
    float4 v[LN_CHUNKS];
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < LN_CHUNKS; ++c) {
        const int i = c * LN_THREADS + threadIdx.x;
        v[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < chunks) {
            v[c] = load4(xr + 4 * i);
            if (d1) {
                const float4 a = load4(d1 + (size_t)s * H + 4 * i);
                v[c].x += a.x; v[c].y += a.y; v[c].z += a.z; v[c].w += a.w;
            }
            if (d2) {
                const float4 a = load4(d2 + (size_t)s * H + 4 * i);
                v[c].x += a.x; v[c].y += a.y; v[c].z += a.z; v[c].w += a.w;
            }
            if (write_back && (d1 || d2)) store4(xr + 4 * i, v[c]);
            sum += (v[c].x + v[c].y) + (v[c].z + v[c].w);
        }
    }
    const float mean = block_sum(sum, scratch) / (float)H;
    float squares = 0.0f;
#pragma unroll
    for (int c = 0; c < LN_CHUNKS; ++c) {
        const int i = c * LN_THREADS + threadIdx.x;
        if (i < chunks) {
            v[c].x -= mean; v[c].y -= mean; v[c].z -= mean; v[c].w -= mean;
            squares += (v[c].x * v[c].x + v[c].y * v[c].y) + (v[c].z * v[c].z + v[c].w * v[c].w);
        }
    }
    const float inv = rsqrtf(block_sum(squares, scratch) / (float)H + eps);
    TA* orow = out + (size_t)r * H;
#pragma unroll
    for (int c = 0; c < LN_CHUNKS; ++c) {
        const int i = c * LN_THREADS + threadIdx.x;
        if (i < chunks) {
            const float4 g = load4(w + 4 * i), o = load4(b + 4 * i);
            store4(orow + 4 * i, make_float4(v[c].x * inv * g.x + o.x, v[c].y * inv * g.y + o.y, v[c].z * inv * g.z + o.z,
                                             v[c].w * inv * g.w + o.w));
        }
    }
}

// Any H: the row is formed three times from its addends (the same sum each time).
template <typename TA, typename TW>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_kernel(float* __restrict__ x, const TA* __restrict__ d1, const TA* __restrict__ d2, const TW* __restrict__ w,
                 const TW* __restrict__ b, TA* __restrict__ out, const int* __restrict__ rows, int H, float eps, int write_back) {
    __shared__ float scratch[32];
    pdl_wait();
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* xr = x + (size_t)s * H;
    const TA* ar = d1 ? d1 + (size_t)s * H : nullptr;
    const TA* br = d2 ? d2 + (size_t)s * H : nullptr;
    auto value = [&](int i) {
        float v = xr[i];
        if (ar) v += to_float(ar[i]);
        if (br) v += to_float(br[i]);
        return v;
    };
    float sum = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) sum += value(i);
    const float mean = block_sum(sum, scratch) / (float)H;
    float squares = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = value(i) - mean;
        squares += d * d;
    }
    const float inv = rsqrtf(block_sum(squares, scratch) / (float)H + eps);
    TA* orow = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = value(i);
        orow[i] = from_float<TA>((v - mean) * inv * to_float(w[i]) + to_float(b[i]));
        if (write_back && (ar || br)) xr[i] = v;  // element i is read by this thread alone
    }
}

template <typename TA, typename TW>
static int layernorm_launch(float* x, const void* d1, const void* d2, const void* w, const void* b, void* out, const int* rows, int R,
                            int H, float eps, int write_back, cudaStream_t stream) {
    auto aligned = [](const void* p) { return p == nullptr || (uintptr_t)p % 16 == 0; };
    const bool vec = H % 4 == 0 && H <= 4 * LN_CHUNKS * LN_THREADS && aligned(x) && aligned(d1) && aligned(d2) && aligned(w) &&
                     aligned(b) && aligned(out) && (H * sizeof(TA)) % 16 == 0 && (H * sizeof(TW)) % 8 == 0;
    if (vec)
        kb_launch(layernorm_vec_kernel<TA, TW>, dim3(R), dim3(LN_THREADS), 0, stream, x, (const TA*)d1, (const TA*)d2, (const TW*)w,
                  (const TW*)b, (TA*)out, rows, H, eps, write_back);
    else
        kb_launch(layernorm_kernel<TA, TW>, dim3(R), dim3(LN_THREADS), 0, stream, x, (const TA*)d1, (const TA*)d2, (const TW*)w,
                  (const TW*)b, (TA*)out, rows, H, eps, write_back);
    return kb_launch_result();
}

// x: [*, H] fp32; d1, d2, out: the activation dtype; w and b: one dtype, fp32 or bf16.
KB_EXPORT int kb_layernorm(float* x, const void* d1, const void* d2, const void* w, const void* b, int w_bf16, void* out, int act_bf16,
                           const int* rows, int R, int H, float eps, cudaStream_t stream) {
    if (R == 0) return 0;
    if (!x || !w || !b || !out) return KB_ERR_NULL;
    if (H < 1) return KB_ERR_BAD_ARG;
    const int write_back = rows ? 0 : 1;
    if (act_bf16) {
        if (w_bf16) return layernorm_launch<__nv_bfloat16, __nv_bfloat16>(x, d1, d2, w, b, out, rows, R, H, eps, write_back, stream);
        return layernorm_launch<__nv_bfloat16, float>(x, d1, d2, w, b, out, rows, R, H, eps, write_back, stream);
    }
    if (w_bf16) return layernorm_launch<float, __nv_bfloat16>(x, d1, d2, w, b, out, rows, R, H, eps, write_back, stream);
    return layernorm_launch<float, float>(x, d1, d2, w, b, out, rows, R, H, eps, write_back, stream);
}
