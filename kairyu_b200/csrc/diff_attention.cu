// Paged attention whose heads take MAPS softmax maps over the same values and combine them
// ("differential attention": o = a_1 - lambda a_2), with a soft cap on the scores, a key width that
// may differ from the value width, an optional sliding window and an optional weightless RMS norm
// of each head's output.  32-bit arithmetic throughout; this file holds the kernels that take every
// size (the 32-bit mode's attention, and bfloat16's for sizes the tensor-core kernels refuse) and
// the write of a step's keys and values into their pages.
//
//   q      [tokens, Hq * MAPS * D]        head by head, a head's maps side by side
//   keys   [pages, page_size, Hkv, MAPS * D]    the same layout per key/value head
//   values [pages, page_size, Hkv, DV]
//   s_m(i, j) = cap * tanh(q_m(i) . k_m(j) * scale / cap)      (cap <= 0: no cap)
//   a_m(i) = sum_j softmax_j(s_m(i, j)) v(j)   over max(0, i + 1 - window) <= j <= i
//   o = a_1 - lambda * a_2   (MAPS = 1: o = a_1);  head_norm: o <- o * rsqrt(mean(o^2) + eps) * out_scale
//   sinks (optional, one fp32 logit a query head): every map's denominator also holds exp(sink_h); a sink
//   is a term exp(sink) of the denominator alone, taken as stored (all zeros: "one added to the denominator")
//   gate (optional, [tokens, Hq * DV], the activations' dtype): o <- o * sigmoid(gate), last of all
//
// Query head h reads key/value head h / (Hq / Hkv).  The order of every sum depends on the
// query's position, the window and the sizes only: warp w of a block takes keys start + w,
// start + w + WARPS, ... with an online softmax of its own per map, and the warps' partial results
// are merged in warp order.  So a token's output does not depend on what else is in the batch
// or on how the prompt was cut.
#include "common.cuh"

#define DA_WARPS 4
#define DA_MAX_D 256
#define DA_MAX_K (DA_MAX_D / 32)

__device__ __forceinline__ float soft_cap(float s, float cap, float inv_cap) { return cap > 0.0f ? cap * tanhf(s * inv_cap) : s; }

template <typename T, int MAPS>
__global__ void __launch_bounds__(DA_WARPS * 32)
diff_attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                              const T* __restrict__ k_cache, const T* __restrict__ v_cache, const int* __restrict__ positions,
                              const int* __restrict__ row_ids, const int* __restrict__ block_table, int max_pages, int Hq,
                              int Hkv, int D, int DV, int page_size, int num_pages, float scale, float cap, int window,
                              float lambda, int head_norm, float eps, float out_scale, const float* __restrict__ sinks,
                              const T* __restrict__ gate, int gate_stride, int* flag) {
    pdl_wait();
    __shared__ float sm_acc[DA_WARPS][MAPS][DA_MAX_D];
    __shared__ float sm_m[DA_WARPS][MAPS];
    __shared__ float sm_l[DA_WARPS][MAPS];
    __shared__ float scratch[32];

    const int t = blockIdx.x;
    const int h = blockIdx.y;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int pos = positions[t];
    const int row = row_ids[t];
    const int kvh = h / (Hq / Hkv);
    const int* table = block_table + (size_t)row * max_pages;
    const int start = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;

    float qv[MAPS][DA_MAX_K];
    const T* qp = q + (size_t)t * q_stride + (size_t)h * MAPS * D;
#pragma unroll
    for (int m = 0; m < MAPS; ++m)
#pragma unroll
        for (int k = 0; k < DA_MAX_K; ++k) {
            const int e = lane + 32 * k;
            qv[m][k] = e < D ? to_float(qp[m * D + e]) : 0.0f;
        }

    float big[MAPS], l[MAPS];
    float acc[MAPS][DA_MAX_K];
#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
        big[m] = -INFINITY;
        l[m] = 0.0f;
#pragma unroll
        for (int k = 0; k < DA_MAX_K; ++k) acc[m][k] = 0.0f;
    }

    for (int j = start + warp; j <= pos; j += DA_WARPS) {
        const int page_index = j / page_size;
        const int page = page_index < max_pages ? table[page_index] : -1;
        if (page < 0 || page >= num_pages) {
            if (lane == 0 && flag) atomicOr(flag, KB_FLAG_BAD_PAGE);
            continue;
        }
        const size_t place = ((size_t)page * page_size + (j % page_size)) * Hkv + kvh;
        const T* kp = k_cache + place * MAPS * D;
        const T* vp = v_cache + place * DV;
        float vv[DA_MAX_K];
#pragma unroll
        for (int k = 0; k < DA_MAX_K; ++k) {
            const int e = lane + 32 * k;
            vv[k] = e < DV ? to_float(vp[e]) : 0.0f;
        }
#pragma unroll
        for (int m = 0; m < MAPS; ++m) {
            float dot = 0.0f;
#pragma unroll
            for (int k = 0; k < DA_MAX_K; ++k) {
                const int e = lane + 32 * k;
                if (e < D) dot += qv[m][k] * to_float(kp[m * D + e]);
            }
            dot = soft_cap(warp_sum(dot) * scale, cap, inv_cap);
            const float m_new = fmaxf(big[m], dot);
            const float alpha = expf(big[m] - m_new);
            const float p = expf(dot - m_new);
            l[m] = l[m] * alpha + p;
#pragma unroll
            for (int k = 0; k < DA_MAX_K; ++k) acc[m][k] = acc[m][k] * alpha + p * vv[k];
            big[m] = m_new;
        }
    }

#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
#pragma unroll
        for (int k = 0; k < DA_MAX_K; ++k) {
            const int e = lane + 32 * k;
            if (e < DV) sm_acc[warp][m][e] = acc[m][k];
        }
        if (lane == 0) {
            sm_m[warp][m] = big[m];
            sm_l[warp][m] = l[m];
        }
    }
    __syncthreads();

    float weights[MAPS][DA_WARPS];
    float denom[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < DA_WARPS; ++w) top = fmaxf(top, sm_m[w][m]);
        const float sink = sinks ? sinks[h] : -INFINITY;
        top = fmaxf(top, sink);
        denom[m] = sinks ? expf(sink - top) : 0.0f;
#pragma unroll
        for (int w = 0; w < DA_WARPS; ++w) {
            weights[m][w] = sm_m[w][m] == -INFINITY ? 0.0f : expf(sm_m[w][m] - top);
            denom[m] += sm_l[w][m] * weights[m][w];
        }
    }
    // DV <= 256 and 128 threads: a thread owns elements threadIdx.x and threadIdx.x + 128
    float o[2];
    float squares = 0.0f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int e = threadIdx.x + i * DA_WARPS * 32;
        o[i] = 0.0f;
        if (e < DV) {
#pragma unroll
            for (int m = 0; m < MAPS; ++m) {
                float a = 0.0f;
#pragma unroll
                for (int w = 0; w < DA_WARPS; ++w) a += sm_acc[w][m][e] * weights[m][w];
                a = denom[m] > 0.0f ? a / denom[m] : 0.0f;
                o[i] = m == 0 ? a : o[i] - lambda * a;
            }
            squares += o[i] * o[i];
        }
    }
    float factor = 1.0f;
    if (head_norm) factor = rsqrtf(block_sum(squares, scratch) / (float)DV + eps) * out_scale;
    T* op = out + (size_t)t * out_stride + (size_t)h * DV;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int e = threadIdx.x + i * DA_WARPS * 32;
        if (e < DV) {
            float v = o[i] * factor;
            if (gate) v *= 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * gate_stride + (size_t)h * DV + e])));
            op[e] = from_float<T>(v);
        }
    }
}

KB_EXPORT int kb_diff_attention_generic(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                                        const void* v_cache, int is_bf16, const int* positions, const int* row_ids,
                                        const int* block_table, int max_pages, int T, int Hq, int Hkv, int maps, int D, int DV,
                                        int page_size, int num_pages, float scale, float cap, int window, float lambda,
                                        int head_norm, float eps, float out_scale, const float* sinks, const void* gate,
                                        int gate_stride, int* flag, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!q || !out || !k_cache || !v_cache || !positions || !row_ids || !block_table) return KB_ERR_NULL;
    if (D < 1 || D > DA_MAX_D || DV < 1 || DV > DA_MAX_D || maps < 1 || maps > 2) return KB_ERR_UNSUPPORTED_SIZE;
    if (Hkv < 1 || Hq % Hkv != 0 || Hq > 65535) return KB_ERR_BAD_ARG;
    dim3 grid(T, Hq);
#define LAUNCH(TT, M)                                                                                                            \
    kb_launch(diff_attention_generic_kernel<TT, M>, grid, dim3(DA_WARPS * 32), 0, stream, (const TT*)q, q_stride, (TT*)out,       \
              out_stride, (const TT*)k_cache, (const TT*)v_cache, positions, row_ids, block_table, max_pages, Hq, Hkv, D, DV,     \
              page_size, num_pages, scale, cap, window, lambda, head_norm, eps, out_scale, sinks, (const TT*)gate, gate_stride, flag)
    if (is_bf16) {
        if (maps == 2) LAUNCH(__nv_bfloat16, 2); else LAUNCH(__nv_bfloat16, 1);
    } else {
        if (maps == 2) LAUNCH(float, 2); else LAUNCH(float, 1);
    }
#undef LAUNCH
    return kb_launch_result();
}

// ------------------------------------------------------------------ keys and values into their pages
// One block a token: columns [k_offset, k_offset + k_width) of its packed row go to the key row of
// its position's page, columns [v_offset, v_offset + v_width) to the value row.  A key row and a
// value row may differ in width.  Positions below the request's write_from lie in pages it only reads.
template <typename T>
__global__ void __launch_bounds__(128)
paged_kv_write_kernel(const T* __restrict__ packed, int stride, int k_offset, int k_width, int v_offset, int v_width,
                      T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ positions,
                      const int* __restrict__ row_ids, const int* __restrict__ block_table, int max_pages,
                      const int* __restrict__ write_from, int page_size, int num_pages, int* flag) {
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int row = row_ids[t];
    if (write_from && pos < write_from[row]) return;
    const int page_index = pos / page_size;
    const int page = (pos >= 0 && page_index < max_pages) ? block_table[(size_t)row * max_pages + page_index] : -1;
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && flag) atomicOr(flag, KB_FLAG_BAD_PAGE);
        return;
    }
    const size_t place = (size_t)page * page_size + (pos % page_size);
    const T* src = packed + (size_t)t * stride;
    for (int i = threadIdx.x; i < k_width; i += blockDim.x) k_cache[place * k_width + i] = src[k_offset + i];
    for (int i = threadIdx.x; i < v_width; i += blockDim.x) v_cache[place * v_width + i] = src[v_offset + i];
}

KB_EXPORT int kb_paged_kv_write(const void* packed, int stride, int is_bf16, int T, int k_offset, int k_width, int v_offset,
                                int v_width, void* k_cache, void* v_cache, const int* positions, const int* row_ids,
                                const int* block_table, int max_pages, const int* write_from, int page_size, int num_pages,
                                int* flag, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!packed || !k_cache || !v_cache || !positions || !row_ids || !block_table) return KB_ERR_NULL;
    if (k_width < 1 || v_width < 0 || page_size < 1) return KB_ERR_BAD_ARG;
    if (is_bf16)
        kb_launch(paged_kv_write_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, (const __nv_bfloat16*)packed, stride, k_offset,
                  k_width, v_offset, v_width, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, positions, row_ids, block_table,
                  max_pages, write_from, page_size, num_pages, flag);
    else
        kb_launch(paged_kv_write_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)packed, stride, k_offset, k_width,
                  v_offset, v_width, (float*)k_cache, (float*)v_cache, positions, row_ids, block_table, max_pages, write_from,
                  page_size, num_pages, flag);
    return kb_launch_result();
}
