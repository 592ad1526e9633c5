// The cache write of latent attention: a token's compressed key/value row
//
//     c[t] = z[t] * rsqrt(mean(z[t]^2) + eps) * w        z = columns [offset, offset + R) of a packed product
//
// is normed in 32-bit and stored once, in the cache's dtype, at the token's place in its request's
// pages (one "head" of R columns).  Keys and values of every head are products of this row, so it
// is all such a layer keeps.  Positions below write_from[row] lie in pages the request only
// reads and are skipped.  One block per token.
//
// With a rotated part (rot > 0) the packed product has rot more columns behind z: one key part that
// all heads share, which carries the position.  It is turned by the token's angles (not normed) and
// stored behind c, so that a cache row is R + rot wide.  The queries' rotated parts (the last rot of
// every head's D + rot columns of the packed query) are turned the same way and written behind the
// first R columns of that head's row of `q_out`, whose first R columns another kernel fills with
// the query carried into the latent space: a cached row then scores against a query row by one
// dot product of R + rot.
#include "common.cuh"
#include "rotary.cuh"

template <typename TZ, typename TW, typename TC>
__global__ void __launch_bounds__(128)
latent_norm_write_kernel(const TZ* __restrict__ z, int z_stride, int offset, int R, const TW* __restrict__ w, float eps,
                         const int* __restrict__ positions, const int* __restrict__ row_ids,
                         const int* __restrict__ block_table, int max_pages, const int* __restrict__ write_from,
                         TC* __restrict__ cache, int page_size, int num_pages, int num_rows, int rot,
                         const float* __restrict__ cos_table, const float* __restrict__ sin_table, int max_pos, int interleaved,
                         int heads, int q_head_width, TZ* __restrict__ q_out, int q_out_stride, int writes, int* flag) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int row = row_ids[t];
    const int rot_half = rot >> 1;
    const bool pos_ok = rot == 0 || (pos >= 0 && pos < max_pos);
    const float* cs = cos_table + (size_t)(pos_ok ? pos : 0) * rot_half;
    const float* sn = sin_table + (size_t)(pos_ok ? pos : 0) * rot_half;
    pdl_wait();
    if (!pos_ok && threadIdx.x == 0 && flag) atomicOr(flag, KB_FLAG_BAD_POS);
    const TZ* zr = z + (size_t)t * z_stride;
    if (rot > 0 && q_out) {
        // head h: packed columns [h * q_head_width + (q_head_width - rot), (h + 1) * q_head_width) -> q_out columns [R, R + rot) of head h
        for (int u = threadIdx.x; u < heads * rot_half; u += blockDim.x) {
            const int h = u / rot_half, i = u % rot_half;
            int a, b;
            rotary_pair(i, rot_half, interleaved, a, b);
            const TZ* src = zr + (size_t)h * q_head_width + (q_head_width - rot);
            float ra, rb;
            rotate(to_float(src[a]), to_float(src[b]), cs[i], sn[i], ra, rb);
            TZ* dst = q_out + (size_t)t * q_out_stride + (size_t)h * (R + rot) + R;
            dst[a] = from_float<TZ>(pos_ok ? ra : 0.0f);
            dst[b] = from_float<TZ>(pos_ok ? rb : 0.0f);
        }
    }
    if (!writes) return;
    zr += offset;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const float v = to_float(zr[i]);
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    if (row < 0 || row >= num_rows) {
        if (threadIdx.x == 0 && flag) atomicOr(flag, KB_FLAG_BAD_ROW);
        return;
    }
    if (write_from && pos < write_from[row]) return;
    const int page_index = pos / page_size;
    const int page = (pos >= 0 && page_index < max_pages) ? block_table[(size_t)row * max_pages + page_index] : -1;
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && flag) atomicOr(flag, KB_FLAG_BAD_PAGE);
        return;
    }
    const float inv = rsqrtf(total / (float)R + eps);
    TC* dst = cache + ((size_t)page * page_size + (pos % page_size)) * (R + rot);
    for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = from_float<TC>(to_float(zr[i]) * inv * to_float(w[i]));
    for (int i = threadIdx.x; i < rot_half; i += blockDim.x) {
        int a, b;
        rotary_pair(i, rot_half, interleaved, a, b);
        float ra, rb;
        rotate(to_float(zr[R + a]), to_float(zr[R + b]), cs[i], sn[i], ra, rb);
        dst[R + a] = from_float<TC>(pos_ok ? ra : 0.0f);
        dst[R + b] = from_float<TC>(pos_ok ? rb : 0.0f);
    }
}

// rot == 0: the plain form (cos, sin, q_out unused).  writes == 0: only the queries' rotated parts are produced.
KB_EXPORT int kb_latent_norm_write(const void* z, int z_stride, int offset, int R, int is_bf16, const void* w, int w_is_bf16,
                                   float eps, const int* positions, const int* row_ids, const int* block_table, int max_pages,
                                   const int* write_from, void* cache, int page_size, int num_pages, int num_rows, int T,
                                   int rot, const float* cos_table, const float* sin_table, int max_pos, int interleaved, int heads,
                                   int q_head_width, void* q_out, int q_out_stride, int writes, int* flag, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!z || !w || !positions || !row_ids) return KB_ERR_NULL;
    if (writes && (!block_table || !cache)) return KB_ERR_NULL;
    if (R < 1 || page_size < 1 || rot < 0 || rot % 2) return KB_ERR_BAD_ARG;
    if (rot > 0 && (!cos_table || !sin_table || max_pos < 1 || (q_out && (heads < 1 || q_head_width < rot)))) return KB_ERR_BAD_ARG;
#define LAUNCH(TZ, TW)                                                                                                   \
    kb_launch(latent_norm_write_kernel<TZ, TW, TZ>, dim3(T), dim3(128), 0, stream, (const TZ*)z, z_stride, offset, R,     \
              (const TW*)w, eps, positions, row_ids, block_table, max_pages, write_from, (TZ*)cache, page_size, num_pages, \
              num_rows, rot, cos_table, sin_table, max_pos, interleaved, heads, q_head_width, (TZ*)q_out, q_out_stride,    \
              writes, flag)
    if (is_bf16) {
        if (w_is_bf16) LAUNCH(__nv_bfloat16, __nv_bfloat16); else LAUNCH(__nv_bfloat16, float);
    } else {
        if (w_is_bf16) LAUNCH(float, __nv_bfloat16); else LAUNCH(float, float);
    }
#undef LAUNCH
    return kb_launch_result();
}
