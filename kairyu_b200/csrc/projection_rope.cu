// Query/key norm over the WHOLE projection, rotation, and the page write of keys and values of
// different widths, for one step's packed rows [q | k | v | ...]:
//
//   q <- q * rsqrt(mean(q^2) + eps) * wq      mean over all Hq * D columns of the token at once
//   k <- k * rsqrt(mean(k^2) + eps) * wk      mean over all Hkv * D columns        (no weights: no norm)
//   per head, the first 2 * rot_half columns turn by the token's angles: pair i is columns
//   (i, i + rot_half) (split halves) or (2i, 2i + 1) (interleaved); columns behind them keep their values
//   q goes back in place, k to the key page [pages, page_size, Hkv, D], v (untouched) to the value
//   page [pages, page_size, Hkv, DV]
//
// Statistics, weights and the rotation are 32-bit, with one rounding at the store.  One block per
// token; a thread owns whole pairs, so the in-place write of q races with nothing.  Positions below
// write_from[row] lie in pages the request only reads and are skipped (q is still produced).
#include "common.cuh"
#include "rotary.cuh"

#define PR_THREADS 256

template <typename T, typename TW>
__global__ void __launch_bounds__(PR_THREADS)
projection_norm_rope_write_kernel(T* __restrict__ packed, int stride, int k_offset, int v_offset, int Hq, int Hkv, int D, int DV,
                                  const TW* __restrict__ wq, const TW* __restrict__ wk, float eps,
                                  const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rot_half, int max_pos,
                                  int interleaved, const int* __restrict__ positions, const int* __restrict__ row_ids,
                                  const int* __restrict__ block_table, int max_pages, const int* __restrict__ write_from,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, int num_pages, int num_rows,
                                  int* flag) {
    __shared__ float scratch[32];
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int row = row_ids[t];
    const bool pos_ok = rot_half == 0 || (pos >= 0 && pos < max_pos);
    const float* cs = cos_table + (size_t)(pos_ok ? pos : 0) * rot_half;
    const float* sn = sin_table + (size_t)(pos_ok ? pos : 0) * rot_half;
    // where the token's key and value rows go (nullptr: nowhere)
    T* k_dst = nullptr;
    T* v_dst = nullptr;
    bool bad_row = false, bad_page = false;
    if (k_cache) {
        if (row < 0 || row >= num_rows) {
            bad_row = true;
        } else if (!(write_from && pos < write_from[row])) {
            const int page_index = pos / page_size;
            const int page = (pos >= 0 && page_index < max_pages) ? block_table[(size_t)row * max_pages + page_index] : -1;
            if (page < 0 || page >= num_pages) {
                bad_page = true;
            } else {
                const size_t place = (size_t)page * page_size + (pos % page_size);
                k_dst = k_cache + place * Hkv * D;
                v_dst = v_cache + place * Hkv * DV;
            }
        }
    }
    pdl_wait();
    if (threadIdx.x == 0 && flag) {
        if (!pos_ok) atomicOr(flag, KB_FLAG_BAD_POS);
        if (bad_row) atomicOr(flag, KB_FLAG_BAD_ROW);
        if (bad_page) atomicOr(flag, KB_FLAG_BAD_PAGE);
    }
    T* q = packed + (size_t)t * stride;
    T* k = q + k_offset;
    const T* v = q + v_offset;
    float inv_q = 1.0f, inv_k = 1.0f;
    if (wq) {
        float sq = 0.0f, sk = 0.0f;
        for (int i = threadIdx.x; i < Hq * D; i += blockDim.x) {
            const float x = to_float(q[i]);
            sq += x * x;
        }
        for (int i = threadIdx.x; i < Hkv * D; i += blockDim.x) {
            const float x = to_float(k[i]);
            sk += x * x;
        }
        inv_q = rsqrtf(block_sum(sq, scratch) / (float)(Hq * D) + eps);
        inv_k = rsqrtf(block_sum(sk, scratch) / (float)(Hkv * D) + eps);
    }
    // a head is rot_half pairs and D - 2 * rot_half single columns: D - rot_half units
    const int units = D - rot_half;
    for (int u = threadIdx.x; u < (Hq + Hkv) * units; u += blockDim.x) {
        const int head = u / units, i = u % units;
        const bool is_q = head < Hq;
        const int first = (is_q ? head : head - Hq) * D;
        const T* src = (is_q ? q : k) + first;
        const TW* w = is_q ? wq : wk;
        const float inv = is_q ? inv_q : inv_k;
        T* dst = is_q ? q + first : (k_dst ? k_dst + first : nullptr);
        if (i < rot_half) {
            int a, b;
            rotary_pair(i, rot_half, interleaved, a, b);
            const float x = to_float(src[a]) * inv * (w ? to_float(w[first + a]) : 1.0f);
            const float y = to_float(src[b]) * inv * (w ? to_float(w[first + b]) : 1.0f);
            float rx, ry;
            rotate(x, y, cs[i], sn[i], rx, ry);
            if (dst) {
                dst[a] = from_float<T>(pos_ok ? rx : 0.0f);
                dst[b] = from_float<T>(pos_ok ? ry : 0.0f);
            }
        } else if (dst) {
            const int c = i + rot_half;
            dst[c] = from_float<T>(to_float(src[c]) * inv * (w ? to_float(w[first + c]) : 1.0f));
        }
    }
    if (v_dst)
        for (int i = threadIdx.x; i < Hkv * DV; i += blockDim.x) v_dst[i] = v[i];
}

// wq/wk null: no norm.  cos/sin null (rot_half 0): no rotation.  k_cache null: q only.
KB_EXPORT int kb_projection_norm_rope_write(void* packed, int stride, int is_bf16, int T, int k_offset, int v_offset, int Hq, int Hkv,
                                            int D, int DV, const void* wq, const void* wk, int w_bf16, float eps,
                                            const float* cos_table, const float* sin_table, int rot_half, int max_pos, int interleaved,
                                            const int* positions, const int* row_ids, const int* block_table, int max_pages,
                                            const int* write_from, void* k_cache, void* v_cache, int page_size, int num_pages,
                                            int num_rows, int* flag, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!packed || !positions || !row_ids) return KB_ERR_NULL;
    if ((wq == nullptr) != (wk == nullptr)) return KB_ERR_BAD_ARG;
    if (Hq < 1 || Hkv < 1 || D < 1 || DV < 1 || rot_half < 0 || 2 * rot_half > D) return KB_ERR_BAD_ARG;
    if (rot_half > 0 && (!cos_table || !sin_table || max_pos < 1)) return KB_ERR_NULL;
    if (k_cache && (!v_cache || !block_table || page_size < 1)) return KB_ERR_NULL;
#define LAUNCH(TT, TW)                                                                                                              \
    kb_launch(projection_norm_rope_write_kernel<TT, TW>, dim3(T), dim3(PR_THREADS), 0, stream, (TT*)packed, stride, k_offset,         \
              v_offset, Hq, Hkv, D, DV, (const TW*)wq, (const TW*)wk, eps, cos_table, sin_table, rot_half, max_pos, interleaved,     \
              positions, row_ids, block_table, max_pages, write_from, (TT*)k_cache, (TT*)v_cache, page_size, num_pages, num_rows, flag)
    if (is_bf16) {
        if (w_bf16) LAUNCH(__nv_bfloat16, __nv_bfloat16); else LAUNCH(__nv_bfloat16, float);
    } else {
        if (w_bf16) LAUNCH(float, __nv_bfloat16); else LAUNCH(float, float);
    }
#undef LAUNCH
    return kb_launch_result();
}
