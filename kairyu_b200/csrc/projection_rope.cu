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
#define PR_MAX_HEADS 512  // heads of q and k together that the 16-byte kernel keeps per-head statistics for

template <typename T, typename TW>
__global__ void __launch_bounds__(PR_THREADS)
projection_norm_rope_write_kernel(T* __restrict__ packed, int stride, int k_offset, int v_offset, int Hq, int Hkv, int D, int DV,
                                  const TW* __restrict__ wq, const TW* __restrict__ wk, float eps, int per_head,
                                  const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rot_half, int max_pos,
                                  int interleaved, const float* __restrict__ v_cos, const float* __restrict__ v_sin, int v_rot_half, const int* __restrict__ positions, const int* __restrict__ row_ids,
                                  const int* __restrict__ block_table, int max_pages, const int* __restrict__ write_from,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, int num_pages, int num_rows,
                                  int* flag) {
    __shared__ float scratch[32];
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int row = row_ids[t];
    const bool pos_ok = (rot_half == 0 && v_rot_half == 0) || (pos >= 0 && pos < max_pos);
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
    // a head is rot_half pairs and D - 2 * rot_half single columns: D - rot_half units
    const int units = D - rot_half;
    // one unit of head `head`: normed by inv and the weight at w_first + column, rotated, stored
    auto unit = [&](int head, int i, float inv, int w_first) {
        const bool is_q = head < Hq;
        const int first = (is_q ? head : head - Hq) * D;
        const T* src = (is_q ? q : k) + first;
        const TW* w = is_q ? wq : wk;
        T* dst = is_q ? q + first : (k_dst ? k_dst + first : nullptr);
        if (i < rot_half) {
            int a, b;
            rotary_pair(i, rot_half, interleaved, a, b);
            const float x = to_float(src[a]) * inv * (w ? to_float(w[w_first + a]) : 1.0f);
            const float y = to_float(src[b]) * inv * (w ? to_float(w[w_first + b]) : 1.0f);
            float rx, ry;
            rotate(x, y, cs[i], sn[i], rx, ry);
            if (dst) {
                dst[a] = from_float<T>(pos_ok ? rx : 0.0f);
                dst[b] = from_float<T>(pos_ok ? ry : 0.0f);
            }
        } else if (dst) {
            const int c = i + rot_half;
            dst[c] = from_float<T>(to_float(src[c]) * inv * (w ? to_float(w[w_first + c]) : 1.0f));
        }
    };
    if (per_head) {
        // statistics a head (the weights are D entries, shared by the heads): a warp takes a head at a time
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
        for (int head = warp; head < Hq + Hkv; head += warps) {
            float inv = 1.0f;
            if (wq) {
                const T* src = head < Hq ? q + head * D : k + (head - Hq) * D;
                float ss = 0.0f;
                for (int i = lane; i < D; i += 32) {
                    const float x = to_float(src[i]);
                    ss += x * x;
                }
                inv = rsqrtf(warp_sum(ss) / (float)D + eps);  // the butterfly also orders these reads before the writes below
            }
            for (int i = lane; i < units; i += 32) unit(head, i, inv, 0);
        }
    } else {
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
        for (int u = threadIdx.x; u < (Hq + Hkv) * units; u += blockDim.x) {
            const int head = u / units;
            unit(head, u % units, head < Hq ? inv_q : inv_k, (head < Hq ? head : head - Hq) * D);
        }
    }
    if (v_dst && v_rot_half > 0) {
        // values turned by their position over their first 2 * v_rot_half columns, with a table of their own
        const float* vc = v_cos + (size_t)(pos_ok ? pos : 0) * v_rot_half;
        const float* vs = v_sin + (size_t)(pos_ok ? pos : 0) * v_rot_half;
        const int v_units = DV - v_rot_half;
        for (int u = threadIdx.x; u < Hkv * v_units; u += blockDim.x) {
            const int first = (u / v_units) * DV, i = u % v_units;
            if (i < v_rot_half) {
                int a, b;
                rotary_pair(i, v_rot_half, interleaved, a, b);
                float rx, ry;
                rotate(to_float(v[first + a]), to_float(v[first + b]), vc[i], vs[i], rx, ry);
                v_dst[first + a] = from_float<T>(pos_ok ? rx : 0.0f);
                v_dst[first + b] = from_float<T>(pos_ok ? ry : 0.0f);
            } else {
                v_dst[first + i + v_rot_half] = v[first + i + v_rot_half];
            }
        }
    } else if (v_dst) {
        for (int i = threadIdx.x; i < Hkv * DV; i += blockDim.x) v_dst[i] = v[i];
    }
}

// Heads of V columns turned in place by the token's position (inverse: by minus it) over their first
// 2 * rot_half columns: what a mixer whose cached values were turned does to its result.  32-bit arithmetic.
template <typename T>
__global__ void __launch_bounds__(PR_THREADS)
rotate_heads_kernel(T* __restrict__ x, int stride, int H, int V, const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                    int rot_half, int max_pos, int interleaved, int inverse, const int* __restrict__ positions, int* flag) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const bool pos_ok = pos >= 0 && pos < max_pos;
    const float* cs = cos_table + (size_t)(pos_ok ? pos : 0) * rot_half;
    const float* sn = sin_table + (size_t)(pos_ok ? pos : 0) * rot_half;
    pdl_wait();
    if (threadIdx.x == 0 && flag && !pos_ok) atomicOr(flag, KB_FLAG_BAD_POS);
    T* row = x + (size_t)t * stride;
    for (int u = threadIdx.x; u < H * rot_half; u += blockDim.x) {
        const int first = (u / rot_half) * V, i = u % rot_half;
        int a, b;
        rotary_pair(i, rot_half, interleaved, a, b);
        float rx, ry;
        rotate(to_float(row[first + a]), to_float(row[first + b]), cs[i], inverse ? -sn[i] : sn[i], rx, ry);
        row[first + a] = from_float<T>(pos_ok ? rx : 0.0f);
        row[first + b] = from_float<T>(pos_ok ? ry : 0.0f);
    }
}

// The same on bfloat16 rows whose heads, offsets and rotated parts are whole 16-byte groups: a thread takes eight
// columns a turn (a group of the first half with its partner group in split halves; four pairs in one group when
// interleaved), so that a row is read and written in 16-byte accesses.  The arithmetic is the scalar kernel's.
struct alignas(16) Bf16x8 {
    __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const Bf16x8& in, float (&out)[8]);

// eight weights from a 16-byte aligned place (at is a multiple of 8), times inv: one or two 16-byte loads
__device__ __forceinline__ void load_weights8(const __nv_bfloat16* w, int at, float inv, float (&out)[8]) {
    if (w) unpack8(*reinterpret_cast<const Bf16x8*>(w + at), out);
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = w ? inv * out[e] : inv;
}

__device__ __forceinline__ void load_floats(const float* at, int count, float* out) {  // count 4 or 8, 16-byte aligned
    for (int e = 0; e < count; e += 4) *reinterpret_cast<float4*>(out + e) = *reinterpret_cast<const float4*>(at + e);
}

__device__ __forceinline__ void load_weights8(const float* w, int at, float inv, float (&out)[8]) {
    if (w) load_floats(w + at, 8, out);
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = w ? inv * out[e] : inv;
}

__device__ __forceinline__ void unpack8(const Bf16x8& in, float (&out)[8]) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 two = __bfloat1622float2(in.v[e]);
        out[2 * e] = two.x;
        out[2 * e + 1] = two.y;
    }
}

__device__ __forceinline__ Bf16x8 pack8(const float (&in)[8]) {
    Bf16x8 out;
#pragma unroll
    for (int e = 0; e < 4; ++e) out.v[e] = __floats2bfloat162_rn(in[2 * e], in[2 * e + 1]);
    return out;
}

template <typename TW>
__global__ void __launch_bounds__(PR_THREADS)
projection_norm_rope_write_vec_kernel(__nv_bfloat16* __restrict__ packed, int stride, int k_offset, int v_offset, int Hq, int Hkv, int D,
                                      int DV, const TW* __restrict__ wq, const TW* __restrict__ wk, float eps, int per_head,
                                      const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rot_half, int max_pos,
                                      int interleaved, const float* __restrict__ v_cos, const float* __restrict__ v_sin, int v_rot_half,
                                      const int* __restrict__ positions, const int* __restrict__ row_ids,
                                      const int* __restrict__ block_table, int max_pages, const int* __restrict__ write_from,
                                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int page_size,
                                      int num_pages, int num_rows, int* flag) {
    __shared__ float scratch[32];
    __shared__ float head_inv[PR_MAX_HEADS];  // per_head: 1 / rms of every head of q, then of k
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int row = row_ids[t];
    const bool pos_ok = (rot_half == 0 && v_rot_half == 0) || (pos >= 0 && pos < max_pos);
    const float* cs = cos_table + (size_t)(pos_ok ? pos : 0) * rot_half;
    const float* sn = sin_table + (size_t)(pos_ok ? pos : 0) * rot_half;
    __nv_bfloat16* k_dst = nullptr;
    __nv_bfloat16* v_dst = nullptr;
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
    __nv_bfloat16* q = packed + (size_t)t * stride;
    __nv_bfloat16* k = q + k_offset;
    const __nv_bfloat16* v = q + v_offset;
    float inv_q = 1.0f, inv_k = 1.0f;
    if (wq && per_head) {
        // statistics a head: a warp takes a head at a time, a lane eight columns a turn
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
        float x[8];
        for (int head = warp; head < Hq + Hkv; head += warps) {
            const __nv_bfloat16* src = head < Hq ? q + head * D : k + (head - Hq) * D;
            float ss = 0.0f;
            for (int i = lane; i < D / 8; i += 32) {
                unpack8(*reinterpret_cast<const Bf16x8*>(src + i * 8), x);
#pragma unroll
                for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
            }
            ss = warp_sum(ss);
            if (lane == 0) head_inv[head] = rsqrtf(ss / (float)D + eps);
        }
        __syncthreads();  // the statistics are read, and every head's columns were read before any is written
    } else if (wq) {
        float sq = 0.0f, sk = 0.0f;
        float x[8];
        for (int i = threadIdx.x; i < Hq * D / 8; i += blockDim.x) {
            unpack8(*reinterpret_cast<const Bf16x8*>(q + i * 8), x);
#pragma unroll
            for (int e = 0; e < 8; ++e) sq += x[e] * x[e];
        }
        for (int i = threadIdx.x; i < Hkv * D / 8; i += blockDim.x) {
            unpack8(*reinterpret_cast<const Bf16x8*>(k + i * 8), x);
#pragma unroll
            for (int e = 0; e < 8; ++e) sk += x[e] * x[e];
        }
        inv_q = rsqrtf(block_sum(sq, scratch) / (float)(Hq * D) + eps);
        inv_k = rsqrtf(block_sum(sk, scratch) / (float)(Hkv * D) + eps);
    }
    const int groups = D / 8;                               // 16-byte groups a head
    const int rot_groups = interleaved ? rot_half / 4 : rot_half / 8;  // groups that begin a rotation (split halves: of the first half)
    const int skip_from = interleaved ? groups : rot_groups, skip_to = interleaved ? groups : 2 * rot_groups;  // partner groups, done with their first
    for (int u = threadIdx.x; u < (Hq + Hkv) * groups; u += blockDim.x) {
        const int head = u / groups, j = u % groups;
        if (j >= skip_from && j < skip_to) continue;
        const bool is_q = head < Hq;
        const int first = (is_q ? head : head - Hq) * D;
        const __nv_bfloat16* src = (is_q ? q : k) + first;
        const TW* w = is_q ? wq : wk;
        const float inv = (wq && per_head) ? head_inv[head] : (is_q ? inv_q : inv_k);
        const int w_first = per_head ? 0 : first;  // per_head: the weights are a head's D entries
        __nv_bfloat16* dst = is_q ? q + first : (k_dst ? k_dst + first : nullptr);
        if (!dst) continue;
        float a[8], wa[8];
        unpack8(*reinterpret_cast<const Bf16x8*>(src + j * 8), a);
        load_weights8(w, w_first + j * 8, inv, wa);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] *= wa[e];
        if (j >= rot_groups) {  // behind the rotated columns
            *reinterpret_cast<Bf16x8*>(dst + j * 8) = pack8(a);
        } else if (interleaved) {
            float c4[4], s4[4];
            load_floats(cs + j * 4, 4, c4);
            load_floats(sn + j * 4, 4, s4);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float rx, ry;
                rotate(a[2 * e], a[2 * e + 1], c4[e], s4[e], rx, ry);
                a[2 * e] = pos_ok ? rx : 0.0f;
                a[2 * e + 1] = pos_ok ? ry : 0.0f;
            }
            *reinterpret_cast<Bf16x8*>(dst + j * 8) = pack8(a);
        } else {
            float b[8], wb[8];
            unpack8(*reinterpret_cast<const Bf16x8*>(src + rot_half + j * 8), b);
            load_weights8(w, w_first + rot_half + j * 8, inv, wb);
            float c8[8], s8[8];
            load_floats(cs + j * 8, 8, c8);
            load_floats(sn + j * 8, 8, s8);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float rx, ry;
                rotate(a[e], b[e] * wb[e], c8[e], s8[e], rx, ry);
                a[e] = pos_ok ? rx : 0.0f;
                b[e] = pos_ok ? ry : 0.0f;
            }
            *reinterpret_cast<Bf16x8*>(dst + j * 8) = pack8(a);
            *reinterpret_cast<Bf16x8*>(dst + rot_half + j * 8) = pack8(b);
        }
    }
    if (v_dst && v_rot_half > 0) {
        // interleaved pairs only (the launcher sends the split-halves layout to the scalar kernel): four pairs a group
        const float* vc = v_cos + (size_t)(pos_ok ? pos : 0) * v_rot_half;
        const float* vs = v_sin + (size_t)(pos_ok ? pos : 0) * v_rot_half;
        const int v_groups = DV / 8, v_rot_groups = v_rot_half / 4;
        for (int i = threadIdx.x; i < Hkv * v_groups; i += blockDim.x) {
            const int j = i % v_groups;
            float a[8];
            unpack8(*reinterpret_cast<const Bf16x8*>(v + i * 8), a);
            if (j < v_rot_groups) {
                float c4[4], s4[4];
                load_floats(vc + j * 4, 4, c4);
                load_floats(vs + j * 4, 4, s4);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float rx, ry;
                    rotate(a[2 * e], a[2 * e + 1], c4[e], s4[e], rx, ry);
                    a[2 * e] = pos_ok ? rx : 0.0f;
                    a[2 * e + 1] = pos_ok ? ry : 0.0f;
                }
            }
            *reinterpret_cast<Bf16x8*>(v_dst + i * 8) = pack8(a);
        }
    } else if (v_dst) {
        for (int i = threadIdx.x; i < Hkv * DV / 8; i += blockDim.x)
            *reinterpret_cast<Bf16x8*>(v_dst + i * 8) = *reinterpret_cast<const Bf16x8*>(v + i * 8);
    }
}

// wq/wk null: no norm; per_head: statistics a head and weights of D entries, else over the whole projection.
// cos/sin null (rot_half 0): no rotation.  v_cos/v_sin (v_rot_half > 0): the values turn too, by a table of their
// own of the same number of positions.  k_cache null: q only.
KB_EXPORT int kb_projection_norm_rope_write(void* packed, int stride, int is_bf16, int T, int k_offset, int v_offset, int Hq, int Hkv,
                                            int D, int DV, const void* wq, const void* wk, int w_bf16, float eps, int per_head,
                                            const float* cos_table, const float* sin_table, int rot_half, int max_pos, int interleaved,
                                            const float* v_cos, const float* v_sin, int v_rot_half,
                                            const int* positions, const int* row_ids, const int* block_table, int max_pages,
                                            const int* write_from, void* k_cache, void* v_cache, int page_size, int num_pages,
                                            int num_rows, int* flag, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!packed || !positions || !row_ids) return KB_ERR_NULL;
    if ((wq == nullptr) != (wk == nullptr)) return KB_ERR_BAD_ARG;
    if (Hq < 1 || Hkv < 0 || (Hkv == 0 && k_cache) || D < 1 || DV < 1 || rot_half < 0 || 2 * rot_half > D) return KB_ERR_BAD_ARG;  // no key heads: queries alone
    if (rot_half > 0 && (!cos_table || !sin_table || max_pos < 1)) return KB_ERR_NULL;
    if (v_rot_half < 0 || 2 * v_rot_half > DV || (v_rot_half > 0 && (!v_cos || !v_sin || max_pos < 1))) return KB_ERR_BAD_ARG;
    if (k_cache && (!v_cache || !block_table || page_size < 1)) return KB_ERR_NULL;
#define LAUNCH(TT, TW)                                                                                                              \
    kb_launch(projection_norm_rope_write_kernel<TT, TW>, dim3(T), dim3(PR_THREADS), 0, stream, (TT*)packed, stride, k_offset,         \
              v_offset, Hq, Hkv, D, DV, (const TW*)wq, (const TW*)wk, eps, per_head, cos_table, sin_table, rot_half, max_pos,       \
              interleaved, v_cos, v_sin, v_rot_half, positions, row_ids, block_table, max_pages, write_from, (TT*)k_cache, (TT*)v_cache, page_size, num_pages, num_rows, flag)
    // whole 16-byte groups everywhere: heads, offsets, rows, the rotated part (split halves: each half) and the pages
    const bool groups_of_eight = (!per_head || Hq + Hkv <= PR_MAX_HEADS) && (v_rot_half == 0 || (interleaved && v_rot_half % 4 == 0 && (uintptr_t)v_cos % 16 == 0 && (uintptr_t)v_sin % 16 == 0)) && is_bf16 && D % 8 == 0 && DV % 8 == 0 && stride % 8 == 0 && k_offset % 8 == 0 && v_offset % 8 == 0 &&
                                 (interleaved ? rot_half % 4 == 0 : rot_half % 8 == 0) && (uintptr_t)packed % 16 == 0 &&
                                 (uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0 && (uintptr_t)wq % 16 == 0 &&
                                 (uintptr_t)wk % 16 == 0 && (uintptr_t)cos_table % 16 == 0 && (uintptr_t)sin_table % 16 == 0;
#define LAUNCH_VEC(TW)                                                                                                              \
    kb_launch(projection_norm_rope_write_vec_kernel<TW>, dim3(T), dim3(PR_THREADS), 0, stream, (__nv_bfloat16*)packed, stride,        \
              k_offset, v_offset, Hq, Hkv, D, DV, (const TW*)wq, (const TW*)wk, eps, per_head, cos_table, sin_table, rot_half, max_pos, \
              interleaved, v_cos, v_sin, v_rot_half, positions, row_ids, block_table, max_pages, write_from, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, \
              page_size, num_pages, num_rows, flag)
    if (groups_of_eight) {
        if (w_bf16) LAUNCH_VEC(__nv_bfloat16); else LAUNCH_VEC(float);
    } else if (is_bf16) {
        if (w_bf16) LAUNCH(__nv_bfloat16, __nv_bfloat16); else LAUNCH(__nv_bfloat16, float);
    } else {
        if (w_bf16) LAUNCH(float, __nv_bfloat16); else LAUNCH(float, float);
    }
#undef LAUNCH
#undef LAUNCH_VEC
    return kb_launch_result();
}

KB_EXPORT int kb_rotate_heads(void* x, int stride, int is_bf16, int T, int H, int V, const float* cos_table, const float* sin_table,
                              int rot_half, int max_pos, int interleaved, int inverse, const int* positions, int* flag, cudaStream_t stream) {
    if (T == 0 || rot_half == 0) return 0;
    if (!x || !cos_table || !sin_table || !positions) return KB_ERR_NULL;
    if (H < 1 || V < 1 || rot_half < 0 || 2 * rot_half > V || max_pos < 1) return KB_ERR_BAD_ARG;
    if (is_bf16)
        kb_launch(rotate_heads_kernel<__nv_bfloat16>, dim3(T), dim3(PR_THREADS), 0, stream, (__nv_bfloat16*)x, stride, H, V, cos_table, sin_table,
                  rot_half, max_pos, interleaved, inverse, positions, flag);
    else
        kb_launch(rotate_heads_kernel<float>, dim3(T), dim3(PR_THREADS), 0, stream, (float*)x, stride, H, V, cos_table, sin_table, rot_half,
                  max_pos, interleaved, inverse, positions, flag);
    return kb_launch_result();
}
