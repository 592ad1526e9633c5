// Mixture of experts: routing, the plan of a step's (token, expert) pairs, and the two grouped
// products of the experts.
//
//   moe_route     per token: the K largest of (router logits + bias) choose the experts (ties go to
//                 the lower index); their weights are the softmax over the K chosen logits.  32-bit.
//   moe_plan      one block: pairs p = t * K + k are counted per expert, the experts' runs are laid
//                 side by side (`sorted` lists the pairs run by run, `token_of` their tokens,
//                 `place_of[p]` is where pair p stands, `ends[e]` where expert e's run ends), and
//                 the runs are cut into tiles of MOE_TM pairs: tile -> (expert, first place, pairs).
//   moe_route_scores  per token: softmax over all outputs, a correction that steers the choice only, groups of
//                 neighbours of which the best stay, the K best that stay; weights = score * scale.  32-bit.
//                 With `sigmoid` the scores are s = sigmoid(logit), each output by itself, instead of the softmax.
//   moe_scale_rows  out[i] = src[token of i] * scale[pair of i]: the experts' input rows for a mixture whose router
//                 weight multiplies an expert's INPUT (the experts are not linear, so it cannot move to the output).
//   moe_activation  y = a * sigmoid(alpha a) * (b + shift) with a = min(gate, limit), b = clamp(up, +-limit)
//                 over rows [gate columns | up columns]: for the path whose products are a library's.
//   moe_grouped   one block per (tile, 64 output columns): a [pairs, K] x [K, 64] product with the
//                 tile's expert's weight.  Gated form: A rows are the tokens' activations (gathered
//                 through the pair list), the weight holds the expert's gate rows and then its up
//                 rows, and the epilogue is the expert's activation
//                     a = min(gate, limit), b = clamp(up, -limit, limit), y = a * sigmoid(alpha a) * (b + shift)
//                 (limit infinite, alpha 1, shift 0: silu(gate) * up)
//                 written at the pair's place in `sorted`.  Plain form: A rows are those y rows, and
//                 the result goes, in 32-bit, to row p of the output, so that the K rows of a token lie
//                 together and whoever adds them (weighted by the router) does so in the order of k.
//                 bfloat16 runs on mma.sync m16n8k16 with 32-bit accumulators, float32 on FMAs; the
//                 sum over K runs in ascending order in both, whatever else the tile holds.
//   moe_combine   out[t] = sum_k weight[t, k] * rows[at(t * K + k)]   (for callers that want plain rows; no weights: a
//                 plain sum) + sigmoid(extra_gate[t]) * extra[t] when an always-on expert's rows are given; a pair whose
//                 id is not below the number of experts with weights is an identity expert: its row is the token's own.
//                 The grouped kernels skip such pairs' tiles.
#include "common.cuh"

#define MOE_TM 64
#define MOE_TN 64
#define MOE_TK 32
#define MOE_MAX_EXPERTS 1024
#define MOE_MAX_TOP 32

template <typename TB>
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, const TB* __restrict__ bias, int E, int K, int* __restrict__ ids,
                 float* __restrict__ weights, int T) {
    pdl_wait();
    // one warp a token: every lane holds the logits e = lane, lane + 32, ...
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= T) return;
    float chosen_value[MOE_MAX_TOP];
    int chosen_id[MOE_MAX_TOP];
    float last_value = INFINITY;
    int last_id = -1;
    for (int k = 0; k < K; ++k) {
        // the largest (value, then lower index) that comes after the one chosen before in that order
        float best = -INFINITY;
        int best_id = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float z = logits[(size_t)t * E + e] + (bias ? to_float(bias[e]) : 0.0f);
            const bool after = z < last_value || (z == last_value && e > last_id);
            if (after && (z > best || (z == best && e < best_id))) {
                best = z;
                best_id = e;
            }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, offset);
            const int other_id = __shfl_xor_sync(0xffffffffu, best_id, offset);
            if (other > best || (other == best && other_id < best_id)) {
                best = other;
                best_id = other_id;
            }
        }
        chosen_value[k] = best;
        chosen_id[k] = best_id;
        last_value = best;
        last_id = best_id;
    }
    if (lane == 0) {
        float denom = 0.0f;
        for (int k = 0; k < K; ++k) denom += expf(chosen_value[k] - chosen_value[0]);
        for (int k = 0; k < K; ++k) {
            ids[(size_t)t * K + k] = chosen_id[k] < E ? chosen_id[k] : 0;
            weights[(size_t)t * K + k] = expf(chosen_value[k] - chosen_value[0]) / denom;
        }
    }
}

// limit may be infinite (no clamps); alpha = 1, shift = 0 is the plain unit silu(gate) * up
__device__ __forceinline__ float expert_activation(float gate, float up, float limit, float alpha, float shift) {
    const float a = fminf(gate, limit);
    const float b = fminf(fmaxf(up, -limit), limit);
    return a * (1.0f / (1.0f + expf(-alpha * a))) * (b + shift);
}

__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, int pairs, int E, int top, int* __restrict__ sorted, int* __restrict__ token_of,
                int* __restrict__ place_of, int* __restrict__ ends, int* __restrict__ tile_expert,
                int* __restrict__ tile_first, int* __restrict__ tile_pairs, int* __restrict__ num_tiles) {
    __shared__ int counts[MOE_MAX_EXPERTS];
    __shared__ int cursor[MOE_MAX_EXPERTS];
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&counts[ids[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < E; ++e) {
            cursor[e] = at;
            for (int first = 0; first < counts[e]; first += MOE_TM) {
                tile_expert[tiles] = e;
                tile_first[tiles] = at + first;
                tile_pairs[tiles] = min(MOE_TM, counts[e] - first);
                ++tiles;
            }
            at += counts[e];
            ends[e] = at;
        }
        *num_tiles = tiles;
    }
    __syncthreads();
    // The order of the pairs inside an expert's run is whatever the additions below give; a pair's
    // result does not depend on its place in a tile.
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int place = atomicAdd(&cursor[ids[p]], 1);
        sorted[place] = p;
        token_of[place] = p / top;
        place_of[p] = place;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_activation_kernel(const T* __restrict__ gate_up, T* __restrict__ y, int F, float limit, float alpha, float shift, size_t total) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t row = i / F, col = i % F;
    const float gate = to_float(gate_up[row * 2 * F + col]), up = to_float(gate_up[row * 2 * F + F + col]);
    y[i] = from_float<T>(expert_activation(gate, up, limit, alpha, shift));
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}


// 8 bfloat16 (or 4 float) of a row into shared memory, zeros beyond the row's end or for a row that is not there
__device__ __forceinline__ void stage_chunk(__nv_bfloat16* dst, const __nv_bfloat16* row, int k, int Kd, bool vec) {
    if (row && vec && k + 8 <= Kd) {
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(row + k);
        return;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) dst[e] = (row && k + e < Kd) ? row[k + e] : __float2bfloat16_rn(0.0f);
}
__device__ __forceinline__ void stage_chunk(float* dst, const float* row, int k, int Kd, bool vec) {
    if (row && vec && k + 4 <= Kd) {
        const float4 v = *reinterpret_cast<const float4*>(row + k);
        dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
        return;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) dst[e] = (row && k + e < Kd) ? row[k + e] : 0.0f;
}

template <typename T> struct MoeTile;
template <> struct MoeTile<__nv_bfloat16> { static constexpr int LD = MOE_TK + 8; static constexpr int CHUNK = 8; };
template <> struct MoeTile<float> { static constexpr int LD = MOE_TK + 1; static constexpr int CHUNK = 4; };

template <typename T, bool GATED>
__global__ void __launch_bounds__(128)
moe_grouped_kernel(const T* __restrict__ A, int lda, const int* __restrict__ sorted, int top, const T* __restrict__ W,
                   int N, int Kd, const int* __restrict__ tile_expert, const int* __restrict__ tile_first,
                   const int* __restrict__ tile_pairs, const int* __restrict__ num_tiles, float limit, float alpha,
                   float shift, int real_experts, void* __restrict__ out, int vec) {
    constexpr int LD = MoeTile<T>::LD;
    constexpr int CHUNK = MoeTile<T>::CHUNK;
    constexpr int NB = GATED ? 2 : 1;
    __shared__ __align__(16) T As[MOE_TM][LD];
    __shared__ __align__(16) T Bs[NB][MOE_TN][LD];
    __shared__ int a_row[MOE_TM];   // source row of A per tile row, -1: none
    __shared__ int o_row[MOE_TM];   // destination row
    pdl_wait();
    const int tile = blockIdx.x;
    if (tile >= *num_tiles) return;
    const int expert = tile_expert[tile], first = tile_first[tile], rows = tile_pairs[tile];
    if (expert >= real_experts) return;  // a run of pairs whose "expert" has no weights (an identity expert): the sum takes the token's row itself
    const int n0 = blockIdx.y * MOE_TN;
    for (int i = threadIdx.x; i < MOE_TM; i += blockDim.x) {
        int src = -1, dst = -1;
        if (i < rows) {
            const int p = sorted[first + i];
            src = GATED ? p / top : first + i;
            dst = GATED ? first + i : p;
        }
        a_row[i] = src;
        o_row[i] = dst;
    }
    __syncthreads();
    const size_t weight_rows = (size_t)(GATED ? 2 : 1) * N;
    const T* We = W + (size_t)expert * weight_rows * Kd;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if constexpr (sizeof(T) == 2) {
        const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
        const int g = lane >> 2, tg = lane & 3;
        float acc[NB][2][4][4];
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[b][i][j][c] = 0.0f;
        for (int k0 = 0; k0 < Kd; k0 += MOE_TK) {
            for (int idx = threadIdx.x; idx < MOE_TM * (MOE_TK / CHUNK); idx += blockDim.x) {
                const int r = idx / (MOE_TK / CHUNK), c = (idx % (MOE_TK / CHUNK)) * CHUNK;
                const int src = a_row[r];
                stage_chunk(&As[r][c], src >= 0 ? A + (size_t)src * lda : nullptr, k0 + c, Kd, vec);
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const int n = n0 + r;
                    stage_chunk(&Bs[b][r][c], n < N ? We + ((size_t)b * N + n) * Kd : nullptr, k0 + c, Kd, vec);
                }
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < MOE_TK; kk += 16) {
                uint32_t a[2][4];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int r = wm + i * 16 + g;
                    a[i][0] = *reinterpret_cast<const uint32_t*>(&As[r][kk + 2 * tg]);
                    a[i][1] = *reinterpret_cast<const uint32_t*>(&As[r + 8][kk + 2 * tg]);
                    a[i][2] = *reinterpret_cast<const uint32_t*>(&As[r][kk + 2 * tg + 8]);
                    a[i][3] = *reinterpret_cast<const uint32_t*>(&As[r + 8][kk + 2 * tg + 8]);
                }
#pragma unroll
                for (int b = 0; b < NB; ++b)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t bf[2];
                        const int n = wn + j * 8 + g;
                        bf[0] = *reinterpret_cast<const uint32_t*>(&Bs[b][n][kk + 2 * tg]);
                        bf[1] = *reinterpret_cast<const uint32_t*>(&Bs[b][n][kk + 2 * tg + 8]);
#pragma unroll
                        for (int i = 0; i < 2; ++i) mma_bf16_16816(acc[b][i][j], a[i], bf);
                    }
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = wm + i * 16 + g + half * 8;
                const int dst = o_row[r];
                if (dst < 0) continue;
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int n = n0 + wn + j * 8 + 2 * tg + c;
                        if (n >= N) continue;
                        if constexpr (GATED)
                            reinterpret_cast<T*>(out)[(size_t)dst * N + n] =
                                from_float<T>(expert_activation(acc[0][i][j][half * 2 + c], acc[1][i][j][half * 2 + c], limit, alpha, shift));
                        else
                            reinterpret_cast<float*>(out)[(size_t)dst * N + n] = acc[0][i][j][half * 2 + c];
                    }
            }
    } else {
        // 32-bit: thread (ty, tx) owns rows ty*4.. and columns tx, tx+8, ...
        const int ty = threadIdx.x >> 3, tx = threadIdx.x & 7;
        float acc[NB][4][8];
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[b][i][j] = 0.0f;
        for (int k0 = 0; k0 < Kd; k0 += MOE_TK) {
            for (int idx = threadIdx.x; idx < MOE_TM * (MOE_TK / CHUNK); idx += blockDim.x) {
                const int r = idx / (MOE_TK / CHUNK), c = (idx % (MOE_TK / CHUNK)) * CHUNK;
                const int src = a_row[r];
                stage_chunk(&As[r][c], src >= 0 ? A + (size_t)src * lda : nullptr, k0 + c, Kd, vec);
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const int n = n0 + r;
                    stage_chunk(&Bs[b][r][c], n < N ? We + ((size_t)b * N + n) * Kd : nullptr, k0 + c, Kd, vec);
                }
            }
            __syncthreads();
#pragma unroll 4
            for (int kk = 0; kk < MOE_TK; ++kk) {
                float av[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) av[i] = As[ty * 4 + i][kk];
#pragma unroll
                for (int b = 0; b < NB; ++b)
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float bv = Bs[b][tx + 8 * j][kk];
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[b][i][j] = fmaf(av[i], bv, acc[b][i][j]);
                    }
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int dst = o_row[ty * 4 + i];
            if (dst < 0) continue;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int n = n0 + tx + 8 * j;
                if (n >= N) continue;
                if constexpr (GATED)
                    reinterpret_cast<T*>(out)[(size_t)dst * N + n] = from_float<T>(expert_activation(acc[0][i][j], acc[NB - 1][i][j], limit, alpha, shift));
                else
                    reinterpret_cast<float*>(out)[(size_t)dst * N + n] = acc[0][i][j];
            }
        }
    }
}

// ------------------------------------------------------------------ few pairs an expert: the weights stream
// A decode step gives an expert a handful of tokens, and what counts is how fast its weight rows stream.
// Here the weight rows are the M side of the mma (16 rows a warp, 64 a block) and up to 8 pairs the N side, so no
// tensor-core work is spent on rows that are not there.  A lane fetches 16 bytes of two weight rows straight
// from global memory (a row gives 128 contiguous bytes per step) and 16 bytes of its pair's row from shared
// memory; the sum over k is taken in a permuted order that both operands share (columns tg*8+4j+{0..3} of a
// 32-column run feed the j-th mma), so no data is shuffled.  The next step's loads are issued before this
// step's products.  More than 8 pairs of a tile go in turns of 8 (the weights come from the L2 the second time).
#define SK_PAIRS 8
#define SK_FEATURES 64

template <bool GATED>
__global__ void __launch_bounds__(128)
moe_skinny_kernel(const __nv_bfloat16* __restrict__ A, int lda, const int* __restrict__ sorted, int top,
                  const __nv_bfloat16* __restrict__ W, int N, int Kd, int Kp, const int* __restrict__ tile_expert,
                  const int* __restrict__ tile_first, const int* __restrict__ tile_pairs, const int* __restrict__ num_tiles,
                  float limit, float alpha, float shift, int real_experts, void* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char sk_shared[];
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(sk_shared);  // [SK_PAIRS][Kp + 32]
    constexpr int NB = GATED ? 2 : 1;
    const int ldx = Kp + 32;  // rows fall on alternate halves of a 128-byte line: 16-byte reads of 8 rows do not collide
    pdl_wait();
    const int tile = blockIdx.x;
    if (tile >= *num_tiles) return;
    const int expert = tile_expert[tile], first = tile_first[tile], rows = tile_pairs[tile];
    if (expert >= real_experts) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tg = lane & 3;
    const int f0 = blockIdx.y * SK_FEATURES + warp * 16;
    const int r0 = f0 + g, r1 = f0 + g + 8;
    const __nv_bfloat16* We = W + (size_t)expert * NB * N * Kd;
    // rows beyond N read row 0 (their results are dropped)
    const __nv_bfloat16* w0[NB];
    const __nv_bfloat16* w1[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        w0[b] = We + ((size_t)b * N + (r0 < N ? r0 : 0)) * Kd;
        w1[b] = We + ((size_t)b * N + (r1 < N ? r1 : 0)) * Kd;
    }
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    for (int sub = 0; sub < rows; sub += SK_PAIRS) {
        const int np = min(SK_PAIRS, rows - sub);
        __syncthreads();
        for (int idx = threadIdx.x; idx < SK_PAIRS * (Kp / 8); idx += blockDim.x) {
            const int i = idx / (Kp / 8), c = (idx % (Kp / 8)) * 8;
            uint4 v = zero4;
            if (i < np && c < Kd) {
                const int place = first + sub + i;
                const int src = GATED ? sorted[place] / top : place;
                v = *reinterpret_cast<const uint4*>(A + (size_t)src * lda + c);
            }
            *reinterpret_cast<uint4*>(xs + (size_t)i * ldx + c) = v;
        }
        __syncthreads();
        float acc[NB][4];
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[b][c] = 0.0f;
        uint4 lo[NB][2], hi[NB][2], nlo[NB][2], nhi[NB][2];
        auto fetch = [&](int kc, uint4 (&dlo)[NB][2], uint4 (&dhi)[NB][2]) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int col = kc + half * 32 + tg * 8;
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    dlo[b][half] = col < Kd ? __ldg(reinterpret_cast<const uint4*>(w0[b] + col)) : zero4;
                    dhi[b][half] = col < Kd ? __ldg(reinterpret_cast<const uint4*>(w1[b] + col)) : zero4;
                }
            }
        };
        fetch(0, lo, hi);
        for (int kc = 0; kc < Kp; kc += 64) {
            if (kc + 64 < Kp) fetch(kc + 64, nlo, nhi);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint4 x = *reinterpret_cast<const uint4*>(xs + (size_t)g * ldx + kc + half * 32 + tg * 8);
                const uint32_t b0[2] = {x.x, x.y}, b1[2] = {x.z, x.w};
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const uint32_t a0[4] = {lo[b][half].x, hi[b][half].x, lo[b][half].y, hi[b][half].y};
                    const uint32_t a1[4] = {lo[b][half].z, hi[b][half].z, lo[b][half].w, hi[b][half].w};
                    mma_bf16_16816(acc[b], a0, b0);
                    mma_bf16_16816(acc[b], a1, b1);
                }
            }
            if (kc + 64 < Kp) {
#pragma unroll
                for (int b = 0; b < NB; ++b)
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        lo[b][half] = nlo[b][half];
                        hi[b][half] = nhi[b][half];
                    }
            }
        }
        // lane (g, tg) holds features r0 (c 0, 1) and r1 (c 2, 3) of pairs 2 tg and 2 tg + 1
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int feature = c < 2 ? r0 : r1;
            const int i = 2 * tg + (c & 1);
            if (feature >= N || i >= np) continue;
            const int place = first + sub + i;
            if constexpr (GATED)
                reinterpret_cast<__nv_bfloat16*>(out)[(size_t)place * N + feature] =
                    __float2bfloat16_rn(expert_activation(acc[0][c], acc[NB - 1][c], limit, alpha, shift));
            else
                reinterpret_cast<float*>(out)[(size_t)sorted[place] * N + feature] = acc[0][c];
        }
    }
}

template <typename TR, typename TO>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const TR* __restrict__ rows, const float* __restrict__ weights, const int* __restrict__ at, int K, int H,
                   TO* __restrict__ out, const int* __restrict__ ids, const TO* __restrict__ x, int real_experts,
                   const TO* __restrict__ extra, const float* __restrict__ extra_gate, int gate_stride) {
    pdl_wait();
    const int t = blockIdx.x;
    const float extra_weight = extra ? (extra_gate ? 1.0f / (1.0f + expf(-extra_gate[(size_t)t * gate_stride])) : 1.0f) : 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = 0.0f;
        for (int k = 0; k < K; ++k) {
            const size_t p = (size_t)t * K + k;
            const float w = weights ? weights[p] : 1.0f;
            if (ids && ids[p] >= real_experts)  // an identity expert: its output is the token's own row
                v += w * to_float(x[(size_t)t * H + i]);
            else
                v += w * to_float(rows[(at ? (size_t)at[p] : p) * H + i]);
        }
        if (extra) v += extra_weight * to_float(extra[(size_t)t * H + i]);
        out[(size_t)t * H + i] = from_float<TO>(v);
    }
}

// out[i] = src[rows ? rows[i] : i / div] * scale[index ? index[i] : i], in 32-bit with one rounding at the store
template <typename T>
__global__ void __launch_bounds__(256)
moe_scale_rows_kernel(const T* __restrict__ src, const int* __restrict__ rows, int div, const float* __restrict__ scale,
                      const int* __restrict__ index, T* __restrict__ out, int H) {
    pdl_wait();
    const int i = blockIdx.x;
    const T* from = src + (size_t)(rows ? rows[i] : i / div) * H;
    const float w = scale[index ? index[i] : i];
    for (int c = threadIdx.x; c < H; c += blockDim.x) out[(size_t)i * H + c] = from_float<T>(to_float(from[c]) * w);
}

KB_EXPORT int kb_moe_scale_rows(const void* src, int is_bf16, const int* rows, int div, const float* scale, const int* index, void* out,
                                int R, int H, cudaStream_t stream) {
    if (R == 0) return 0;
    if (!src || !scale || !out) return KB_ERR_NULL;
    if (H < 1 || (!rows && div < 1)) return KB_ERR_BAD_ARG;
    if (is_bf16)
        kb_launch(moe_scale_rows_kernel<__nv_bfloat16>, dim3(R), dim3(256), 0, stream, (const __nv_bfloat16*)src, rows, div, scale, index,
                  (__nv_bfloat16*)out, H);
    else
        kb_launch(moe_scale_rows_kernel<float>, dim3(R), dim3(256), 0, stream, (const float*)src, rows, div, scale, index, (float*)out, H);
    return kb_launch_result();
}

// Routing by scores: s = softmax(logits) over all n outputs; the choice runs on c = s + correction
// (the correction steers the choice only).  The outputs form `groups` equal runs of neighbours; a
// group's value is its largest c, the `keep` best groups stay (ties: the lower group) and the rest
// count as minus infinity.  The K largest c that stay are chosen (ties: the lower index); their
// weights are s * scale, not renormalised.  One warp a token; 32-bit.
template <typename TB>
__global__ void __launch_bounds__(128)
moe_route_scores_kernel(const float* __restrict__ logits, const TB* __restrict__ correction, int n, int K, int groups, int keep,
                        float scale, int sigmoid, int stride, int* __restrict__ ids, float* __restrict__ weights, int T) {
    extern __shared__ float route_shared[];  // per warp: s[n], c[n], group values [groups]
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    float* s = route_shared + (size_t)warp * (2 * n + groups);
    float* c = s + n;
    float* group_value = c + n;
    const float* z = logits + (size_t)t * stride;  // a row may hold further columns behind the n router outputs
    float top = -INFINITY;
    for (int e = lane; e < n; e += 32) top = fmaxf(top, z[e]);
    top = warp_max(top);
    float sum = 0.0f;
    for (int e = lane; e < n; e += 32) {
        const float p = sigmoid ? 1.0f / (1.0f + expf(-z[e])) : expf(z[e] - top);
        s[e] = p;
        sum += p;
    }
    sum = sigmoid ? 1.0f : warp_sum(sum);
    for (int e = lane; e < n; e += 32) {
        s[e] = s[e] / sum;
        c[e] = s[e] + (correction ? to_float(correction[e]) : 0.0f);
    }
    __syncwarp();
    const int per = n / groups;
    if (keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            float best = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, c[e]);
            group_value[g] = best;
        }
        __syncwarp();
        // group g stays if fewer than `keep` groups come before it in the order (value down, index up)
        for (int g = lane; g < groups; g += 32) {
            const float mine = group_value[g];
            int before = 0;
            for (int o = 0; o < groups; ++o) before += (group_value[o] > mine || (group_value[o] == mine && o < g)) ? 1 : 0;
            if (before >= keep)
                for (int e = g * per; e < (g + 1) * per; ++e) c[e] = -INFINITY;
        }
        __syncwarp();
    }
    float last_value = INFINITY;
    int last_id = -1;
    for (int k = 0; k < K; ++k) {
        float best = -INFINITY;
        int best_id = 0x7fffffff;
        for (int e = lane; e < n; e += 32) {
            const float v = c[e];
            const bool after = v < last_value || (v == last_value && e > last_id);
            if (after && (v > best || (v == best && e < best_id))) {
                best = v;
                best_id = e;
            }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, offset);
            const int other_id = __shfl_xor_sync(0xffffffffu, best_id, offset);
            if (other > best || (other == best && other_id < best_id)) {
                best = other;
                best_id = other_id;
            }
        }
        if (best_id >= n) best_id = 0;  // fewer than K outputs stayed: nothing sensible is left to choose
        if (lane == 0) {
            ids[(size_t)t * K + k] = best_id;
            weights[(size_t)t * K + k] = s[best_id] * scale;
        }
        last_value = best;
        last_id = best_id;
    }
}

KB_EXPORT int kb_moe_route_scores(const float* logits, const void* correction, int correction_is_bf16, int n, int K, int groups,
                                  int keep, float scale, int sigmoid, int stride, int* ids, float* weights, int T, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!logits || !ids || !weights) return KB_ERR_NULL;
    if (n < 1 || K < 1 || K > n || n > MOE_MAX_EXPERTS) return KB_ERR_UNSUPPORTED_SIZE;
    if (groups < 1 || n % groups != 0 || keep < 1 || keep > groups || K > keep * (n / groups) || stride < n) return KB_ERR_BAD_ARG;
    const size_t smem = (size_t)4 * (2 * n + groups) * sizeof(float);
    if (smem > 48 * 1024) return KB_ERR_UNSUPPORTED_SIZE;
    if (correction_is_bf16)
        kb_launch(moe_route_scores_kernel<__nv_bfloat16>, dim3((T + 3) / 4), dim3(128), smem, stream, logits, (const __nv_bfloat16*)correction,
                  n, K, groups, keep, scale, sigmoid, stride, ids, weights, T);
    else
        kb_launch(moe_route_scores_kernel<float>, dim3((T + 3) / 4), dim3(128), smem, stream, logits, (const float*)correction, n, K, groups,
                  keep, scale, sigmoid, stride, ids, weights, T);
    return kb_launch_result();
}

KB_EXPORT int kb_moe_route(const float* logits, const void* bias, int bias_is_bf16, int E, int K, int* ids, float* weights, int T,
                           cudaStream_t stream) {
    if (T == 0) return 0;
    if (!logits || !ids || !weights) return KB_ERR_NULL;
    if (E < 1 || K < 1 || K > E || K > MOE_MAX_TOP || E > MOE_MAX_EXPERTS) return KB_ERR_UNSUPPORTED_SIZE;
    if (bias_is_bf16)
        kb_launch(moe_route_kernel<__nv_bfloat16>, dim3((T + 3) / 4), dim3(128), 0, stream, logits, (const __nv_bfloat16*)bias, E, K, ids, weights, T);
    else
        kb_launch(moe_route_kernel<float>, dim3((T + 3) / 4), dim3(128), 0, stream, logits, (const float*)bias, E, K, ids, weights, T);
    return kb_launch_result();
}

KB_EXPORT int kb_moe_max_tiles(int pairs, int E) { return (pairs + MOE_TM - 1) / MOE_TM + E; }

KB_EXPORT int kb_moe_plan(const int* ids, int pairs, int E, int top, int* sorted, int* token_of, int* place_of, int* ends,
                          int* tile_expert, int* tile_first, int* tile_pairs, int* num_tiles, cudaStream_t stream) {
    if (pairs == 0) return 0;
    if (!ids || !sorted || !token_of || !place_of || !ends || !tile_expert || !tile_first || !tile_pairs || !num_tiles) return KB_ERR_NULL;
    if (E < 1 || E > MOE_MAX_EXPERTS || top < 1) return KB_ERR_UNSUPPORTED_SIZE;
    kb_launch(moe_plan_kernel, dim3(1), dim3(1024), 0, stream, ids, pairs, E, top, sorted, token_of, place_of, ends, tile_expert, tile_first,
              tile_pairs, num_tiles);
    return kb_launch_result();
}

KB_EXPORT int kb_moe_activation(const void* gate_up, void* y, int is_bf16, int rows, int F, float limit, float alpha, float shift,
                                cudaStream_t stream) {
    if (rows == 0) return 0;
    if (!gate_up || !y) return KB_ERR_NULL;
    const size_t total = (size_t)rows * F;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (is_bf16)
        kb_launch(moe_activation_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)y, F, limit, alpha, shift, total);
    else
        kb_launch(moe_activation_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gate_up, (float*)y, F, limit, alpha, shift, total);
    return kb_launch_result();
}

KB_EXPORT int kb_moe_grouped(const void* A, int lda, const int* sorted, int top, const void* W, int N, int Kd, int is_bf16,
                             int gated, const int* tile_expert, const int* tile_first, const int* tile_pairs,
                             const int* num_tiles, int max_tiles, float limit, float alpha, float shift, int real_experts, void* out,
                             cudaStream_t stream) {
    if (max_tiles == 0) return 0;
    if (!A || !sorted || !W || !tile_expert || !tile_first || !tile_pairs || !num_tiles || !out) return KB_ERR_NULL;
    if (N < 1 || Kd < 1 || top < 1) return KB_ERR_BAD_ARG;
    const int per16 = is_bf16 ? 8 : 4;
    const int vec = (Kd % per16 == 0 && lda % per16 == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0) ? 1 : 0;
    dim3 grid(max_tiles, (N + MOE_TN - 1) / MOE_TN);
#define LAUNCH(T, G)                                                                                                          \
    kb_launch(moe_grouped_kernel<T, G>, grid, dim3(128), 0, stream, (const T*)A, lda, sorted, top, (const T*)W, N, Kd, tile_expert, \
              tile_first, tile_pairs, num_tiles, limit, alpha, shift, real_experts, out, vec)
    if (is_bf16) {
        if (gated) LAUNCH(__nv_bfloat16, true); else LAUNCH(__nv_bfloat16, false);
    } else {
        if (gated) LAUNCH(float, true); else LAUNCH(float, false);
    }
#undef LAUNCH
    return kb_launch_result();
}

KB_EXPORT int kb_moe_skinny(const void* A, int lda, const int* sorted, int top, const void* W, int N, int Kd, int gated,
                            const int* tile_expert, const int* tile_first, const int* tile_pairs, const int* num_tiles,
                            int max_tiles, float limit, float alpha, float shift, int real_experts, void* out, cudaStream_t stream) {
    if (max_tiles == 0) return 0;
    if (!A || !sorted || !W || !tile_expert || !tile_first || !tile_pairs || !num_tiles || !out) return KB_ERR_NULL;
    if (N < 1 || Kd < 8 || top < 1 || Kd % 8 != 0 || lda % 8 != 0 || ((uintptr_t)A % 16) != 0 || ((uintptr_t)W % 16) != 0) return KB_ERR_BAD_ARG;
    const int Kp = (Kd + 63) / 64 * 64;
    const size_t smem = (size_t)SK_PAIRS * (Kp + 32) * sizeof(__nv_bfloat16);
    if (smem > 200 * 1024) return KB_ERR_UNSUPPORTED_SIZE;
    dim3 grid(max_tiles, (N + SK_FEATURES - 1) / SK_FEATURES);
    if (gated) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(moe_skinny_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kb_launch(moe_skinny_kernel<true>, grid, dim3(128), smem, stream, (const __nv_bfloat16*)A, lda, sorted, top, (const __nv_bfloat16*)W, N, Kd, Kp,
                  tile_expert, tile_first, tile_pairs, num_tiles, limit, alpha, shift, real_experts, out);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(moe_skinny_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kb_launch(moe_skinny_kernel<false>, grid, dim3(128), smem, stream, (const __nv_bfloat16*)A, lda, sorted, top, (const __nv_bfloat16*)W, N, Kd, Kp,
                  tile_expert, tile_first, tile_pairs, num_tiles, limit, alpha, shift, real_experts, out);
    }
    return kb_launch_result();
}

KB_EXPORT int kb_moe_combine(const void* rows, int rows_is_bf16, const float* weights, const int* at, int K, int H, void* out,
                             int out_is_bf16, int T, const int* ids, const void* x, int real_experts, const void* extra,
                             const float* extra_gate, int gate_stride, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!rows || !out || (ids && !x)) return KB_ERR_NULL;
#define LAUNCH(TR, TO)                                                                                                     \
    kb_launch(moe_combine_kernel<TR, TO>, dim3(T), dim3(256), 0, stream, (const TR*)rows, weights, at, K, H, (TO*)out, ids, \
              (const TO*)x, real_experts, (const TO*)extra, extra_gate, gate_stride)
    if (rows_is_bf16) {
        if (out_is_bf16) LAUNCH(__nv_bfloat16, __nv_bfloat16); else LAUNCH(__nv_bfloat16, float);
    } else {
        if (out_is_bf16) LAUNCH(float, __nv_bfloat16); else LAUNCH(float, float);
    }
#undef LAUNCH
    return kb_launch_result();
}
