// A recurrence over a matrix-valued state, shared by the mixers whose memory is one matrix S [D, V] per
// head and request, kept in 32-bit and rewritten by every token:
//
//     S <- g S + k u^T,    o = S^T q        (o sees the token's own write)
//
//   DELTA:    u = beta (v - (g S)^T k)      the delta rule: what is written is the part of v the decayed memory lacks
//   !DELTA:   u = beta v                    a plain outer-product write (a selective state-space layer: k = B, q = C,
//                                           v = x, beta = the step size)
//   CHANNEL:  g is a row of D numbers a token and head (one decay a key channel, acting on the rows of S)
//   !CHANNEL: g is one number a token and head
//
// With a = S^T (g k) and b = S^T (g q) of the OLD S:  u = beta (v - a),  o = b + (k.q) u,  S = g S + k u^T,
// which is the recurrence with one pass over S for the dots and one for the update.  Without the delta u does
// not depend on S, the state's chain is one multiply-add a token, and the loop over tokens is unrolled so that the
// read-outs' butterflies overlap.
//
// One block per (request, head, group of columns of S); columns are independent of one another, LANES lanes
// own a column (a lane holds D/LANES of its entries in registers), the two dot products of a token meet in one
// butterfly, and the next chunk's rows are fetched while this chunk is walked.  Every sum runs in an order that
// depends on the sizes alone, never on the batch or on how a prompt was cut: tokens are staged in chunks, but a
// chunk's edge changes no arithmetic.  The state is stored column by column ([heads, V, D]).
#pragma once
#include "common.cuh"

#define LR_WARPS 8
#define LR_MAX_TAPS 16

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float a) { return a > 20.0f ? a : log1pf(expf(a)); }

// input of a causal convolution `back` tokens before token t (offset o within its row's portion): in the step's
// rows, or among the request's kept inputs ([n - 1, C], oldest first)
template <typename TA>
__device__ __forceinline__ float conv_input(const TA* __restrict__ proj, int stride, const float* __restrict__ kept,
                                            int C, int n, int t, int o, int back, int c) {
    if (o - back >= 0) return to_float(proj[(size_t)(t - back) * stride + c]);
    return kept[(size_t)((n - 1) + (o - back)) * C + c];
}

// per request: the last (n - 1) inputs of the step become the kept inputs; a thread reads all it needs of a
// (request, channel) before it writes
template <typename TA>
__global__ void __launch_bounds__(128)
conv_state_kernel(const TA* __restrict__ proj, int stride, float* __restrict__ conv_state, int n, int C,
                  const int* __restrict__ qo_indptr, const int* __restrict__ state_slots) {
    const int row = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t0 = qo_indptr[row];
    const int count = qo_indptr[row + 1] - t0;
    float* kept = conv_state + (size_t)state_slots[row] * (n - 1) * C;
    pdl_wait();
    if (c >= C || count < 1) return;
    float next[LR_MAX_TAPS];
#pragma unroll
    for (int i = 0; i < LR_MAX_TAPS; ++i) {
        if (i < n - 1) {
            const int off = count - (n - 1) + i;
            next[i] = off >= 0 ? to_float(proj[(size_t)(t0 + off) * stride + c]) : kept[(size_t)((n - 1) + off) * C + c];
        }
    }
#pragma unroll
    for (int i = 0; i < LR_MAX_TAPS; ++i)
        if (i < n - 1) kept[(size_t)i * C + c] = next[i];
}

static inline int launch_conv_state(const void* proj, int stride, int is_bf16, float* conv_state, int n, int C, const int* qo_indptr,
                                    const int* state_slots, int num_rows, cudaStream_t stream) {
    dim3 grid(num_rows, (C + 127) / 128);
    if (is_bf16)
        kb_launch(conv_state_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)proj, stride, conv_state, n, C, qo_indptr, state_slots);
    else
        kb_launch(conv_state_kernel<float>, grid, dim3(128), 0, stream, (const float*)proj, stride, conv_state, n, C, qo_indptr, state_slots);
    return kb_launch_result();
}

// tokens staged at a time: what fits 36 KB of shared memory with `arrays` staged rows of LD floats a token
__host__ __device__ constexpr int lr_chunk(int LD, int arrays) {
    return arrays * 16 * LD * 4 <= 36864 ? 16 : (arrays * 8 * LD * 4 <= 36864 ? 8 : 4);
}

template <int DPT, int LANES, bool PREFETCH, bool DELTA, bool CHANNEL>
__global__ void __launch_bounds__(32 * LR_WARPS)
linear_recurrence_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vv,
                         const float* __restrict__ beta, const float* __restrict__ decay, float* __restrict__ states,
                         const int* __restrict__ qo_indptr, const int* __restrict__ state_slots, int KH, int D, int H, int V,
                         float* __restrict__ out) {
    constexpr int LD = LANES * DPT;               // entries of a key or query row as staged (zeros beyond D)
    constexpr int PER_WARP = 32 / LANES;          // columns of S a warp owns
    constexpr int COLS = LR_WARPS * PER_WARP;     // columns a block owns
    constexpr int CHUNK = lr_chunk(LD, CHANNEL ? 3 : 2);
    constexpr int GD = CHANNEL ? LD : 1;
    __shared__ __align__(16) float ks[CHUNK][LD];
    __shared__ __align__(16) float qs[CHUNK][LD];
    __shared__ __align__(16) float gcs[CHUNK][GD];  // CHANNEL: a token's decays a key channel
    __shared__ float vs[CHUNK][COLS];
    __shared__ float bs[CHUNK], gs[CHUNK], kqs[CHUNK];
    const int row = blockIdx.x, h = blockIdx.y;
    const int col0 = blockIdx.z * COLS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int part = lane % LANES;                    // this lane holds entries part, part + LANES, ... of its column
    const int local = warp * PER_WARP + lane / LANES;  // its column among the block's
    const int col = col0 + local;
    const int kh = h / (H / KH);
    const int t0 = qo_indptr[row], t1 = qo_indptr[row + 1];
    float* Sg = states + (((size_t)state_slots[row] * H + h) * V + (col < V ? col : 0)) * D;
    pdl_wait();
    float S[DPT];
#pragma unroll
    for (int m = 0; m < DPT; ++m) {
        const int i = m * LANES + part;
        S[m] = (i < D && col < V) ? Sg[i] : 0.0f;
    }
    // The next chunk's rows are fetched into registers while this chunk's tokens are walked, and put
    // into shared memory behind the barrier that ends the walk: the loads' latency is off the chain.
    // (A step of single tokens has no next chunk, and runs leaner without: PREFETCH is off for it.)
    constexpr int THREADS = 32 * LR_WARPS;
    constexpr int NP = PREFETCH ? CHUNK * LD / THREADS : 1;                    // key (and query) entries a thread fetches a chunk
    constexpr int NV = PREFETCH ? (CHUNK * COLS + THREADS - 1) / THREADS : 1;  // value entries
    constexpr int NG = CHANNEL ? NP : 1;
    float pk[NP], pq[NP], pc[NG], pv[NV], pb = 0.0f, pg = 0.0f;
    auto fetch = [&](int c0) {
        const int nt = min(CHUNK, t1 - c0);
#pragma unroll
        for (int j = 0; j < NP; ++j) {
            const int idx = j * THREADS + threadIdx.x;
            const int tt = idx / LD, i = idx % LD;
            const bool live = tt < nt && i < D;
            const size_t src = ((size_t)(c0 + tt) * KH + kh) * D + i;
            pk[j] = live ? kn[src] : 0.0f;
            pq[j] = live ? qn[src] : 0.0f;
            if constexpr (CHANNEL) pc[j] = live ? decay[((size_t)(c0 + tt) * H + h) * D + i] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int idx = j * THREADS + threadIdx.x;
            const int tt = idx / COLS, c = idx % COLS;
            pv[j] = (tt < nt && col0 + c < V) ? vv[((size_t)(c0 + tt) * H + h) * V + col0 + c] : 0.0f;
        }
        if (threadIdx.x < nt) {
            pb = beta[(size_t)(c0 + threadIdx.x) * H + h];
            if constexpr (!CHANNEL) pg = decay[(size_t)(c0 + threadIdx.x) * H + h];
        }
    };
    if (PREFETCH && t0 < t1) fetch(t0);
    for (int c0 = t0; c0 < t1; c0 += CHUNK) {
        const int nt = min(CHUNK, t1 - c0);
        __syncthreads();
        if constexpr (PREFETCH) {
#pragma unroll
            for (int j = 0; j < NP; ++j) {
                const int idx = j * THREADS + threadIdx.x;
                ks[idx / LD][idx % LD] = pk[j];
                qs[idx / LD][idx % LD] = pq[j];
                if constexpr (CHANNEL) gcs[idx / LD][idx % LD] = pc[j];
            }
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int idx = j * THREADS + threadIdx.x;
                if (idx < CHUNK * COLS) vs[idx / COLS][idx % COLS] = pv[j];
            }
            if (threadIdx.x < CHUNK) {
                bs[threadIdx.x] = pb;
                gs[threadIdx.x] = pg;
            }
        } else {
            for (int idx = threadIdx.x; idx < nt * LD; idx += blockDim.x) {
                const int tt = idx / LD, i = idx % LD;
                const size_t src = ((size_t)(c0 + tt) * KH + kh) * D + i;
                ks[tt][i] = i < D ? kn[src] : 0.0f;
                qs[tt][i] = i < D ? qn[src] : 0.0f;
                if constexpr (CHANNEL) gcs[tt][i] = i < D ? decay[((size_t)(c0 + tt) * H + h) * D + i] : 0.0f;
            }
            for (int idx = threadIdx.x; idx < nt * COLS; idx += blockDim.x) {
                const int tt = idx / COLS, j = idx % COLS;
                vs[tt][j] = col0 + j < V ? vv[((size_t)(c0 + tt) * H + h) * V + col0 + j] : 0.0f;
            }
            if (threadIdx.x < nt) {
                bs[threadIdx.x] = beta[(size_t)(c0 + threadIdx.x) * H + h];
                if constexpr (!CHANNEL) gs[threadIdx.x] = decay[(size_t)(c0 + threadIdx.x) * H + h];
            }
        }
        __syncthreads();
        if (PREFETCH && c0 + CHUNK < t1) fetch(c0 + CHUNK);
        for (int tt = warp; tt < nt; tt += LR_WARPS) {
            float dot = 0.0f;
            for (int i = lane; i < LD; i += 32) dot += ks[tt][i] * qs[tt][i];
            dot = warp_sum(dot);
            if (lane == 0) kqs[tt] = dot;
        }
        __syncthreads();
        const bool upper = (part & (LANES / 2)) != 0;
        if constexpr (!DELTA) {
            // Without the delta what is written does not depend on S: the state's chain is one multiply-add a token, and
            // the read-outs' sums hang off it.  Four tokens are unrolled so that their butterflies are in flight together.
#pragma unroll 4
            for (int tt = 0; tt < nt; ++tt) {
                const float g = gs[tt];
                const float u = bs[tt] * vs[tt][local];
                float b = 0.0f;
#pragma unroll
                for (int m = 0; m < DPT; ++m) {
                    b = fmaf(S[m], qs[tt][m * LANES + part], b);
                    S[m] = fmaf(ks[tt][m * LANES + part], u, g * S[m]);
                }
#pragma unroll
                for (int offset = LANES / 2; offset > 0; offset >>= 1) b += __shfl_xor_sync(0xffffffffu, b, offset);
                if (part == 0 && col < V) out[((size_t)(c0 + tt) * H + h) * V + col] = g * b + kqs[tt] * u;
            }
            continue;
        }
#pragma unroll 4
        for (int tt = 0; tt < nt; ++tt) {  // unrolled so that the next tokens' shared loads are issued ahead of this token's chain
            float kv[DPT];
            float sg[CHANNEL ? DPT : 1];
            float a = 0.0f, b = 0.0f;
#pragma unroll
            for (int m = 0; m < DPT; ++m) {
                kv[m] = ks[tt][m * LANES + part];
                if constexpr (CHANNEL) {
                    sg[m] = S[m] * gcs[tt][m * LANES + part];
                    a = fmaf(sg[m], kv[m], a);
                    b = fmaf(sg[m], qs[tt][m * LANES + part], b);
                } else {
                    a = fmaf(S[m], kv[m], a);
                    b = fmaf(S[m], qs[tt][m * LANES + part], b);
                }
            }
            // Both sums in one butterfly: the first exchange leaves the lower half of a column's lanes with the
            // halves' sum of a and the upper half with that of b; the later stages add within each half.
            const float given = __shfl_xor_sync(0xffffffffu, upper ? a : b, LANES / 2);
            float z = (upper ? b : a) + given;
#pragma unroll
            for (int offset = LANES / 4; offset > 0; offset >>= 1) z += __shfl_xor_sync(0xffffffffu, z, offset);
            a = __shfl_sync(0xffffffffu, z, lane & ~(LANES - 1));  // every lane needs a; b stays with the upper half
            const float g = CHANNEL ? 1.0f : gs[tt];
            const float u = bs[tt] * (vs[tt][local] - g * a);
#pragma unroll
            for (int m = 0; m < DPT; ++m) {
                if constexpr (CHANNEL) S[m] = fmaf(kv[m], u, sg[m]);
                else S[m] = fmaf(kv[m], u, g * S[m]);
            }
            if (part == LANES / 2 && col < V) out[((size_t)(c0 + tt) * H + h) * V + col] = g * z + kqs[tt] * u;
        }
    }
#pragma unroll
    for (int m = 0; m < DPT; ++m) {
        const int i = m * LANES + part;
        if (i < D && col < V) Sg[i] = S[m];
    }
}

// decay: [tokens, H] (!CHANNEL) or [tokens, H, D] (CHANNEL).  states: [slots, H, V, D].
template <bool DELTA, bool CHANNEL>
static int launch_linear_recurrence(const float* qn, const float* kn, const float* vv, const float* beta, const float* decay,
                                    float* states, const int* qo_indptr, const int* state_slots, int KH, int D, int H, int V,
                                    float* out, int num_rows, int single_tokens, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    if (!qn || !kn || !vv || !beta || !decay || !states || !qo_indptr || !state_slots || !out) return KB_ERR_NULL;
    if (D < 1 || D > 512 || KH < 1 || H % KH != 0 || V < 1 || H > 65535) return KB_ERR_UNSUPPORTED_SIZE;
    // Sixteen lanes a column whatever the step holds, so that a sum's order never depends on the batch
    // (measured at dim 128, 16 heads, vdim 128: one row of 2,048 tokens 695 us against 742 at 32 lanes and 788
    // at 8; four rows of 512 tokens 430 against 529 and 278; 64 rows of one token 31 against 41 at 32).
    constexpr int LANES = 16;
    const int cols = LR_WARPS * (32 / LANES);
    dim3 grid(num_rows, H, (V + cols - 1) / cols);
    const dim3 block(32 * LR_WARPS);
#define LR_LAUNCH(DPT, PF) kb_launch(linear_recurrence_kernel<DPT, LANES, PF, DELTA, CHANNEL>, grid, block, 0, stream, qn, kn, vv, beta, decay, states, qo_indptr, state_slots, KH, D, H, V, out)
#define LR_PICK(PF)                                                                                                           \
    do {                                                                                                                      \
        if (D <= 32) LR_LAUNCH(2, PF); else if (D <= 64) LR_LAUNCH(4, PF); else if (D <= 128) LR_LAUNCH(8, PF);               \
        else if (D <= 256) LR_LAUNCH(16, PF); else LR_LAUNCH(32, PF);                                                         \
    } while (0)
    if (single_tokens) LR_PICK(false); else LR_PICK(true);
#undef LR_PICK
#undef LR_LAUNCH
    return kb_launch_result();
}
