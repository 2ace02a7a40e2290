// Routed experts: router scores, the plan of a step (which rows go to which expert), the gather that scales each
// expert's input by the router's weight, grouped matrix products over the rows sorted by expert, and the sum of a
// token's expert outputs.
//
//   s = sigmoid(z) (z: router logits, float32);  a token takes the `top` experts with the largest s (ties: lowest
//   index); its weight for expert e is s_e, not renormalised, and multiplies the expert's INPUT:
//       y = sum over chosen e of  Wdown_e (act(Wgate_e (s_e h)) * (Wup_e (s_e h)))
//
// Nothing here needs the host to know how many rows an expert got: the plan lives in device memory and the grouped
// product is launched for an upper bound of row tiles (tiles beyond the plan's count return at once), so the whole
// feed-forward can be recorded into a CUDA graph.  Every output element adds its products in the order k = 0, 1, ...,
// and a token's expert outputs are added in the order of its choices, so a row's result does not depend on the batch.
#include "common.cuh"

namespace iian {

constexpr int kTileM = 64, kTileN = 64, kTileK = 16;

// One warp per token.  ids / wts: [N, top].
// mode 0: the weight of a chosen expert is sigmoid(logit); mode 1: the softmax over the chosen logits only.  bias (optional,
// float32 [E]) is added to the logits before anything else.
__global__ void moe_route_kernel(const float * __restrict__ logits, long long ld, int E, int top, int * __restrict__ ids,
                                 float * __restrict__ wts, int N, const float * __restrict__ bias, int mode) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long t = (long long) blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= N) return;
    const float * z = logits + t * ld;
    unsigned long long taken_lo = 0;          // experts already chosen, for the lanes' own candidates (by slot i / 32)
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane, i = 0; e < E; e += 32, i++) {
            if (i < 64 && ((taken_lo >> i) & 1ull)) continue;
            const float v = bias != nullptr ? z[e] + bias[e] : z[e];
            if (v > best || (v == best && e < best_e)) { best = v; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
        }
        if (best_e != 0x7fffffff && (best_e & 31) == lane) taken_lo |= 1ull << (best_e >> 5);
        if (lane == 0) {
            ids[t * top + k] = best_e == 0x7fffffff ? 0 : best_e;
            wts[t * top + k] = best_e == 0x7fffffff ? (mode == 1 ? -INFINITY : 0.0f) : mode == 1 ? best : 1.0f / (1.0f + expf(-best));
        }
    }
    if (mode == 1 && lane == 0) {      // the chosen logits came in falling order: the first is their maximum
        const float mx = wts[t * top];
        float sum = 0.0f;
        for (int k = 0; k < top; k++) {
            const float e = expf(wts[t * top + k] - mx);
            wts[t * top + k] = e;
            sum += e;
        }
        for (int k = 0; k < top; k++) wts[t * top + k] /= sum;
    }
}

// Routing without a router: row `tokens[t]` of a table [V, top] names the token's experts (the entries of a row differ);
// each weighs `weight`.  rows (optional): the token of output row r is tokens[rows[r]].
__global__ void moe_table_route_kernel(const int * __restrict__ tokens, const int * __restrict__ rows, const int * __restrict__ table,
                                       int V, int E, int top, int * __restrict__ ids, float * __restrict__ wts, float weight, int N,
                                       int n_tokens) {
    pdl_wait();
    pdl_launch_dependents();
    const long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long) N * top) return;
    const int r = (int) (i / top), k = (int) (i - (long long) r * top);
    int t = rows != nullptr ? rows[r] : r;
    t = min(max(t, 0), n_tokens - 1);
    const int tok = min(max(tokens[t], 0), V - 1);          // never read outside the table
    ids[i] = min(max(table[(size_t) tok * top + k], 0), E - 1);
    wts[i] = weight;
}

// One block.  offsets: [E + 1] first sorted row of each expert; pos: [M] sorted row of each (token, choice);
// tiles: [2 * max_tiles + 1]: n_tiles, then (expert, first row) per row tile of tile_rows rows.
__global__ void moe_plan_kernel(const int * __restrict__ ids, int M, int E, int * __restrict__ offsets, int * __restrict__ pos,
                                int * __restrict__ tiles, int max_tiles, int tile_rows) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ int sm[];               // counts [E], cursor [E]
    int * counts = sm;
    int * cursor = sm + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < M; i += blockDim.x) atomicAdd(&counts[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0, nt = 0;
        for (int e = 0; e < E; e++) {
            offsets[e] = run;
            cursor[e] = run;
            for (int r = 0; r < counts[e] && nt < max_tiles; r += tile_rows) {
                tiles[1 + 2 * nt] = e;
                tiles[2 + 2 * nt] = run + r;
                nt++;
            }
            run += counts[e];
        }
        offsets[E] = run;
        tiles[0] = nt;
    }
    __syncthreads();
    // the order of an expert's rows among themselves is left to the atomics: a row's arithmetic does not depend on it
    for (int i = threadIdx.x; i < M; i += blockDim.x) pos[i] = atomicAdd(&cursor[ids[i]], 1);
}

// xs[pos[t * top + k], :] = A(w[t, k] * h[t, :]);  rows[pos] = t * top + k
template <typename A>
__global__ void moe_scatter_kernel(const A * __restrict__ h, const int * __restrict__ pos, const float * __restrict__ wts,
                                   A * __restrict__ xs, int W, int top) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = blockIdx.x;              // (token, choice)
    const size_t t = i / top;
    const float w = wts != nullptr ? wts[i] : 1.0f;
    const A * src = h + t * W;
    A * dst = xs + (size_t) pos[i] * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) dst[c] = from_f32<A>(w * to_f32(src[c]));
}

// out[t, :] = sum_k [wts[t, k] *] ys[pos[t * top + k], :]  (k ascending)
template <typename A>
__global__ void moe_combine_kernel(const A * __restrict__ ys, const int * __restrict__ pos, const float * __restrict__ wts,
                                   A * __restrict__ out, int W, int top, const A * add) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float acc = 0.0f;
        for (int k = 0; k < top; k++) {
            const float y = to_f32(ys[(size_t) pos[t * top + k] * W + c]);
            acc += wts != nullptr ? wts[t * top + k] * y : y;
        }
        if (add != nullptr) acc += to_f32(add[t * W + c]);        // may be `out` itself: read before it is written
        out[t * W + c] = from_f32<A>(acc);
    }
}

// act 0: silu(g) * u; 1: gelu_tanh(g) * u; 2: with g' = min(g, limit), u' = clamp(u, -limit, limit):
// g' sigmoid(1.702 g') (u' + 1)
__device__ __forceinline__ float moe_gated(float g, float u, int act, float limit) {
    if (act == 0) return g / (1.0f + expf(-g)) * u;
    if (act == 2) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
    }
    const float t = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.0f + tanhf(t)) * u;
}

// Rows [r0, r0 + rows) of x (sorted by expert) times expert e's weight block w[e] ([n_out, K], row-major):
// out[r, m] = sum_k x[r, k] * w[e][m, k];  with GATED, w2[e] is a second block of the same shape and
// out[r, m] = act(x . w[e][m]) * (x . w2[e][m]); with GATED and w2 == w, an expert's block holds both, 2 n_out rows in
// groups of 16: 8 rows of the first, then the 8 rows of the second for the same features.
template <typename A, typename WT, bool GATED>
__global__ void __launch_bounds__(256) moe_grouped_gemm_kernel(const A * __restrict__ x, const WT * __restrict__ w,
                                                               const WT * __restrict__ w2, A * __restrict__ out,
                                                               const int * __restrict__ offsets, const int * __restrict__ tiles,
                                                               int n_out, int K, int act, float limit) {
    pdl_wait();
    pdl_launch_dependents();
    if ((int) blockIdx.y >= tiles[0]) return;
    const int e = tiles[1 + 2 * blockIdx.y], r0 = tiles[2 + 2 * blockIdx.y];
    const int r_end = min(offsets[e + 1], r0 + kTileM);
    __shared__ float xs[kTileK][kTileM + 4];
    __shared__ float ws[kTileK][kTileN + 4];
    __shared__ float w2s[GATED ? kTileK : 1][kTileN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.x * kTileN;
    const int tx = tid % 16, ty = tid / 16;
    const int lrow = tid / 4, lk = (tid % 4) * 4;
    const bool il = GATED && w2 == w;
    const WT * we = w + (size_t) e * n_out * K * (il ? 2 : 1);
    const WT * w2e = GATED ? (il ? we + (size_t) 8 * K : w2 + (size_t) e * n_out * K) : nullptr;
    float acc[4][4], acc2[GATED ? 4 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            acc[i][j] = 0.0f;
            if (GATED) acc2[i][j] = 0.0f;
        }
    for (int k0 = 0; k0 < K; k0 += kTileK) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int k = k0 + lk + q;
            const int r = r0 + lrow, m = m0 + lrow;
            xs[lk + q][lrow] = (r < r_end && k < K) ? to_f32(x[(size_t) r * K + k]) : 0.0f;
            const size_t wr = il ? (size_t) (m / 8) * 16 + m % 8 : (size_t) m;       // row of the weight block
            ws[lk + q][lrow] = (m < n_out && k < K) ? to_f32(we[wr * K + k]) : 0.0f;
            if (GATED) w2s[lk + q][lrow] = (m < n_out && k < K) ? to_f32(w2e[wr * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kTileK; k++) {
            float a[4], b[4], b2[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                b[j] = ws[k][tx * 4 + j];
                if (GATED) b2[j] = w2s[k][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (GATED) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = r0 + ty * 4 + i;
        if (r >= r_end) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int m = m0 + tx * 4 + j;
            if (m >= n_out) continue;
            float v = acc[i][j];
            // the gate and up products are rounded to the activation type first, as separate products would leave them
            if (GATED) v = moe_gated(to_f32(from_f32<A>(v)), to_f32(from_f32<A>(acc2[i][j])), act, limit);
            out[(size_t) r * n_out + m] = from_f32<A>(v);
        }
    }
}

}  // namespace iian

using namespace iian;

IIAN_API int iian_moe_tile_rows() { return kTileM; }

// logits f32 (row stride ld) -> ids i32 [N, top], wts f32 [N, top]
IIAN_API int iian_moe_route(const float * logits, long long ld, int E, int top, int * ids, float * wts, int N, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (E <= 0 || top <= 0 || top > E || E > 2048) return IIAN_ERR_SHAPE;
    const int warps = 4;
    return iian_launch(moe_route_kernel, dim3((N + warps - 1) / warps), dim3(warps * 32), 0, stream, logits, ld, E, top, ids, wts, N,
                       (const float *) nullptr, 0);
}

// The same with a bias on the logits (float32 [E] or null) and the weights as the softmax over the chosen logits only.
IIAN_API int iian_moe_route_softmax(const float * logits, long long ld, const float * bias, int E, int top, int * ids, float * wts,
                                    int N, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (E <= 0 || top <= 0 || top > E || E > 2048) return IIAN_ERR_SHAPE;
    const int warps = 4;
    return iian_launch(moe_route_kernel, dim3((N + warps - 1) / warps), dim3(warps * 32), 0, stream, logits, ld, E, top, ids, wts, N,
                       bias, 1);
}

// tokens i32 [n_tokens], rows i32 [N] or null (then N == n_tokens), table i32 [V, top] -> ids i32 [N, top], wts f32 [N, top]
IIAN_API int iian_moe_table_route(const int * tokens, const int * rows, const int * table, int V, int E, int top, int * ids,
                                  float * wts, float weight, int N, int n_tokens, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (E <= 0 || top <= 0 || top > E || E > 2048 || V <= 0 || n_tokens <= 0) return IIAN_ERR_SHAPE;
    const long long total = (long long) N * top;
    return iian_launch(moe_table_route_kernel, dim3((unsigned) ((total + 255) / 256)), dim3(256), 0, stream, tokens, rows, table, V, E,
                       top, ids, wts, weight, N, n_tokens);
}

// ids [M] -> offsets [E + 1], pos [M], tiles [1 + 2 * max_tiles]
IIAN_API int iian_moe_plan(const int * ids, int M, int E, int * offsets, int * pos, int * tiles, int max_tiles, int tile_rows,
                           cudaStream_t stream) {
    if (M <= 0) return IIAN_OK;
    if (E <= 0 || E > 2048 || tile_rows <= 0 || max_tiles < (M + tile_rows - 1) / tile_rows + E) return IIAN_ERR_SHAPE;
    return iian_launch(moe_plan_kernel, dim3(1), dim3(1024), (size_t) 2 * E * sizeof(int), stream, ids, M, E, offsets, pos, tiles,
                       max_tiles, tile_rows);
}

IIAN_API int iian_moe_scatter(const void * h, const int * pos, const float * wts, void * xs, int act_dtype, int N, int W, int top,
                              cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    const int threads = W >= 1024 ? 256 : 128;
    const unsigned blocks = (unsigned) ((size_t) N * top);
    if (act_dtype == IIAN_F32) return iian_launch(moe_scatter_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float *) h, pos, wts, (float *) xs, W, top);
    if (act_dtype == IIAN_BF16) return iian_launch(moe_scatter_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16 *) h, pos, wts, (__nv_bfloat16 *) xs, W, top);
    return IIAN_ERR_DTYPE;
}

// wts: f32 [N, top], the weight of each expert's OUTPUT in the sum, or null (plain sum); add: A [N, W] or null, rows added
// after the experts' sum (an expert every token uses); it may be `out`.
IIAN_API int iian_moe_combine_add(const void * ys, const int * pos, const float * wts, const void * add, void * out, int act_dtype,
                                  int N, int W, int top, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    const int threads = W >= 1024 ? 256 : 128;
    if (act_dtype == IIAN_F32) return iian_launch(moe_combine_kernel<float>, dim3(N), dim3(threads), 0, stream, (const float *) ys, pos, wts, (float *) out, W, top, (const float *) add);
    if (act_dtype == IIAN_BF16) return iian_launch(moe_combine_kernel<__nv_bfloat16>, dim3(N), dim3(threads), 0, stream, (const __nv_bfloat16 *) ys, pos, wts, (__nv_bfloat16 *) out, W, top, (const __nv_bfloat16 *) add);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_moe_combine_weighted(const void * ys, const int * pos, const float * wts, void * out, int act_dtype, int N, int W,
                                       int top, cudaStream_t stream) {
    return iian_moe_combine_add(ys, pos, wts, nullptr, out, act_dtype, N, W, top, stream);
}

IIAN_API int iian_moe_combine(const void * ys, const int * pos, void * out, int act_dtype, int N, int W, int top, cudaStream_t stream) {
    return iian_moe_combine_weighted(ys, pos, nullptr, out, act_dtype, N, W, top, stream);
}

// x [M, K] sorted by expert; w (and w2, for the gated form) [E, n_out, K]; out [M, n_out]; act: 0 silu, 1 gelu (tanh).
// w2 == w: the gated form over blocks [E, 2 n_out, K] that hold both matrices interleaved in groups of 8 rows.
// The plan's row tiles must be of iian_moe_tile_rows() rows.  act 2 (clamped, see moe_gated) takes `limit`.
IIAN_API int iian_moe_grouped_gemm_act(const void * x, const void * w, const void * w2, void * out, const int * offsets,
                                       const int * tiles, int max_tiles, int act_dtype, int w_dtype, int n_out, int K, int act,
                                       float limit, cudaStream_t stream) {
    if (max_tiles <= 0 || n_out <= 0) return IIAN_OK;
    if (K <= 0 || max_tiles > 65535) return IIAN_ERR_SHAPE;
    dim3 grid((n_out + kTileN - 1) / kTileN, max_tiles);
    typedef __nv_bfloat16 bf;
#define IIAN_MOE(AT, WT)                                                                                                     \
    do {                                                                                                                     \
        if (w2 != nullptr)                                                                                                   \
            return iian_launch(moe_grouped_gemm_kernel<AT, WT, true>, grid, dim3(256), 0, stream, (const AT *) x, (const WT *) w, \
                               (const WT *) w2, (AT *) out, offsets, tiles, n_out, K, act, limit);                           \
        return iian_launch(moe_grouped_gemm_kernel<AT, WT, false>, grid, dim3(256), 0, stream, (const AT *) x, (const WT *) w, \
                           (const WT *) w2, (AT *) out, offsets, tiles, n_out, K, act, limit);                               \
    } while (0)
    if (act_dtype == IIAN_F32 && w_dtype == IIAN_F32) IIAN_MOE(float, float);
    if (act_dtype == IIAN_BF16 && w_dtype == IIAN_BF16) IIAN_MOE(bf, bf);
#undef IIAN_MOE
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_moe_grouped_gemm(const void * x, const void * w, const void * w2, void * out, const int * offsets, const int * tiles,
                                   int max_tiles, int act_dtype, int w_dtype, int n_out, int K, int act, cudaStream_t stream) {
    return iian_moe_grouped_gemm_act(x, w, w2, out, offsets, tiles, max_tiles, act_dtype, w_dtype, n_out, K, act, 0.0f, stream);
}
