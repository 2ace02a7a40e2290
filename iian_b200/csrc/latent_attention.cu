// Attention over a cached low-rank latent (general form: any element type and sizes).
//
// Per token the cache holds ONE row of `rank + rot` numbers: the normalised latent c (rank) and a rotated key part
// shared by all heads (rot).  With the per-head up-projections folded to the query side, head h scores key j as
//     s_j = (qa_h . c_j + qr_h . kr_j) * scale,     qa_h = Wuk_h^T q_h   (the query moved into latent space)
// and its output is  o_h = Wuv_h (sum_j p_j c_j):  every head reads the same cache row, keys and values are never
// expanded.  The softmax may carry a sink: a number per head that joins the denominator (exp(sink_h), counted once,
// not scaled) without a key or a value.  Key j is visible to a query at position p iff j <= p and (window == 0 or
// p - j < window).
//
// Kernels:
//   latent_prep      per token: RMS norm of the latent (float32 sums), rotation of the shared key part and of the
//                    rotated part of every query head (frequencies and angles in float64, so they are at least as
//                    exact as 32-bit ones at any position), write of the cache row, copy of the rotated query parts
//                    into the attention's query rows
//   head_linear      per token and head a small matrix product with that head's block of a stacked weight, in either
//                    orientation (reduce over the weight's rows, or over its columns)
//   latent_attention one warp per (token, head); keys in tiles of 32 that start at multiples of 32 of the ABSOLUTE key
//                    position, so the order of every sum depends on the token's own position only
#include "common.cuh"

namespace iian {

constexpr int kLatWarps = 4;
constexpr int kLatMaxRank = 1024;
constexpr int kLatMaxWidth = 1536;       // rank + rot

// Entry i of a vector after the rotation of its first rot_dims entries.  style 0 pairs entry i with entry i + rot_dims / 2,
// style 1 pairs entry 2 i with entry 2 i + 1; pair number n turns by the angle whose cos and sin are cs_sn[2 n], [2 n + 1].
template <typename A>
__device__ __forceinline__ float rotated_entry(const A * v, int i, int half, int rot_dims, int style, const float * cs_sn) {
    if (i >= rot_dims) return to_f32(v[i]);
    if (style == 1) {
        const int n = i >> 1;
        return (i & 1) ? rot_hi(to_f32(v[i - 1]), to_f32(v[i]), cs_sn[2 * n], cs_sn[2 * n + 1])
                       : rot_lo(to_f32(v[i]), to_f32(v[i + 1]), cs_sn[2 * n], cs_sn[2 * n + 1]);
    }
    if (i < half) return rot_lo(to_f32(v[i]), to_f32(v[i + half]), cs_sn[2 * i], cs_sn[2 * i + 1]);
    return rot_hi(to_f32(v[i - half]), to_f32(v[i]), cs_sn[2 * (i - half)], cs_sn[2 * (i - half) + 1]);
}

// qd row: [.. q (H * (dim + rot)) .. dkv (rank + rot) ..] at q_off / dkv_off, row stride ld; with `qm` the queries are
// rows of a matrix of their own (row stride ld_q) instead.
// cache rows: [cells, rank + rot].  q_cat rows: [H, rank + rot]; this kernel fills [rank, rank + rot) of every head.
template <typename A>
__global__ void latent_prep_kernel(const A * __restrict__ qd, long long ld, int q_off, int dkv_off,
                                   const A * __restrict__ qm, long long ld_q, int style,
                                   A * __restrict__ cache, A * __restrict__ q_cat, const float * __restrict__ norm_w,
                                   const double * __restrict__ inv_freq, const int * __restrict__ positions,
                                   const int * __restrict__ slots, int H, int dim, int rot, int rank, int rot_dims,
                                   float eps, long long n_cells) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[32];
    extern __shared__ float cs_sn[];          // [rot_dims / 2][2]
    const size_t t = blockIdx.x;
    const A * row = qd + t * ld;
    const int half = rot_dims >> 1;
    const int p = positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const double a = (double) p * inv_freq[i];
        double s, c;
        sincos(a, &s, &c);
        cs_sn[2 * i] = (float) c;
        cs_sn[2 * i + 1] = (float) s;
    }
    // the latent: x / sqrt(mean(x^2) + eps) * w
    const A * dkv = row + dkv_off;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_f32(dkv[i]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);              // also orders the writes of cs_sn before their use
    const float inv = 1.0f / sqrtf(ss / (float) rank + eps);
    const long long cell = slots != nullptr ? slots[t] : -1;
    const int width = rank + rot;
    if (cell >= 0 && cell < n_cells) {
        A * crow = cache + (size_t) cell * width;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) crow[i] = from_f32<A>(to_f32(dkv[i]) * inv * norm_w[i]);
        const A * kr = dkv + rank;
        for (int i = threadIdx.x; i < rot; i += blockDim.x) crow[rank + i] = from_f32<A>(rotated_entry(kr, i, half, rot_dims, style, cs_sn));
    }
    // the rotated part of every query head
    const A * q = qm != nullptr ? qm + t * ld_q : row + q_off;
    for (int e = threadIdx.x; e < H * rot; e += blockDim.x) {
        const int h = e / rot, i = e - h * rot;
        const A * qr = q + (size_t) h * (dim + rot) + dim;
        q_cat[(t * H + h) * width + rank + i] = from_f32<A>(rotated_entry(qr, i, half, rot_dims, style, cs_sn));
    }
}

// out[t, h, j] = sum_i in[t * ld_in + h * in_hs + i] * w[h * w_hs + i * w_is + j * w_js],  i < n_in, j < n_out,
// written at out[t * ld_out + h * out_hs + j].  One thread per (t, h, j); i ascending.
template <typename A, typename W>
__global__ void head_linear_kernel(const A * __restrict__ in, long long ld_in, int in_hs, const W * __restrict__ w,
                                   long long w_hs, long long w_is, long long w_js, A * __restrict__ out, long long ld_out,
                                   int out_hs, int N, int H, int n_in, int n_out) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float xin[];            // the input vector of this (t, h)
    const int h = blockIdx.y;
    const size_t t = blockIdx.x;
    const A * x = in + t * ld_in + (size_t) h * in_hs;
    for (int i = threadIdx.x; i < n_in; i += blockDim.x) xin[i] = to_f32(x[i]);
    __syncthreads();
    const W * wh = w + (size_t) h * w_hs;
    for (int j = threadIdx.x; j < n_out; j += blockDim.x) {
        float acc = 0.0f;
        const W * wj = wh + (size_t) j * w_js;
        for (int i = 0; i < n_in; i++) acc = fmaf(xin[i], to_f32(wj[(size_t) i * w_is]), acc);
        out[t * ld_out + (size_t) h * out_hs + j] = from_f32<A>(acc);
    }
}

// The same products for steps of up to 8 tokens in bfloat16, where the weights should cross the memory system once and
// as many of their bytes as possible should be in flight at once: every load is 16 bytes, a block takes one head and a
// slab of its outputs for ALL tokens, and the inputs of the tokens wait in shared memory as float32.
//   OUT_FAST  the weight is contiguous along the outputs (w_js == 1).  128 threads = 16 groups of 8; a group covers 64
//             outputs of one input row (8 per thread), the groups take the input rows 16 apart; sums meet by shuffles
//             inside a warp (4 groups) and through shared memory across the 4 warps.
//   else      the weight is contiguous along the inputs (w_is == 1).  A warp owns an output at a time, a lane 8
//             consecutive inputs per step of 256; sums meet in a shuffle reduction.
constexpr int kSmallTokens = 8;
template <bool OUT_FAST>
__global__ void __launch_bounds__(128) head_linear_small_kernel(
    const __nv_bfloat16 * __restrict__ in, long long ld_in, int in_hs, const __nv_bfloat16 * __restrict__ w, long long w_hs,
    long long w_stride, __nv_bfloat16 * __restrict__ out, long long ld_out, int out_hs, int N, int n_in, int n_out) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float xin[];            // [kSmallTokens][n_in], then (OUT_FAST) [4][kSmallTokens][64]
    const int h = blockIdx.y;
    for (int e = threadIdx.x; e < kSmallTokens * n_in; e += blockDim.x) {
        const int t = e / n_in, i = e - t * n_in;
        xin[e] = t < N ? to_f32(in[(size_t) t * ld_in + (size_t) h * in_hs + i]) : 0.0f;
    }
    __syncthreads();
    const __nv_bfloat16 * wh = w + (size_t) h * w_hs;
    if (OUT_FAST) {
        const int ct = threadIdx.x & 7, ig = threadIdx.x >> 3, warp = threadIdx.x >> 5;
        const int j = blockIdx.x * 64 + ct * 8;
        float acc[kSmallTokens][8];
#pragma unroll
        for (int t = 0; t < kSmallTokens; t++)
#pragma unroll
            for (int c = 0; c < 8; c++) acc[t][c] = 0.0f;
        if (j < n_out) {                                     // n_out is a multiple of 8: a thread's 8 outputs are in or out together
#pragma unroll 8
            for (int i = ig; i < n_in; i += 16) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(wh + (size_t) i * w_stride + j);
                float wv[8];
                unpack8(raw, wv);
#pragma unroll
                for (int t = 0; t < kSmallTokens; t++) {
                    const float x = xin[t * n_in + i];
#pragma unroll
                    for (int c = 0; c < 8; c++) acc[t][c] = fmaf(x, wv[c], acc[t][c]);
                }
            }
        }
        float * red = xin + kSmallTokens * n_in;             // [4 warps][kSmallTokens][64]
#pragma unroll
        for (int t = 0; t < kSmallTokens; t++)
#pragma unroll
            for (int c = 0; c < 8; c++) {
                float v = acc[t][c];
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                if ((threadIdx.x & 31) < 8) red[(warp * kSmallTokens + t) * 64 + ct * 8 + c] = v;
            }
        __syncthreads();
        for (int e = threadIdx.x; e < N * 64; e += blockDim.x) {
            const int t = e >> 6, c = e & 63;
            const int jo = blockIdx.x * 64 + c;
            if (jo >= n_out) continue;
            const float v = red[(0 * kSmallTokens + t) * 64 + c] + red[(1 * kSmallTokens + t) * 64 + c] +
                            red[(2 * kSmallTokens + t) * 64 + c] + red[(3 * kSmallTokens + t) * 64 + c];
            out[(size_t) t * ld_out + (size_t) h * out_hs + jo] = __float2bfloat16_rn(v);
        }
    } else {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int j = blockIdx.x * 8 + warp; j < min(n_out, (int) blockIdx.x * 8 + 8); j += 4) {
            const __nv_bfloat16 * wj = wh + (size_t) j * w_stride;
            float acc[kSmallTokens];
#pragma unroll
            for (int t = 0; t < kSmallTokens; t++) acc[t] = 0.0f;
#pragma unroll 2
            for (int i = lane * 8; i < n_in; i += 256) {     // n_in is a multiple of 8
                const uint4 raw = *reinterpret_cast<const uint4 *>(wj + i);
                float wv[8];
                unpack8(raw, wv);
#pragma unroll
                for (int t = 0; t < kSmallTokens; t++) {
                    const float4 x0 = *reinterpret_cast<const float4 *>(xin + t * n_in + i);
                    const float4 x1 = *reinterpret_cast<const float4 *>(xin + t * n_in + i + 4);
                    acc[t] += x0.x * wv[0] + x0.y * wv[1] + x0.z * wv[2] + x0.w * wv[3] + x1.x * wv[4] + x1.y * wv[5] + x1.z * wv[6] + x1.w * wv[7];
                }
            }
#pragma unroll
            for (int t = 0; t < kSmallTokens; t++) acc[t] = warp_sum(acc[t]);
            if (lane == 0)
                for (int t = 0; t < N; t++) out[(size_t) t * ld_out + (size_t) h * out_hs + j] = __float2bfloat16_rn(acc[t]);
        }
    }
}

template <typename A>
__global__ void latent_attention_kernel(const A * __restrict__ q, const A * __restrict__ cache, A * __restrict__ out,
                                        const float * __restrict__ sink, const int * __restrict__ positions,
                                        const int * __restrict__ seq_of_token, const int * __restrict__ block_table,
                                        int max_blocks, const int * __restrict__ ctx_len, int N, int H, int rank, int width,
                                        int page_size, int num_pages, float scale, int window) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float qs_all[];         // [kLatWarps][width]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long) blockIdx.x * kLatWarps + warp;
    if (item >= (long long) N * H) return;
    const int t = (int) (item / H), h = (int) (item % H);
    float * qs = qs_all + (size_t) warp * width;
    A * o = out + ((size_t) t * H + h) * rank;
    const int s = seq_of_token[t];
    if (s < 0) {   // padding token
        for (int d = lane; d < rank; d += 32) o[d] = from_f32<A>(0.0f);
        return;
    }
    const int p = positions[t];
    int hi = p;
    if (ctx_len != nullptr) hi = min(hi, ctx_len[s] - 1);
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const A * qp = q + ((size_t) t * H + h) * width;
    for (int d = lane; d < width; d += 32) qs[d] = to_f32(qp[d]);
    __syncwarp();

    constexpr int kAcc = kLatMaxRank / 32;
    float acc[kAcc];
#pragma unroll
    for (int i = 0; i < kAcc; i++) acc[i] = 0.0f;
    // the sink opens the running softmax: maximum sink, denominator exp(sink - sink) = 1, no value
    float m = sink != nullptr ? sink[h] : -INFINITY;
    float l = sink != nullptr ? 1.0f : 0.0f;
    const int * bt = block_table + (size_t) s * max_blocks;

    for (int kb = (lo / 32) * 32; kb <= hi; kb += 32) {
        const int j = kb + lane;
        bool valid = j >= lo && j <= hi;
        const A * kp = nullptr;
        if (valid) {
            const int page = bt[j / page_size];
            if (page < 0 || page >= num_pages) valid = false;      // a page that was given back is never inside the window
            else kp = cache + ((size_t) page * page_size + (j % page_size)) * width;
        }
        float sc = -INFINITY;
        if (valid) {
            float dot = 0.0f;
            for (int d = 0; d < width; d++) dot = fmaf(qs[d], to_f32(kp[d]), dot);
            sc = dot * scale;
        }
        const float tile_max = warp_max(sc);
        if (tile_max == -INFINITY) continue;
        const float m_new = fmaxf(m, tile_max);
        const float pj = valid ? expf(sc - m_new) : 0.0f;
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        l = l * corr + warp_sum(pj);
#pragma unroll
        for (int i = 0; i < kAcc; i++) acc[i] *= corr;
        m = m_new;
        for (int jj = 0; jj < 32; jj++) {
            const float pjj = __shfl_sync(0xffffffffu, pj, jj);
            const unsigned long long vaddr = __shfl_sync(0xffffffffu, (unsigned long long) kp, jj);
            if (pjj == 0.0f) continue;
            const A * vrow = (const A *) vaddr;
#pragma unroll
            for (int i = 0; i < kAcc; i++) {
                const int d = lane + 32 * i;
                if (d < rank) acc[i] = fmaf(pjj, to_f32(vrow[d]), acc[i]);
            }
        }
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;     // a row that sees no key and has no sink yields zeros
#pragma unroll
    for (int i = 0; i < kAcc; i++) {
        const int d = lane + 32 * i;
        if (d < rank) o[d] = from_f32<A>(acc[i] * inv);
    }
}

}  // namespace iian

using namespace iian;

// qm: the queries as rows of a matrix of their own (row stride ld_q), or null: then they sit in qd at q_off.
// style: 0 pairs entry i with entry i + rot_dims / 2, 1 pairs entry 2 i with entry 2 i + 1.
IIAN_API int iian_latent_prep_split(const void * qd, long long ld, int q_off, int dkv_off, const void * qm, long long ld_q,
                                    int style, void * cache, void * q_cat, const float * norm_w, const double * inv_freq,
                                    const int * positions, const int * slots, int act_dtype, int N, int H, int dim, int rot,
                                    int rank, int rot_dims, float eps, long long n_cells, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > rot || rank <= 0 || H <= 0 || dim < 0 || (style != 0 && style != 1)) return IIAN_ERR_SHAPE;
    const size_t smem = (size_t) (rot_dims > 0 ? rot_dims : 2) * sizeof(float);
    if (smem > 40 * 1024) return IIAN_ERR_LIMIT;
    const int threads = 128;
    if (act_dtype == IIAN_F32)
        return iian_launch(latent_prep_kernel<float>, dim3(N), dim3(threads), smem, stream, (const float *) qd, ld, q_off, dkv_off,
                           (const float *) qm, ld_q, style, (float *) cache, (float *) q_cat, norm_w, inv_freq, positions, slots, H,
                           dim, rot, rank, rot_dims, eps, n_cells);
    if (act_dtype == IIAN_BF16)
        return iian_launch(latent_prep_kernel<__nv_bfloat16>, dim3(N), dim3(threads), smem, stream, (const __nv_bfloat16 *) qd, ld,
                           q_off, dkv_off, (const __nv_bfloat16 *) qm, ld_q, style, (__nv_bfloat16 *) cache,
                           (__nv_bfloat16 *) q_cat, norm_w, inv_freq, positions, slots, H, dim, rot, rank, rot_dims, eps, n_cells);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_latent_prep(const void * qd, long long ld, int q_off, int dkv_off, void * cache, void * q_cat,
                              const float * norm_w, const double * inv_freq, const int * positions, const int * slots,
                              int act_dtype, int N, int H, int dim, int rot, int rank, int rot_dims, float eps,
                              long long n_cells, cudaStream_t stream) {
    return iian_latent_prep_split(qd, ld, q_off, dkv_off, nullptr, 0, 0, cache, q_cat, norm_w, inv_freq, positions, slots,
                                  act_dtype, N, H, dim, rot, rank, rot_dims, eps, n_cells, stream);
}

IIAN_API int iian_head_linear(const void * in, long long ld_in, int in_hs, const void * w, int w_dtype, long long w_hs,
                              long long w_is, long long w_js, void * out, long long ld_out, int out_hs, int act_dtype, int N,
                              int H, int n_in, int n_out, cudaStream_t stream) {
    if (N <= 0 || H <= 0 || n_out <= 0) return IIAN_OK;
    if (n_in <= 0 || H > 65535) return IIAN_ERR_SHAPE;
    const size_t smem = (size_t) n_in * sizeof(float);
    if (smem > 48 * 1024) return IIAN_ERR_LIMIT;
    const int threads = n_out >= 256 ? 256 : n_out >= 128 ? 128 : 64;
    typedef __nv_bfloat16 bf;
    if (act_dtype == IIAN_F32 && w_dtype == IIAN_F32)
        return iian_launch(head_linear_kernel<float, float>, dim3(N, H), dim3(threads), smem, stream, (const float *) in, ld_in, in_hs,
                           (const float *) w, w_hs, w_is, w_js, (float *) out, ld_out, out_hs, N, H, n_in, n_out);
    if (act_dtype == IIAN_BF16 && w_dtype == IIAN_BF16)
        return iian_launch(head_linear_kernel<bf, bf>, dim3(N, H), dim3(threads), smem, stream, (const bf *) in, ld_in, in_hs,
                           (const bf *) w, w_hs, w_is, w_js, (bf *) out, ld_out, out_hs, N, H, n_in, n_out);
    if (act_dtype == IIAN_BF16 && w_dtype == IIAN_F32)
        return iian_launch(head_linear_kernel<bf, float>, dim3(N, H), dim3(threads), smem, stream, (const bf *) in, ld_in, in_hs,
                           (const float *) w, w_hs, w_is, w_js, (bf *) out, ld_out, out_hs, N, H, n_in, n_out);
    return IIAN_ERR_DTYPE;
}

// The form for up to 8 tokens (bfloat16 activations and weights); w_is or w_js must be 1, the contiguous extent of the
// weight a multiple of 8 and every row of it 16-byte aligned (else IIAN_ERR_SHAPE / IIAN_ERR_ALIGN: use the general form).
IIAN_API int iian_head_linear_small(const void * in, long long ld_in, int in_hs, const void * w, long long w_hs, long long w_is,
                                    long long w_js, void * out, long long ld_out, int out_hs, int N, int H, int n_in, int n_out,
                                    cudaStream_t stream) {
    if (N <= 0 || H <= 0 || n_out <= 0) return IIAN_OK;
    if (N > kSmallTokens || n_in <= 0 || H > 65535 || (w_is != 1 && w_js != 1)) return IIAN_ERR_SHAPE;
    typedef __nv_bfloat16 bf;
    const bool out_fast = w_js == 1;
    const long long stride = out_fast ? w_is : w_js;
    if ((out_fast ? n_out : n_in) % 8 != 0) return IIAN_ERR_SHAPE;
    if (((uintptr_t) w & 15) || stride % 8 != 0 || w_hs % 8 != 0) return IIAN_ERR_ALIGN;
    const size_t smem = ((size_t) kSmallTokens * n_in + (out_fast ? 4 * kSmallTokens * 64 : 0)) * sizeof(float);
    if (smem > 48 * 1024) return IIAN_ERR_LIMIT;
    if (out_fast)
        return iian_launch(head_linear_small_kernel<true>, dim3((n_out + 63) / 64, H), dim3(128), smem, stream, (const bf *) in, ld_in,
                           in_hs, (const bf *) w, w_hs, stride, (bf *) out, ld_out, out_hs, N, n_in, n_out);
    return iian_launch(head_linear_small_kernel<false>, dim3((n_out + 7) / 8, H), dim3(128), smem, stream, (const bf *) in, ld_in,
                       in_hs, (const bf *) w, w_hs, stride, (bf *) out, ld_out, out_hs, N, n_in, n_out);
}

// q: [N, H, width]; cache: [num_pages * page_size, width]; out: [N, H, rank]; sink: f32 [H] or null;
// block_table: [S, max_blocks]; ctx_len may be null (then only causality bounds the keys).
IIAN_API int iian_latent_attention(const void * q, const void * cache, void * out, const float * sink, const int * positions,
                                   const int * seq_of_token, const int * block_table, int max_blocks, const int * ctx_len,
                                   int act_dtype, int N, int H, int rank, int width, int page_size, int num_pages, float scale,
                                   int window, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (rank <= 0 || rank > kLatMaxRank || width < rank || width > kLatMaxWidth || H <= 0 || page_size <= 0) return IIAN_ERR_SHAPE;
    const long long items = (long long) N * H;
    const unsigned blocks = (unsigned) ((items + kLatWarps - 1) / kLatWarps);
    const int threads = kLatWarps * 32;
    const size_t smem = (size_t) kLatWarps * width * sizeof(float);
    if (act_dtype == IIAN_F32)
        return iian_launch(latent_attention_kernel<float>, dim3(blocks), dim3(threads), smem, stream, (const float *) q, (const float *) cache,
                           (float *) out, sink, positions, seq_of_token, block_table, max_blocks, ctx_len, N, H, rank, width, page_size,
                           num_pages, scale, window);
    if (act_dtype == IIAN_BF16)
        return iian_launch(latent_attention_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), smem, stream, (const __nv_bfloat16 *) q,
                           (const __nv_bfloat16 *) cache, (__nv_bfloat16 *) out, sink, positions, seq_of_token, block_table, max_blocks,
                           ctx_len, N, H, rank, width, page_size, num_pages, scale, window);
    return IIAN_ERR_DTYPE;
}
