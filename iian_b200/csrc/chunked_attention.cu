// Paged attention without rotation, for mixers whose positions enter through the mask and a penalty on distance:
//     s_ij = (q_i . k_j) * scale - r1_h * ln(1 + r2_h * (i - j))
// Key j is visible to position i iff j <= i and, with a chunk size c > 0, floor(i / c) == floor(j / c) (chunks are counted
// from position 0 of the sequence); with a window w > 0 instead, iff i - j < w.  Keys have `dk` entries per head, values
// `dv` (they may differ); values are stored divided by their root mean square.  The output may be multiplied element by
// element with sigmoid(gate).
//
// Kernels:
//   kv_store_normed    per token: K as projected and V / sqrt(mean(V^2) + eps) per head into their cache cells
//   chunked_attention  general form (any element type and sizes): one warp per (token, head), keys in tiles of 32 that
//                      start at multiples of 32 of the ABSOLUTE key position, so the order of every sum depends on the
//                      token's own position only
#include "common.cuh"

namespace iian {

constexpr int kCaMaxDim = 512;
constexpr int kCaWarps = 4;

// proj rows: [.. k (nkv * dk) | v (nkv * dv) ..] at k_off / v_off, row stride ld.
// caches: K [pages, nkv, page_size, dk], V [pages, nkv, page_size, dv].
template <typename A>
__global__ void kv_store_normed_kernel(const A * __restrict__ proj, long long ld, int k_off, int v_off,
                                       A * __restrict__ k_cache, A * __restrict__ v_cache, const int * __restrict__ slots,
                                       int nkv, int dk, int dv, int page_size, long long n_cells, float eps, int norm_values) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const size_t t = blockIdx.x;
    const long long cell = slots[t];
    if (cell < 0 || cell >= n_cells) return;
    const long long page = cell / page_size, off = cell % page_size;
    const A * row = proj + t * ld;
    for (int g = warp; g < nkv; g += warps) {
        const A * ks = row + k_off + (size_t) g * dk;
        A * kd = k_cache + ((page * nkv + g) * page_size + off) * dk;
        for (int d = lane; d < dk; d += 32) kd[d] = ks[d];
        const A * vs = row + v_off + (size_t) g * dv;
        A * vd = v_cache + ((page * nkv + g) * page_size + off) * dv;
        float inv = 1.0f;
        if (norm_values) {
            float ss = 0.0f;
            for (int d = lane; d < dv; d += 32) {
                const float x = to_f32(vs[d]);
                ss = fmaf(x, x, ss);
            }
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float) dv + eps);
        }
        for (int d = lane; d < dv; d += 32) vd[d] = from_f32<A>(to_f32(vs[d]) * inv);
    }
}

template <typename A>
__global__ void chunked_attention_kernel(
    const A * __restrict__ q, long long ld_q, const A * __restrict__ k_cache, const A * __restrict__ v_cache,
    A * __restrict__ out, const int * __restrict__ positions, const int * __restrict__ seq_of_token,
    const int * __restrict__ block_table, int max_blocks, const int * __restrict__ ctx_len,
    int N, int nh, int nkv, int dk, int dv, int page_size, int num_pages, float scale, int chunk, int window,
    const float * __restrict__ r1, const float * __restrict__ r2, const A * __restrict__ gate, long long ld_gate) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float qs[kCaWarps][kCaMaxDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long) blockIdx.x * kCaWarps + warp;
    if (item >= (long long) N * nh) return;
    const int t = (int) (item / nh), h = (int) (item % nh);
    const int kvh = h / (nh / nkv);
    A * o = out + ((size_t) t * nh + h) * dv;
    const int s = seq_of_token[t];
    if (s < 0) {   // padding token
        for (int d = lane; d < dv; d += 32) o[d] = from_f32<A>(0.0f);
        return;
    }
    const int p = positions[t];
    int hi = p;
    if (ctx_len != nullptr) hi = min(hi, ctx_len[s] - 1);
    int lo = 0;
    if (chunk > 0) lo = (p / chunk) * chunk;
    else if (window > 0) lo = max(0, p - window + 1);
    const float b1 = r1 != nullptr ? r1[h] : 0.0f, b2 = r2 != nullptr ? r2[h] : 0.0f;

    const A * qp = q + (size_t) t * ld_q + (size_t) h * dk;
    for (int d = lane; d < dk; d += 32) qs[warp][d] = to_f32(qp[d]);
    __syncwarp();

    constexpr int kAcc = kCaMaxDim / 32;
    float acc[kAcc];
#pragma unroll
    for (int i = 0; i < kAcc; i++) acc[i] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    const int * bt = block_table + (size_t) s * max_blocks;

    for (int kb = (lo / 32) * 32; kb <= hi; kb += 32) {
        const int j = kb + lane;
        bool valid = j >= lo && j <= hi;
        const A * kp = nullptr;
        const A * vp = nullptr;
        if (valid) {
            const int page = bt[j / page_size];
            if (page < 0 || page >= num_pages) {
                valid = false;
            } else {
                const size_t cell = ((size_t) page * nkv + kvh) * page_size + (j % page_size);
                kp = k_cache + cell * dk;
                vp = v_cache + cell * dv;
            }
        }
        float sc = -INFINITY;
        if (valid) {
            float dot = 0.0f;
            for (int d = 0; d < dk; d++) dot = fmaf(qs[warp][d], to_f32(kp[d]), dot);
            sc = dot * scale - b1 * log1pf(b2 * (float) (p - j));
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
            const unsigned long long vaddr = __shfl_sync(0xffffffffu, (unsigned long long) vp, jj);
            if (pjj == 0.0f) continue;
            const A * vrow = (const A *) vaddr;
#pragma unroll
            for (int i = 0; i < kAcc; i++) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] = fmaf(pjj, to_f32(vrow[d]), acc[i]);
            }
        }
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < kAcc; i++) {
        const int d = lane + 32 * i;
        if (d < dv) {
            float v = acc[i] * inv;
            if (gate != nullptr) v *= 1.0f / (1.0f + expf(-to_f32(gate[(size_t) t * ld_gate + h * dv + d])));
            o[d] = from_f32<A>(v);
        }
    }
}

}  // namespace iian

using namespace iian;

IIAN_API int iian_kv_store_normed(const void * proj, long long ld, int k_off, int v_off, void * k_cache, void * v_cache,
                                  const int * slots, int act_dtype, int N, int nkv, int dk, int dv, int page_size,
                                  long long n_cells, float eps, int norm_values, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (nkv <= 0 || dk <= 0 || dv <= 0 || page_size <= 0) return IIAN_ERR_SHAPE;
    if (act_dtype == IIAN_F32)
        return iian_launch(kv_store_normed_kernel<float>, dim3(N), dim3(128), 0, stream, (const float *) proj, ld, k_off, v_off,
                           (float *) k_cache, (float *) v_cache, slots, nkv, dk, dv, page_size, n_cells, eps, norm_values);
    if (act_dtype == IIAN_BF16)
        return iian_launch(kv_store_normed_kernel<__nv_bfloat16>, dim3(N), dim3(128), 0, stream, (const __nv_bfloat16 *) proj, ld,
                           k_off, v_off, (__nv_bfloat16 *) k_cache, (__nv_bfloat16 *) v_cache, slots, nkv, dk, dv, page_size,
                           n_cells, eps, norm_values);
    return IIAN_ERR_DTYPE;
}

// q: rows of nh * dk with row stride ld_q; out: [N, nh * dv]; r1, r2: float32 [nh] or null (no penalty);
// gate: rows of nh * dv with row stride ld_gate, or null.  chunk / window: 0 = none (at most one of them).
IIAN_API int iian_chunked_attention(const void * q, long long ld_q, const void * k_cache, const void * v_cache, void * out,
                                    const int * positions, const int * seq_of_token, const int * block_table, int max_blocks,
                                    const int * ctx_len, int act_dtype, int N, int nh, int nkv, int dk, int dv, int page_size,
                                    int num_pages, float scale, int chunk, int window, const float * r1, const float * r2,
                                    const void * gate, long long ld_gate, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (dk <= 0 || dk > kCaMaxDim || dv <= 0 || dv > kCaMaxDim || nkv <= 0 || nh % nkv != 0 || page_size <= 0 ||
        (chunk > 0 && window > 0)) return IIAN_ERR_SHAPE;
    const long long items = (long long) N * nh;
    const unsigned blocks = (unsigned) ((items + kCaWarps - 1) / kCaWarps);
    if (act_dtype == IIAN_F32)
        return iian_launch(chunked_attention_kernel<float>, dim3(blocks), dim3(kCaWarps * 32), 0, stream, (const float *) q, ld_q,
                           (const float *) k_cache, (const float *) v_cache, (float *) out, positions, seq_of_token, block_table,
                           max_blocks, ctx_len, N, nh, nkv, dk, dv, page_size, num_pages, scale, chunk, window, r1, r2,
                           (const float *) gate, ld_gate);
    if (act_dtype == IIAN_BF16)
        return iian_launch(chunked_attention_kernel<__nv_bfloat16>, dim3(blocks), dim3(kCaWarps * 32), 0, stream,
                           (const __nv_bfloat16 *) q, ld_q, (const __nv_bfloat16 *) k_cache, (const __nv_bfloat16 *) v_cache,
                           (__nv_bfloat16 *) out, positions, seq_of_token, block_table, max_blocks, ctx_len, N, nh, nkv, dk, dv,
                           page_size, num_pages, scale, chunk, window, r1, r2, (const __nv_bfloat16 *) gate, ld_gate);
    return IIAN_ERR_DTYPE;
}
