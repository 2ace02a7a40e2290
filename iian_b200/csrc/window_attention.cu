// Rotated attention over a paged K/V cache with a sliding window that may keep the first keys of the sequence, a sink in the
// softmax's denominator and a gate per head or per entry of the output.
//
//     key j is visible to position i  iff  j <= i and (window == 0 or i - j < window or j < keep_first)
//     s_ij = (q_i . k_j) * scale;   p = softmax over the visible keys, the denominator also holding exp(sink_h) if given
//     o_i = sum_j p_ij v_j,  times sigmoid(gate) (one number per head, or one per entry)
//
// Keys have `dk` entries per head, values `dv` (they may differ).  Kept keys keep their true positions: they were rotated and
// stored like every other key, so nothing but the mask knows about them.
//
// Kernels:
//   rotary_table_scaled   cos and sin of position * frequency, the product and the functions in float64, both multiplied by a
//                         magnitude (frequency tables that were rescaled for long contexts bring one); float32 [N, half, 2]
//   rotate_unit_store     per token and head: rotation of the first `rot` entries of q and k (entry i with entry i + rot / 2),
//                         THEN optionally each head of q and k divided by its root mean square (no weight); q to the
//                         attention's rows, k and v (as projected) to their cache cells
//   window_attention      general form (any element type and sizes up to 512): one warp per (token, head), keys in tiles of 32
//                         that start at multiples of 32 of the ABSOLUTE key position, so the order of every sum depends on the
//                         token's own position only
#include "common.cuh"

namespace iian {

constexpr int kWaMaxDim = 512;
constexpr int kWaWarps = 4;

__global__ void rotary_table_scaled_kernel(const double * __restrict__ inv_freq, const int * __restrict__ positions,
                                           float2 * __restrict__ table, int half, long long total, double magnitude) {
    pdl_wait();
    pdl_launch_dependents();
    const long long idx = (long long) blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int t = (int) (idx / half), p = (int) (idx % half);
    double sn, cs;
    sincos((double) positions[t] * inv_freq[p], &sn, &cs);
    table[idx] = make_float2((float) (cs * magnitude), (float) (sn * magnitude));
}

// proj rows: q (nh * dk) at q_off, k (nkv * dk) at k_off, v (nkv * dv) at v_off, row stride ld.  q_out: [N, nh, dk].
// caches: K [pages, nkv, page_size, dk], V [pages, nkv, page_size, dv]; k_cache == null: q only.
// table: float2 [N, rot / 2] (cos, sin) or null (no rotation).
template <typename A>
__global__ void rotate_unit_store_kernel(const A * __restrict__ proj, long long ld, int q_off, int k_off, int v_off,
                                         A * __restrict__ q_out, A * __restrict__ k_cache, A * __restrict__ v_cache,
                                         const float2 * __restrict__ table, const int * __restrict__ slots, int N, int nh, int nkv,
                                         int dk, int dv, int rot, int page_size, long long n_cells, float eps, int unit_norm) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float xs[kWaWarps][kWaMaxDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_token = nh + (k_cache != nullptr ? nkv : 0);
    const long long item = (long long) blockIdx.x * kWaWarps + warp;
    if (item >= (long long) N * per_token) return;
    const int t = (int) (item / per_token), hh = (int) (item % per_token);
    const bool is_q = hh < nh;
    const int g = is_q ? hh : hh - nh;
    const A * row = proj + (size_t) t * ld;
    A * dst;
    if (is_q) {
        dst = q_out + ((size_t) t * nh + g) * dk;
    } else {
        const long long cell = slots[t];
        if (cell < 0 || cell >= n_cells) return;            // padding token: nothing is stored
        const long long page = cell / page_size, off = cell % page_size;
        dst = k_cache + ((page * nkv + g) * page_size + off) * dk;
        const A * vs = row + v_off + (size_t) g * dv;
        A * vd = v_cache + ((page * nkv + g) * page_size + off) * dv;
        for (int d = lane; d < dv; d += 32) vd[d] = vs[d];
    }
    const A * src = row + (is_q ? q_off : k_off) + (size_t) g * dk;
    for (int d = lane; d < dk; d += 32) xs[warp][d] = to_f32(src[d]);
    __syncwarp();
    const int half = rot / 2;
    const float2 * tab = table != nullptr ? table + (size_t) t * half : nullptr;
    float ss = 0.0f;
    float vals[kWaMaxDim / 32];
#pragma unroll
    for (int i = 0; i < kWaMaxDim / 32; i++) {
        const int d = lane + 32 * i;
        float v = 0.0f;
        if (d < dk) {
            v = xs[warp][d];
            if (tab != nullptr && d < 2 * half) {
                if (d < half) {
                    const float2 cs = tab[d];
                    v = rot_lo(v, xs[warp][d + half], cs.x, cs.y);
                } else {
                    const float2 cs = tab[d - half];
                    v = rot_hi(xs[warp][d - half], v, cs.x, cs.y);
                }
            }
        }
        vals[i] = v;
        ss = fmaf(v, v, ss);
    }
    float inv = 1.0f;
    if (unit_norm) {
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float) dk + eps);
    }
#pragma unroll
    for (int i = 0; i < kWaMaxDim / 32; i++) {
        const int d = lane + 32 * i;
        if (d < dk) dst[d] = from_f32<A>(vals[i] * inv);
    }
}

template <typename A>
__global__ void window_attention_kernel(
    const A * __restrict__ q, long long ld_q, const A * __restrict__ k_cache, const A * __restrict__ v_cache,
    A * __restrict__ out, const int * __restrict__ positions, const int * __restrict__ seq_of_token,
    const int * __restrict__ block_table, int max_blocks, const int * __restrict__ ctx_len,
    int N, int nh, int nkv, int dk, int dv, int page_size, int num_pages, float scale, int window, int keep_first,
    const float * __restrict__ sink, const A * __restrict__ gate, long long ld_gate, int gate_per_head) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float qs[kWaWarps][kWaMaxDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long) blockIdx.x * kWaWarps + warp;
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
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int kept = min(keep_first, lo);                    // keys [0, kept) are seen although the window has passed them
    const int lo_tile = (lo / 32) * 32;
    const int kept_end = ((kept + 31) / 32) * 32;            // first tile start at or behind the kept keys

    const A * qp = q + (size_t) t * ld_q + (size_t) h * dk;
    for (int d = lane; d < dk; d += 32) qs[warp][d] = to_f32(qp[d]);
    __syncwarp();

    constexpr int kAcc = kWaMaxDim / 32;
    float acc[kAcc];
#pragma unroll
    for (int i = 0; i < kAcc; i++) acc[i] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    if (sink != nullptr) {       // the running softmax starts at the sink: maximum sink, sum 1, no value
        m = sink[h];
        l = 1.0f;
    }
    const int * bt = block_table + (size_t) s * max_blocks;

    for (int kb = 0; kb <= hi; kb += 32) {
        if (kb >= kept_end && kb < lo_tile) {
            kb = lo_tile - 32;                               // jump over the tiles between the kept keys and the window
            continue;
        }
        const int j = kb + lane;
        bool valid = j <= hi && (j >= lo || j < kept);
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
    float inv = l > 0.0f ? 1.0f / l : 0.0f;
    if (gate != nullptr && gate_per_head) inv *= 1.0f / (1.0f + expf(-to_f32(gate[(size_t) t * ld_gate + h])));
#pragma unroll
    for (int i = 0; i < kAcc; i++) {
        const int d = lane + 32 * i;
        if (d < dv) {
            float v = acc[i] * inv;
            if (gate != nullptr && !gate_per_head) v *= 1.0f / (1.0f + expf(-to_f32(gate[(size_t) t * ld_gate + h * dv + d])));
            o[d] = from_f32<A>(v);
        }
    }
}

}  // namespace iian

using namespace iian;

IIAN_API int iian_rotary_table_scaled(const double * inv_freq, const int * positions, void * table, int N, int half,
                                      double magnitude, cudaStream_t stream) {
    const long long total = (long long) N * half;
    if (total <= 0) return IIAN_OK;
    const int threads = 128;
    return iian_launch(rotary_table_scaled_kernel, dim3((unsigned) ((total + threads - 1) / threads)), dim3(threads), 0, stream,
                       inv_freq, positions, (float2 *) table, half, total, magnitude);
}

IIAN_API int iian_rotate_unit_store(const void * proj, long long ld, int q_off, int k_off, int v_off, void * q_out, void * k_cache,
                                    void * v_cache, const void * table, const int * slots, int act_dtype, int N, int nh, int nkv,
                                    int dk, int dv, int rot, int page_size, long long n_cells, float eps, int unit_norm,
                                    cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (nh <= 0 || nkv < 0 || dk <= 0 || dk > kWaMaxDim || dv <= 0 || rot < 0 || rot > dk || (rot & 1) || page_size <= 0)
        return IIAN_ERR_SHAPE;
    if (k_cache != nullptr && (v_cache == nullptr || slots == nullptr || nkv <= 0)) return IIAN_ERR_SHAPE;
    if (rot > 0 && table == nullptr) return IIAN_ERR_SHAPE;
    const long long items = (long long) N * (nh + (k_cache != nullptr ? nkv : 0));
    const unsigned blocks = (unsigned) ((items + kWaWarps - 1) / kWaWarps);
    const float2 * tab = rot > 0 ? (const float2 *) table : nullptr;
    if (act_dtype == IIAN_F32)
        return iian_launch(rotate_unit_store_kernel<float>, dim3(blocks), dim3(kWaWarps * 32), 0, stream, (const float *) proj, ld,
                           q_off, k_off, v_off, (float *) q_out, (float *) k_cache, (float *) v_cache, tab, slots, N, nh, nkv, dk, dv,
                           rot, page_size, n_cells, eps, unit_norm);
    if (act_dtype == IIAN_BF16)
        return iian_launch(rotate_unit_store_kernel<__nv_bfloat16>, dim3(blocks), dim3(kWaWarps * 32), 0, stream,
                           (const __nv_bfloat16 *) proj, ld, q_off, k_off, v_off, (__nv_bfloat16 *) q_out, (__nv_bfloat16 *) k_cache,
                           (__nv_bfloat16 *) v_cache, tab, slots, N, nh, nkv, dk, dv, rot, page_size, n_cells, eps, unit_norm);
    return IIAN_ERR_DTYPE;
}

// q: rows of nh * dk with row stride ld_q; out: [N, nh * dv]; sink: float32 [nh] or null; gate: rows with row stride ld_gate
// holding nh numbers (gate_per_head) or nh * dv, or null.  window: 0 = every earlier key; keep_first only with a window.
IIAN_API int iian_window_attention(const void * q, long long ld_q, const void * k_cache, const void * v_cache, void * out,
                                   const int * positions, const int * seq_of_token, const int * block_table, int max_blocks,
                                   const int * ctx_len, int act_dtype, int N, int nh, int nkv, int dk, int dv, int page_size,
                                   int num_pages, float scale, int window, int keep_first, const float * sink, const void * gate,
                                   long long ld_gate, int gate_per_head, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (dk <= 0 || dk > kWaMaxDim || dv <= 0 || dv > kWaMaxDim || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || window < 0 ||
        keep_first < 0) return IIAN_ERR_SHAPE;
    const long long items = (long long) N * nh;
    const unsigned blocks = (unsigned) ((items + kWaWarps - 1) / kWaWarps);
    if (act_dtype == IIAN_F32)
        return iian_launch(window_attention_kernel<float>, dim3(blocks), dim3(kWaWarps * 32), 0, stream, (const float *) q, ld_q,
                           (const float *) k_cache, (const float *) v_cache, (float *) out, positions, seq_of_token, block_table,
                           max_blocks, ctx_len, N, nh, nkv, dk, dv, page_size, num_pages, scale, window, keep_first, sink,
                           (const float *) gate, ld_gate, gate_per_head);
    if (act_dtype == IIAN_BF16)
        return iian_launch(window_attention_kernel<__nv_bfloat16>, dim3(blocks), dim3(kWaWarps * 32), 0, stream,
                           (const __nv_bfloat16 *) q, ld_q, (const __nv_bfloat16 *) k_cache, (const __nv_bfloat16 *) v_cache,
                           (__nv_bfloat16 *) out, positions, seq_of_token, block_table, max_blocks, ctx_len, N, nh, nkv, dk, dv,
                           page_size, num_pages, scale, window, keep_first, sink, (const __nv_bfloat16 *) gate, ld_gate,
                           gate_per_head);
    return IIAN_ERR_DTYPE;
}
