// Row-wise kernels around gated mixers and a re-injected embedding.
//
//   stream_concat:   out[t] = A([x_t + (d1_t + d2_t) ; e_t])      the input of a product that mixes the stream with
//                                                                  what the embedding left (sums in float32)
//   sigmoid_mul:     out = x * sigmoid(g)                          an output gate, element by element
//   head_norm_gate:  out[t, h, :] = x[t, h, :] / sqrt(mean(x[t, h, :]^2) + eps) * w[h, :] * sigmoid(g[t, h, :])
//                                                                  every head by its own root mean square, then a weight
//                                                                  per column and an output gate
//
// `A` is the activation type; every sum, the sigmoid and the norm are float32.  A row's result depends on that row only.
#include "common.cuh"

namespace iian {

__device__ __forceinline__ float sigmoid_f32(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename A>
__global__ void stream_concat_kernel(const float * __restrict__ x, const A * __restrict__ d1, const A * __restrict__ d2,
                                     const float * __restrict__ e, A * __restrict__ out, int H) {
    pdl_wait();
    const size_t t = blockIdx.x;
    const float * xr = x + t * H;
    const float * er = e + t * H;
    A * o = out + t * 2 * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (d1 != nullptr && d2 != nullptr) v += to_f32(d1[t * H + i]) + to_f32(d2[t * H + i]);
        else if (d1 != nullptr) v += to_f32(d1[t * H + i]);
        o[i] = from_f32<A>(v);
        o[H + i] = from_f32<A>(er[i]);
    }
}

template <typename A>
__global__ void sigmoid_mul_kernel(const A * __restrict__ x, const A * __restrict__ g, long long ld_g, A * __restrict__ out,
                                   int M, size_t total) {
    pdl_wait();
    const size_t idx = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t row = idx / M;
    const int col = (int) (idx - row * M);
    out[idx] = from_f32<A>(to_f32(x[idx]) * sigmoid_f32(to_f32(g[row * ld_g + col])));
}

// one warp per (token, head)
template <typename A>
__global__ void head_norm_gate_kernel(const float * __restrict__ x, const float * __restrict__ w, const A * __restrict__ g,
                                      long long ld_g, A * __restrict__ out, long long items, int heads, int dv, float eps, int gate_act) {
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long) blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= items) return;
    const long long t = item / heads;
    const int h = (int) (item - t * heads);
    const float * xr = x + item * dv;
    float ss = 0.0f;
    for (int d = lane; d < dv; d += 32) ss += xr[d] * xr[d];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float) dv + eps);
    for (int d = lane; d < dv; d += 32) {
        float v = xr[d] * inv * w[h * dv + d];
        if (g != nullptr) {
            const float z = to_f32(g[t * ld_g + h * dv + d]);
            v *= gate_act == 1 ? z * sigmoid_f32(z) : sigmoid_f32(z);
        }
        out[item * dv + d] = from_f32<A>(v);
    }
}

template <typename A>
__global__ void weighted_sum2_kernel(const A * __restrict__ x, float a, const A * __restrict__ y, float b, A * __restrict__ out,
                                     long long total) {
    pdl_wait();
    const long long idx = (long long) blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    out[idx] = from_f32<A>(fmaf(a, to_f32(x[idx]), b * to_f32(y[idx])));
}

// the same with a block per (token, head), for heads (or whole rows) of many entries
template <typename A>
__global__ void head_norm_gate_block_kernel(const float * __restrict__ x, const float * __restrict__ w, const A * __restrict__ g,
                                            long long ld_g, A * __restrict__ out, int heads, int dv, float eps, int gate_act) {
    pdl_wait();
    __shared__ float scratch[32];
    const long long item = blockIdx.x;
    const long long t = item / heads;
    const int h = (int) (item - t * heads);
    const float * xr = x + item * dv;
    float ss = 0.0f;
    for (int d = threadIdx.x; d < dv; d += blockDim.x) ss += xr[d] * xr[d];
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float) dv + eps);
    for (int d = threadIdx.x; d < dv; d += blockDim.x) {
        float v = xr[d] * inv * w[h * dv + d];
        if (g != nullptr) {
            const float z = to_f32(g[t * ld_g + h * dv + d]);
            v *= gate_act == 1 ? z * sigmoid_f32(z) : sigmoid_f32(z);
        }
        out[item * dv + d] = from_f32<A>(v);
    }
}

}  // namespace iian

using namespace iian;

// x, e: f32 [N, H]; d1, d2: A [N, H] or null (d2 only with d1); out: A [N, 2 H]
IIAN_API int iian_stream_concat(const float * x, const void * d1, const void * d2, const float * e, void * out, int act_dtype,
                                int N, int H, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (d1 == nullptr && d2 != nullptr) return IIAN_ERR_SHAPE;
    const int threads = H >= 1024 ? 256 : 128;
    if (act_dtype == IIAN_F32) return iian_launch(stream_concat_kernel<float>, dim3(N), dim3(threads), 0, stream, x, (const float *) d1, (const float *) d2, e, (float *) out, H);
    if (act_dtype == IIAN_BF16) return iian_launch(stream_concat_kernel<__nv_bfloat16>, dim3(N), dim3(threads), 0, stream, x, (const __nv_bfloat16 *) d1, (const __nv_bfloat16 *) d2, e, (__nv_bfloat16 *) out, H);
    return IIAN_ERR_DTYPE;
}

// x, out: A [N, M] contiguous; g: A, rows of M with row stride ld_g
IIAN_API int iian_sigmoid_mul(const void * x, const void * g, long long ld_g, void * out, int act_dtype, int N, int M,
                              cudaStream_t stream) {
    const size_t total = (size_t) N * M;
    if (total == 0) return IIAN_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned) ((total + threads - 1) / threads);
    if (act_dtype == IIAN_F32) return iian_launch(sigmoid_mul_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float *) x, (const float *) g, ld_g, (float *) out, M, total);
    if (act_dtype == IIAN_BF16) return iian_launch(sigmoid_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16 *) x, (const __nv_bfloat16 *) g, ld_g, (__nv_bfloat16 *) out, M, total);
    return IIAN_ERR_DTYPE;
}

// x: f32 [N, heads, dv]; w: f32 [heads * dv]; g: A rows of heads * dv with row stride ld_g, or null; out: A [N, heads * dv].
// gate_act: what the gate's column passes before it multiplies: 0 sigmoid, 1 silu.
IIAN_API int iian_head_norm_gate_act(const float * x, const float * w, const void * g, long long ld_g, void * out, int act_dtype,
                                     int N, int heads, int dv, float eps, int gate_act, cudaStream_t stream) {
    const long long items = (long long) N * heads;
    if (items <= 0) return IIAN_OK;
    if (dv <= 0 || (gate_act != 0 && gate_act != 1)) return IIAN_ERR_SHAPE;
    if (dv >= 1024 && items <= 0x7fffffff) {          // long rows: a block each
        const int threads = dv >= 4096 ? 512 : 256;
        if (act_dtype == IIAN_F32) return iian_launch(head_norm_gate_block_kernel<float>, dim3((unsigned) items), dim3(threads), 0, stream, x, w, (const float *) g, ld_g, (float *) out, heads, dv, eps, gate_act);
        if (act_dtype == IIAN_BF16) return iian_launch(head_norm_gate_block_kernel<__nv_bfloat16>, dim3((unsigned) items), dim3(threads), 0, stream, x, w, (const __nv_bfloat16 *) g, ld_g, (__nv_bfloat16 *) out, heads, dv, eps, gate_act);
        return IIAN_ERR_DTYPE;
    }
    const int warps = 4;
    const unsigned blocks = (unsigned) ((items + warps - 1) / warps);
    if (act_dtype == IIAN_F32) return iian_launch(head_norm_gate_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, x, w, (const float *) g, ld_g, (float *) out, items, heads, dv, eps, gate_act);
    if (act_dtype == IIAN_BF16) return iian_launch(head_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), 0, stream, x, w, (const __nv_bfloat16 *) g, ld_g, (__nv_bfloat16 *) out, items, heads, dv, eps, gate_act);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_head_norm_gate(const float * x, const float * w, const void * g, long long ld_g, void * out, int act_dtype,
                                 int N, int heads, int dv, float eps, cudaStream_t stream) {
    return iian_head_norm_gate_act(x, w, g, ld_g, out, act_dtype, N, heads, dv, eps, 0, stream);
}

// out = a * x + b * y, element by element (x, y, out: A, same shape; the sum in float32)
IIAN_API int iian_weighted_sum2(const void * x, float a, const void * y, float b, void * out, int act_dtype, long long total,
                                cudaStream_t stream) {
    if (total <= 0) return IIAN_OK;
    const unsigned blocks = (unsigned) ((total + 255) / 256);
    if (act_dtype == IIAN_F32) return iian_launch(weighted_sum2_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float *) x, a, (const float *) y, b, (float *) out, total);
    if (act_dtype == IIAN_BF16) return iian_launch(weighted_sum2_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16 *) x, a, (const __nv_bfloat16 *) y, b, (__nv_bfloat16 *) out, total);
    return IIAN_ERR_DTYPE;
}
