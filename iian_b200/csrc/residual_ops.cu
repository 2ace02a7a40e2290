// Row-wise kernels around a residual stream whose sub-layer outputs are added with a factor, a feed-forward activation with
// two learned numbers, a second token-indexed input per layer, and a cap on the logits.
//
//   scaled_add_rms_norm   x += m * d (float32, in place);  out = x / sqrt(mean(x^2) + eps) * w      (d, out optional)
//   scaled_add_unit_rms   x += m * y / sqrt(mean(y^2) + eps) * w                                     a normalised addend
//   gelu_mul_table        out[r, :] = gelu_tanh(g[r, :]) * table[token(r), off : off + n]            token(r) = tokens[rows ? rows[r] : r]
//   rms_norm_rows         out = x / sqrt(mean(x^2) + eps) * w for rows x of a wider matrix (row stride ld)
//   xielu                 z > 0: softplus(p) z^2 + z / 2;  else (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
//   tanh_cap              z <- cap * tanh(z / cap), in place
//   normed_add_rms_norm   x += y / sqrt(mean(y^2) + eps_y) * u [+ e]  (a sub-layer output that passes a norm of its own before
//                         it joins the stream; e: a second float32 addend);  out = x / sqrt(mean(x^2) + eps) * w    (each optional)
//
// `A` is the activation type; sums, norms and the stream are float32.  A row's result depends on that row only.
#include "common.cuh"
#include <initializer_list>

namespace iian {

template <typename A>
__global__ void scaled_add_rms_norm_kernel(float * __restrict__ residual, const A * __restrict__ delta, float mult,
                                           const float * __restrict__ weight, A * __restrict__ out, A * __restrict__ copy,
                                           int H, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const size_t base = (size_t) blockIdx.x * H;
    float * r = residual + base;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (delta != nullptr) {
            v = fmaf(mult, to_f32(delta[base + i]), v);
            r[i] = v;
        }
        if (copy != nullptr) copy[base + i] = from_f32<A>(v);
        ss = fmaf(v, v, ss);
    }
    if (out == nullptr) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float) H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[base + i] = from_f32<A>(r[i] * inv * weight[i]);
}

template <typename A>
__global__ void scaled_add_unit_rms_kernel(float * __restrict__ residual, const A * __restrict__ y, float mult,
                                           const float * __restrict__ weight, int H, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const size_t base = (size_t) blockIdx.x * H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_f32(y[base + i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = mult / sqrtf(ss / (float) H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        residual[base + i] = fmaf(to_f32(y[base + i]) * inv, weight[i], residual[base + i]);
}

// ---- the same with four entries per access and the row kept in registers between the two passes -------------------------
// (H a multiple of 4, at most blockDim.x * 4 * KEEP entries, every pointer aligned to four entries)
constexpr int kRowKeep = 4;

__device__ __forceinline__ float4 load4(const float * p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16 * p) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float * p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16 * p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned *>(&a);
    raw.y = *reinterpret_cast<unsigned *>(&b);
    *reinterpret_cast<uint2 *>(p) = raw;
}

template <typename A>
__global__ void scaled_add_rms_norm_vec_kernel(float * __restrict__ residual, const A * __restrict__ delta, float mult,
                                               const float * __restrict__ weight, A * __restrict__ out, A * __restrict__ copy,
                                               int H, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const size_t base = (size_t) blockIdx.x * H;
    float4 v[kRowKeep];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < kRowKeep; k++) {
        const int i = 4 * (threadIdx.x + k * blockDim.x);
        v[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < H) v[k] = load4(residual + base + i);
    }
    if (delta != nullptr) {
#pragma unroll
        for (int k = 0; k < kRowKeep; k++) {
            const int i = 4 * (threadIdx.x + k * blockDim.x);
            if (i < H) {
                const float4 d = load4(delta + base + i);
                v[k].x = fmaf(mult, d.x, v[k].x); v[k].y = fmaf(mult, d.y, v[k].y);
                v[k].z = fmaf(mult, d.z, v[k].z); v[k].w = fmaf(mult, d.w, v[k].w);
                store4(residual + base + i, v[k]);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < kRowKeep; k++) {
        const int i = 4 * (threadIdx.x + k * blockDim.x);
        if (i < H && copy != nullptr) store4(copy + base + i, v[k]);
        ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss);
        ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss);
    }
    if (out == nullptr) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float) H + eps);
#pragma unroll
    for (int k = 0; k < kRowKeep; k++) {
        const int i = 4 * (threadIdx.x + k * blockDim.x);
        if (i < H) {
            const float4 w = load4(weight + i);
            store4(out + base + i, make_float4(v[k].x * inv * w.x, v[k].y * inv * w.y, v[k].z * inv * w.z, v[k].w * inv * w.w));
        }
    }
}

template <typename A>
__global__ void scaled_add_unit_rms_vec_kernel(float * __restrict__ residual, const A * __restrict__ y, float mult,
                                               const float * __restrict__ weight, int H, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const size_t base = (size_t) blockIdx.x * H;
    float4 v[kRowKeep], r[kRowKeep], w[kRowKeep];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < kRowKeep; k++) {
        const int i = 4 * (threadIdx.x + k * blockDim.x);
        v[k] = r[k] = w[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < H) {
            v[k] = load4(y + base + i);
            r[k] = load4(residual + base + i);
            w[k] = load4(weight + i);
        }
        ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss);
        ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = mult / sqrtf(ss / (float) H + eps);
#pragma unroll
    for (int k = 0; k < kRowKeep; k++) {
        const int i = 4 * (threadIdx.x + k * blockDim.x);
        if (i < H)
            store4(residual + base + i, make_float4(fmaf(v[k].x * inv, w[k].x, r[k].x), fmaf(v[k].y * inv, w[k].y, r[k].y),
                                                    fmaf(v[k].z * inv, w[k].z, r[k].z), fmaf(v[k].w * inv, w[k].w, r[k].w)));
    }
}

// threads of a block for the vector forms, or 0: the row does not fit them (not a multiple of 4, too long, not aligned)
static int row_vec_threads(int H, int elem_bytes, std::initializer_list<const void *> act_ptrs, std::initializer_list<const void *> f32_ptrs) {
    if (H % 4 != 0 || H > 1024 * 4 * kRowKeep) return 0;
    for (const void * p : act_ptrs) if ((uintptr_t) p % (4 * elem_bytes)) return 0;
    for (const void * p : f32_ptrs) if ((uintptr_t) p % 16) return 0;
    int t = 128;
    while (t * 4 * kRowKeep < H) t *= 2;
    // short rows: spread over more threads than one access each needs, so that a row's latency is one trip
    while (t < 256 && t * 4 < H) t *= 2;
    return t;
}

template <typename A>
__global__ void rms_norm_rows_kernel(const A * __restrict__ x, long long ld, const float * __restrict__ weight,
                                     A * __restrict__ out, int H, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const A * r = x + (size_t) blockIdx.x * ld;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_f32(r[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float) H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        out[(size_t) blockIdx.x * H + i] = from_f32<A>(to_f32(r[i]) * inv * weight[i]);
}

__device__ __forceinline__ float gelu_tanh_f32(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename A, typename W>
__global__ void gelu_mul_table_kernel(const A * __restrict__ g, const W * __restrict__ table, long long ld_table, int off,
                                      const int * __restrict__ tokens, const int * __restrict__ rows, A * __restrict__ out,
                                      long long total, int n, int vocab) {
    pdl_wait();
    pdl_launch_dependents();
    const long long e = (long long) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const long long r = e / n;
    const int c = (int) (e - r * n);
    int tok = tokens[rows != nullptr ? rows[r] : r];
    tok = min(max(tok, 0), vocab - 1);
    out[e] = from_f32<A>(gelu_tanh_f32(to_f32(g[e])) * to_f32(table[(size_t) tok * ld_table + off + c]));
}

__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

template <typename A>
__global__ void xielu_kernel(const A * __restrict__ x, const float * __restrict__ pq, A * __restrict__ out, long long total) {
    pdl_wait();
    pdl_launch_dependents();
    const long long e = (long long) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const float ap = softplus_f(pq[0]), an = 0.5f + softplus_f(pq[1]);
    const float z = to_f32(x[e]);
    const float y = z > 0.0f ? fmaf(ap * z, z, 0.5f * z) : fmaf(an, expm1f(z) - z, 0.5f * z);
    out[e] = from_f32<A>(y);
}

// exp(z) - 1 - z for z <= 0.  32-bit rows keep expm1f; bfloat16 rows take the fast exponent: near zero the result is
// added to z / 2, far finer than the row's rounding.
template <typename A> __device__ __forceinline__ float xielu_tail(float z) { return expm1f(z) - z; }
template <> __device__ __forceinline__ float xielu_tail<__nv_bfloat16>(float z) { return __expf(z) - 1.0f - z; }

template <typename A>
__device__ __forceinline__ float4 xielu4(float4 z, float ap, float an) {
    z.x = z.x > 0.0f ? fmaf(ap * z.x, z.x, 0.5f * z.x) : fmaf(an, xielu_tail<A>(z.x), 0.5f * z.x);
    z.y = z.y > 0.0f ? fmaf(ap * z.y, z.y, 0.5f * z.y) : fmaf(an, xielu_tail<A>(z.y), 0.5f * z.y);
    z.z = z.z > 0.0f ? fmaf(ap * z.z, z.z, 0.5f * z.z) : fmaf(an, xielu_tail<A>(z.z), 0.5f * z.z);
    z.w = z.w > 0.0f ? fmaf(ap * z.w, z.w, 0.5f * z.w) : fmaf(an, xielu_tail<A>(z.w), 0.5f * z.w);
    return z;
}

// four entries at a time (total a multiple of 4, both pointers aligned to four entries); a thread takes kXieluQuads quads a
// block's width apart, all loads issued before the first use
constexpr int kXieluQuads = 4;
template <typename A>
__global__ void xielu_vec_kernel(const A * __restrict__ x, const float * __restrict__ pq, A * __restrict__ out, long long quads) {
    pdl_wait();
    pdl_launch_dependents();
    const long long e0 = (long long) blockIdx.x * blockDim.x * kXieluQuads + threadIdx.x;
    float4 z[kXieluQuads];
#pragma unroll
    for (int i = 0; i < kXieluQuads; i++) {
        const long long e = e0 + (long long) i * blockDim.x;
        if (e < quads) z[i] = load4(x + 4 * e);
    }
    const float ap = softplus_f(pq[0]), an = 0.5f + softplus_f(pq[1]);
#pragma unroll
    for (int i = 0; i < kXieluQuads; i++) {
        const long long e = e0 + (long long) i * blockDim.x;
        if (e < quads) store4(out + 4 * e, xielu4<A>(z[i], ap, an));
    }
}

__global__ void tanh_cap_kernel(float * __restrict__ x, float cap, long long total) {
    pdl_wait();
    pdl_launch_dependents();
    const long long e = (long long) blockIdx.x * blockDim.x + threadIdx.x;
    if (e < total) x[e] = cap * tanhf(x[e] / cap);
}

// ---- a normalised addend, then the next norm: both of a row in one pass over registers -----------------------------------
// y (optional), u (optional: without it y is added as it is), e (optional float32 rows), w / out (optional)
template <typename A>
__global__ void normed_add_rms_norm_kernel(float * __restrict__ residual, const A * __restrict__ y, const float * __restrict__ u,
                                           float eps_y, const float * __restrict__ extra, const float * __restrict__ weight,
                                           A * __restrict__ out, int H, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const size_t base = (size_t) blockIdx.x * H;
    float * r = residual + base;
    float inv_y = 1.0f;
    if (y != nullptr && u != nullptr) {
        float sy = 0.0f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = to_f32(y[base + i]);
            sy = fmaf(v, v, sy);
        }
        sy = block_sum(sy, scratch);
        inv_y = 1.0f / sqrtf(sy / (float) H + eps_y);
    }
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (y != nullptr) v += u != nullptr ? to_f32(y[base + i]) * inv_y * u[i] : to_f32(y[base + i]);
        if (extra != nullptr) v += extra[base + i];
        r[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (out == nullptr) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float) H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[base + i] = from_f32<A>(r[i] * inv * weight[i]);
}

template <typename A>
__global__ void normed_add_rms_norm_vec_kernel(float * __restrict__ residual, const A * __restrict__ y, const float * __restrict__ u,
                                               float eps_y, const float * __restrict__ extra, const float * __restrict__ weight,
                                               A * __restrict__ out, int H, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const size_t base = (size_t) blockIdx.x * H;
    float4 v[kRowKeep], a[kRowKeep];
#pragma unroll
    for (int k = 0; k < kRowKeep; k++) {
        const int i = 4 * (threadIdx.x + k * blockDim.x);
        v[k] = a[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < H) {
            v[k] = load4(residual + base + i);
            if (y != nullptr) a[k] = load4(y + base + i);
        }
    }
    if (y != nullptr && u != nullptr) {
        float sy = 0.0f;
#pragma unroll
        for (int k = 0; k < kRowKeep; k++) {
            sy = fmaf(a[k].x, a[k].x, sy); sy = fmaf(a[k].y, a[k].y, sy);
            sy = fmaf(a[k].z, a[k].z, sy); sy = fmaf(a[k].w, a[k].w, sy);
        }
        sy = block_sum(sy, scratch);
        const float inv_y = 1.0f / sqrtf(sy / (float) H + eps_y);
#pragma unroll
        for (int k = 0; k < kRowKeep; k++) {
            const int i = 4 * (threadIdx.x + k * blockDim.x);
            if (i < H) {
                const float4 w4 = load4(u + i);
                a[k].x = a[k].x * inv_y * w4.x; a[k].y = a[k].y * inv_y * w4.y;
                a[k].z = a[k].z * inv_y * w4.z; a[k].w = a[k].w * inv_y * w4.w;
            }
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < kRowKeep; k++) {
        const int i = 4 * (threadIdx.x + k * blockDim.x);
        if (i < H) {
            v[k].x += a[k].x; v[k].y += a[k].y; v[k].z += a[k].z; v[k].w += a[k].w;
            if (extra != nullptr) {
                const float4 e4 = load4(extra + base + i);
                v[k].x += e4.x; v[k].y += e4.y; v[k].z += e4.z; v[k].w += e4.w;
            }
            if (y != nullptr || extra != nullptr) store4(residual + base + i, v[k]);
        }
        ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss);
        ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss);
    }
    if (out == nullptr) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float) H + eps);
#pragma unroll
    for (int k = 0; k < kRowKeep; k++) {
        const int i = 4 * (threadIdx.x + k * blockDim.x);
        if (i < H) {
            const float4 w4 = load4(weight + i);
            store4(out + base + i, make_float4(v[k].x * inv * w4.x, v[k].y * inv * w4.y, v[k].z * inv * w4.z, v[k].w * inv * w4.w));
        }
    }
}

}  // namespace iian

using namespace iian;

// delta, out, copy may be null: without delta nothing is added; without out no norm is taken; copy receives the new
// stream in the activation type.
IIAN_API int iian_scaled_add_rms_norm(float * residual, const void * delta, float mult, const float * weight, void * out,
                                      void * copy, int act_dtype, int N, int H, float eps, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (H <= 0) return IIAN_ERR_SHAPE;
    if (act_dtype != IIAN_F32 && act_dtype != IIAN_BF16) return IIAN_ERR_DTYPE;
    if (const int vt = row_vec_threads(H, act_dtype == IIAN_F32 ? 4 : 2, {delta, out, copy}, {residual, weight})) {
        if (act_dtype == IIAN_F32)
            return iian_launch(scaled_add_rms_norm_vec_kernel<float>, dim3(N), dim3(vt), 0, stream, residual, (const float *) delta,
                               mult, weight, (float *) out, (float *) copy, H, eps);
        return iian_launch(scaled_add_rms_norm_vec_kernel<__nv_bfloat16>, dim3(N), dim3(vt), 0, stream, residual,
                           (const __nv_bfloat16 *) delta, mult, weight, (__nv_bfloat16 *) out, (__nv_bfloat16 *) copy, H, eps);
    }
    const int threads = H >= 1024 ? 256 : 128;
    if (act_dtype == IIAN_F32)
        return iian_launch(scaled_add_rms_norm_kernel<float>, dim3(N), dim3(threads), 0, stream, residual, (const float *) delta,
                           mult, weight, (float *) out, (float *) copy, H, eps);
    if (act_dtype == IIAN_BF16)
        return iian_launch(scaled_add_rms_norm_kernel<__nv_bfloat16>, dim3(N), dim3(threads), 0, stream, residual,
                           (const __nv_bfloat16 *) delta, mult, weight, (__nv_bfloat16 *) out, (__nv_bfloat16 *) copy, H, eps);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_scaled_add_unit_rms(float * residual, const void * y, float mult, const float * weight, int act_dtype, int N,
                                      int H, float eps, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (H <= 0) return IIAN_ERR_SHAPE;
    if (act_dtype != IIAN_F32 && act_dtype != IIAN_BF16) return IIAN_ERR_DTYPE;
    if (const int vt = row_vec_threads(H, act_dtype == IIAN_F32 ? 4 : 2, {y}, {residual, weight})) {
        if (act_dtype == IIAN_F32)
            return iian_launch(scaled_add_unit_rms_vec_kernel<float>, dim3(N), dim3(vt), 0, stream, residual, (const float *) y, mult,
                               weight, H, eps);
        return iian_launch(scaled_add_unit_rms_vec_kernel<__nv_bfloat16>, dim3(N), dim3(vt), 0, stream, residual,
                           (const __nv_bfloat16 *) y, mult, weight, H, eps);
    }
    const int threads = H >= 1024 ? 256 : 128;
    if (act_dtype == IIAN_F32)
        return iian_launch(scaled_add_unit_rms_kernel<float>, dim3(N), dim3(threads), 0, stream, residual, (const float *) y, mult,
                           weight, H, eps);
    if (act_dtype == IIAN_BF16)
        return iian_launch(scaled_add_unit_rms_kernel<__nv_bfloat16>, dim3(N), dim3(threads), 0, stream, residual,
                           (const __nv_bfloat16 *) y, mult, weight, H, eps);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_rms_norm_rows(const void * x, long long ld, const float * weight, void * out, int act_dtype, int N, int H,
                                float eps, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (H <= 0) return IIAN_ERR_SHAPE;
    const int threads = H >= 1024 ? 256 : 128;
    if (act_dtype == IIAN_F32)
        return iian_launch(rms_norm_rows_kernel<float>, dim3(N), dim3(threads), 0, stream, (const float *) x, ld, weight, (float *) out, H, eps);
    if (act_dtype == IIAN_BF16)
        return iian_launch(rms_norm_rows_kernel<__nv_bfloat16>, dim3(N), dim3(threads), 0, stream, (const __nv_bfloat16 *) x, ld, weight,
                           (__nv_bfloat16 *) out, H, eps);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_gelu_mul_table(const void * g, const void * table, int table_dtype, long long ld_table, int off,
                                 const int * tokens, const int * rows, void * out, int act_dtype, int R, int n, int vocab,
                                 cudaStream_t stream) {
    const long long total = (long long) R * n;
    if (total <= 0) return IIAN_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned) ((total + threads - 1) / threads);
    if (act_dtype == IIAN_F32 && table_dtype == IIAN_F32)
        return iian_launch(gelu_mul_table_kernel<float, float>, dim3(blocks), dim3(threads), 0, stream, (const float *) g,
                           (const float *) table, ld_table, off, tokens, rows, (float *) out, total, n, vocab);
    if (act_dtype == IIAN_BF16 && table_dtype == IIAN_BF16)
        return iian_launch(gelu_mul_table_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream,
                           (const __nv_bfloat16 *) g, (const __nv_bfloat16 *) table, ld_table, off, tokens, rows,
                           (__nv_bfloat16 *) out, total, n, vocab);
    if (act_dtype == IIAN_BF16 && table_dtype == IIAN_F32)
        return iian_launch(gelu_mul_table_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(threads), 0, stream,
                           (const __nv_bfloat16 *) g, (const float *) table, ld_table, off, tokens, rows, (__nv_bfloat16 *) out,
                           total, n, vocab);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_xielu(const void * x, const float * pq, void * out, int act_dtype, long long total, cudaStream_t stream) {
    if (total <= 0) return IIAN_OK;
    const int threads = 256;
    const int eb = act_dtype == IIAN_F32 ? 4 : 2;
    if (total % 4 == 0 && (uintptr_t) x % (4 * eb) == 0 && (uintptr_t) out % (4 * eb) == 0 && (act_dtype == IIAN_F32 || act_dtype == IIAN_BF16)) {
        const long long quads = total / 4;
        const unsigned vb = (unsigned) ((quads + (long long) threads * kXieluQuads - 1) / ((long long) threads * kXieluQuads));
        if (act_dtype == IIAN_F32)
            return iian_launch(xielu_vec_kernel<float>, dim3(vb), dim3(threads), 0, stream, (const float *) x, pq, (float *) out, quads);
        return iian_launch(xielu_vec_kernel<__nv_bfloat16>, dim3(vb), dim3(threads), 0, stream, (const __nv_bfloat16 *) x, pq,
                           (__nv_bfloat16 *) out, quads);
    }
    const unsigned blocks = (unsigned) ((total + threads - 1) / threads);
    if (act_dtype == IIAN_F32)
        return iian_launch(xielu_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float *) x, pq, (float *) out, total);
    if (act_dtype == IIAN_BF16)
        return iian_launch(xielu_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16 *) x, pq,
                           (__nv_bfloat16 *) out, total);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_tanh_cap(float * x, float cap, long long total, cudaStream_t stream) {
    if (total <= 0) return IIAN_OK;
    if (!(cap > 0.0f)) return IIAN_ERR_SHAPE;
    const int threads = 256;
    const unsigned blocks = (unsigned) ((total + threads - 1) / threads);
    return iian_launch(tanh_cap_kernel, dim3(blocks), dim3(threads), 0, stream, x, cap, total);
}

// residual: f32 [N, H] in place; y: A [N, H] or null; u: f32 [H] or null (y joins the stream as it is); extra: f32 [N, H] or
// null; weight f32 [H] and out A [N, H]: both or neither.
IIAN_API int iian_normed_add_rms_norm(float * residual, const void * y, const float * u, float eps_y, const float * extra,
                                      const float * weight, void * out, int act_dtype, int N, int H, float eps,
                                      cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (H <= 0 || (out != nullptr && weight == nullptr)) return IIAN_ERR_SHAPE;
    if (act_dtype != IIAN_F32 && act_dtype != IIAN_BF16) return IIAN_ERR_DTYPE;
    if (const int vt = row_vec_threads(H, act_dtype == IIAN_F32 ? 4 : 2, {y, out}, {residual, u, extra, weight})) {
        if (act_dtype == IIAN_F32)
            return iian_launch(normed_add_rms_norm_vec_kernel<float>, dim3(N), dim3(vt), 0, stream, residual, (const float *) y, u,
                               eps_y, extra, weight, (float *) out, H, eps);
        return iian_launch(normed_add_rms_norm_vec_kernel<__nv_bfloat16>, dim3(N), dim3(vt), 0, stream, residual,
                           (const __nv_bfloat16 *) y, u, eps_y, extra, weight, (__nv_bfloat16 *) out, H, eps);
    }
    const int threads = H >= 1024 ? 256 : 128;
    if (act_dtype == IIAN_F32)
        return iian_launch(normed_add_rms_norm_kernel<float>, dim3(N), dim3(threads), 0, stream, residual, (const float *) y, u,
                           eps_y, extra, weight, (float *) out, H, eps);
    return iian_launch(normed_add_rms_norm_kernel<__nv_bfloat16>, dim3(N), dim3(threads), 0, stream, residual,
                       (const __nv_bfloat16 *) y, u, eps_y, extra, weight, (__nv_bfloat16 *) out, H, eps);
}
