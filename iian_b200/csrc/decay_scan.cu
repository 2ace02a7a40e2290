// Linear attention with a decay: a matrix state per head that every token multiplies row by row and adds an outer product to,
//
//     S_t = diag(a_t) S_{t-1} + k_t v_t^T          o_t = S_t^T q_t          S: [d, dv] float32, zero at a request's start
//
// with the decay a_t either one constant per head (the same for every key channel and token) or one number per key channel
// and token, a_t = sigmoid(z_t + b)^(1/tau) from a float32 pre-activation z.  q, k, v come out of a stacked projection in the
// activation type and may pass silu on the way in; q takes a factor.  Decays, their logarithms, the state, every product and
// sum of the recurrence and the read-out are float32.
//
// The columns of S are independent (column j: s_j <- a * s_j + k v_j; o_j = q . s_j), so a CTA owns 16 of them for one
// (sequence, head): L lanes per column hold the column in registers (entries lane, lane + L, ...), the step's tokens of that
// sequence pass in order, a chunk at a time through shared memory (transformed once per CTA: activation, factor, decay), and a
// token's read-out is one shuffle tree over the L lanes -- four tokens' trees are issued together, since only the update of
// s lies on the chain from token to token.  Every sum has an order fixed by (d, L), so the result does not depend on how a
// sequence was cut into steps or what else is in the batch.
#include "common.cuh"

namespace iian {

constexpr int kDsCols = 16;

struct DecayScanParams {
    const void * proj;            // A [n, ld]
    long long ld;
    int q_off, k_off, v_off;
    int act;                      // 0: as projected; 1: silu on q, k and v
    float q_scale;
    const float * head_decay;     // f32 [H] or null
    const float * z;              // f32 rows of H * d with row stride ld_z (used without head_decay)
    long long ld_z;
    const float * z_bias;         // f32 [H * d] or null
    float inv_tau;
    float * state;                // f32 [slots, H, d, dv]
    const int * cu_q;             // i32 [S + 1]
    const int * state_slots;      // i32 [S]   (-1: padding sequence)
    float * out;                  // f32 [n, H * dv]
    int H, d, dv, L, dpad, chunk, num_slots;
};

__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }

template <typename A, int EPL>
__global__ void decay_scan_kernel(const DecayScanParams p) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float smem[];
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int L = p.L, d = p.d, dv = p.dv, dpad = p.dpad, H = p.H;
    const int col = tid / L, lane = tid % L;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int col0 = blockIdx.x * kDsCols;
    const int r0 = p.cu_q[seq], r1 = p.cu_q[seq + 1];
    const int slot = p.state_slots[seq];
    const int c = col0 + col;
    const bool col_ok = c < dv;
    if (slot < 0 || slot >= p.num_slots) {        // a padding sequence: its rows read as zero, no state is touched
        if (lane == 0 && col_ok)
            for (int r = r0; r < r1; r++) p.out[(size_t) r * H * dv + (size_t) h * dv + c] = 0.0f;
        return;
    }
    const bool per_channel = p.head_decay == nullptr;
    float * q_s = smem;
    float * k_s = q_s + (size_t) p.chunk * dpad;
    float * v_s = k_s + (size_t) p.chunk * dpad;
    float * a_s = v_s + (size_t) p.chunk * kDsCols;      // only with a decay per channel
    const float a_head = per_channel ? 0.0f : p.head_decay[h];

    float s[EPL];
    float * st = p.state + ((size_t) slot * H + h) * d * dv;
#pragma unroll
    for (int e = 0; e < EPL; e++) {
        const int i = lane + e * L;
        s[e] = (col_ok && i < d) ? st[(size_t) i * dv + c] : 0.0f;
    }
    const A * proj = (const A *) p.proj;

    for (int cr = r0; cr < r1; cr += p.chunk) {
        const int cnt = min(p.chunk, r1 - cr);
        __syncthreads();                                  // the chunk before has been read by everyone
        for (int idx = tid; idx < cnt * dpad; idx += nthreads) {
            const int t = idx / dpad, i = idx - t * dpad;
            float qv = 0.0f, kv = 0.0f, av = 0.0f;
            if (i < d) {
                const A * row = proj + (size_t) (cr + t) * p.ld;
                qv = to_f32(row[p.q_off + h * d + i]);
                kv = to_f32(row[p.k_off + h * d + i]);
                if (p.act == 1) { qv = silu_f32(qv); kv = silu_f32(kv); }
                qv *= p.q_scale;
                if (per_channel) {
                    float zz = p.z[(size_t) (cr + t) * p.ld_z + h * d + i];
                    if (p.z_bias != nullptr) zz += p.z_bias[h * d + i];
                    const float logsig = fminf(zz, 0.0f) - log1pf(expf(-fabsf(zz)));
                    av = expf(logsig * p.inv_tau);
                }
            }
            q_s[idx] = qv;
            k_s[idx] = kv;
            if (per_channel) a_s[idx] = av;
        }
        for (int idx = tid; idx < cnt * kDsCols; idx += nthreads) {
            const int t = idx / kDsCols, j = idx - t * kDsCols;
            float vv = 0.0f;
            if (col0 + j < dv) {
                vv = to_f32(proj[(size_t) (cr + t) * p.ld + p.v_off + h * dv + col0 + j]);
                if (p.act == 1) vv = silu_f32(vv);
            }
            v_s[idx] = vv;
        }
        __syncthreads();
        for (int t4 = 0; t4 < cnt; t4 += 4) {
            float part[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                part[u] = 0.0f;
                const int t = t4 + u;
                if (t < cnt) {
                    const float vj = v_s[t * kDsCols + col];
                    const float * qr = q_s + (size_t) t * dpad + lane;
                    const float * kr = k_s + (size_t) t * dpad + lane;
                    const float * ar = a_s + (size_t) t * dpad + lane;
#pragma unroll
                    for (int e = 0; e < EPL; e++) {
                        const float a = per_channel ? ar[e * L] : a_head;
                        s[e] = fmaf(a, s[e], __fmul_rn(kr[e * L], vj));
                        part[u] = fmaf(qr[e * L], s[e], part[u]);
                    }
                }
            }
            for (int o = L >> 1; o > 0; o >>= 1) {
#pragma unroll
                for (int u = 0; u < 4; u++) part[u] += __shfl_xor_sync(0xffffffffu, part[u], o);
            }
            if (lane == 0 && col_ok) {
#pragma unroll
                for (int u = 0; u < 4; u++)
                    if (t4 + u < cnt) p.out[(size_t) (cr + t4 + u) * H * dv + (size_t) h * dv + c] = part[u];
            }
        }
    }
    if (col_ok) {
#pragma unroll
        for (int e = 0; e < EPL; e++) {
            const int i = lane + e * L;
            if (i < d) st[(size_t) i * dv + c] = s[e];
        }
    }
}

}  // namespace iian

using namespace iian;

// lanes that share a column of the state for heads of d key channels
IIAN_API int iian_decay_scan_lanes(int d) {
    int L = 4;
    while (L < 32 && d > 8 * L) L *= 2;
    return L;
}

// proj: A rows [.. q (H * d) .. k (H * d) .. v (H * dv) ..] at the given column offsets, row stride ld.
// head_decay: f32 [H] (one constant decay per head) or null, then z: f32 rows of H * d (row stride ld_z), z_bias f32 [H * d]
// or null, inv_tau.  state: f32 [num_slots, H, d, dv].  out: f32 [n, H * dv].  max_q_len: the longest portion of the step
// (sizes the chunks; 0: unknown).
IIAN_API int iian_decay_scan(const void * proj, long long ld, int q_off, int k_off, int v_off, int act, float q_scale,
                             const float * head_decay, const float * z, long long ld_z, const float * z_bias, float inv_tau,
                             float * state, const int * cu_q, const int * state_slots, float * out, int act_dtype, int S, int H,
                             int d, int dv, int num_slots, int max_q_len, cudaStream_t stream) {
    if (S <= 0) return IIAN_OK;
    if (H <= 0 || d <= 0 || d > 512 || dv <= 0 || (act != 0 && act != 1)) return IIAN_ERR_SHAPE;
    if (head_decay == nullptr && z == nullptr) return IIAN_ERR_SHAPE;
    if (S > 65535 || H > 65535) return IIAN_ERR_LIMIT;
    DecayScanParams p;
    p.proj = proj; p.ld = ld; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.act = act; p.q_scale = q_scale;
    p.head_decay = head_decay; p.z = z; p.ld_z = ld_z; p.z_bias = z_bias; p.inv_tau = inv_tau;
    p.state = state; p.cu_q = cu_q; p.state_slots = state_slots; p.out = out;
    p.H = H; p.d = d; p.dv = dv; p.num_slots = num_slots;
    p.L = iian_decay_scan_lanes(d);
    const int epl = (d + p.L - 1) / p.L > 8 ? 16 : 8;
    p.dpad = p.L * epl;
    int chunk = d <= 128 ? 16 : d <= 256 ? 8 : 4;
    if (max_q_len > 0 && max_q_len < chunk) chunk = max_q_len;
    p.chunk = chunk;
    const size_t smem = ((size_t) chunk * p.dpad * (head_decay == nullptr ? 3 : 2) + (size_t) chunk * kDsCols) * sizeof(float);
    dim3 grid((dv + kDsCols - 1) / kDsCols, H, S), block(kDsCols * p.L);
#define IIAN_DS(AT, E) return iian_launch(decay_scan_kernel<AT, E>, grid, block, smem, stream, p)
    if (act_dtype == IIAN_F32) { if (epl == 8) IIAN_DS(float, 8); IIAN_DS(float, 16); }
    if (act_dtype == IIAN_BF16) { if (epl == 8) IIAN_DS(__nv_bfloat16, 8); IIAN_DS(__nv_bfloat16, 16); }
#undef IIAN_DS
    return IIAN_ERR_DTYPE;
}
