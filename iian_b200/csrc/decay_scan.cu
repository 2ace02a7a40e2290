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
// (sequence, head): L lanes per column hold the column in registers, four neighbouring entries at a time (entries
// 4 (g L + lane) .. + 3 for g = 0, 1, ..: the lanes of a column read neighbouring 16-byte pieces of a token's row).  The step's
// tokens of that sequence pass in order, a chunk at a time through shared memory, transformed once per CTA on the way in
// (activation, factor, decay); with bfloat16 rows that are 16-byte aligned the next chunk's rows are fetched into registers
// while the current chunk is walked.  A token's read-out is one shuffle tree over the L lanes -- four tokens' trees are issued
// together, since only the update of s lies on the chain from token to token.  Every sum has an order fixed by (d, L), so the
// result does not depend on how a sequence was cut into steps or what else is in the batch.
//
// The state is stored column by column in blocks of 16 columns, [slot][head][block][16][d4] with d4 = d rounded up to a multiple
// of 4: a CTA's share is one contiguous piece, a lane's entries are 16-byte pieces of its column, and the lanes of a column
// read neighbouring pieces -- the state goes straight between global memory and registers.
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
    float * state;                // f32 [slots, H, blocks, 16, d4]
    const int * cu_q;             // i32 [S + 1]
    const int * state_slots;      // i32 [S]   (-1: padding sequence)
    float * out;                  // f32 [n, H * dv]
    int H, d, dv, L, dpad, chunk, num_slots;
};

__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float decay_of(float zz, float inv_tau) {       // sigmoid(zz)^(1/tau) through the logarithm
    const float logsig = fminf(zz, 0.0f) - log1pf(expf(-fabsf(zz)));
    return expf(logsig * inv_tau);
}

// VEC: A is bfloat16 and every row piece the kernel reads starts on a 16-byte boundary (d, the column offsets and ld are
// multiples of 8, the base pointers aligned): pieces of 8 entries are fetched a chunk ahead into registers.
template <typename A, int EPL, bool VEC>
__global__ void decay_scan_kernel(const DecayScanParams p) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float smem[];
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

    // ---- the state: a column is contiguous (d rounded up to a multiple of 4 floats), a lane's pieces are 16 bytes each ---------
    float s[EPL];
    const int d4 = (d + 3) & ~3;
    float * st = p.state + ((((size_t) slot * H + h) * gridDim.x + blockIdx.x) * kDsCols + col) * (size_t) d4;
#pragma unroll
    for (int g = 0; g < EPL / 4; g++) {
        const int i4 = 4 * (g * L + lane);
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (col_ok && i4 < d4) v = *reinterpret_cast<const float4 *>(st + i4);
        s[4 * g + 0] = v.x; s[4 * g + 1] = v.y; s[4 * g + 2] = v.z; s[4 * g + 3] = v.w;
    }
    const A * proj = (const A *) p.proj;

    // ---- fetching a chunk ------------------------------------------------------------------------------------------------------
    constexpr int GP = 2, VP = 4;                         // pieces of 8 entries and single values a thread fetches per chunk
    const int pieces_per_token = d / 8;
    uint4 rq[GP] = {}, rk[GP] = {};
    float4 rz[GP][2] = {};
    unsigned short rv[VP] = {};
    auto fetch = [&](int cr, int cnt) {                   // VEC: the chunk's rows into registers
#pragma unroll
        for (int g = 0; g < GP; g++) {
            const int pc = tid + g * nthreads;
            if (pc < cnt * pieces_per_token) {
                const int t = pc / pieces_per_token, i = (pc - t * pieces_per_token) * 8;
                const __nv_bfloat16 * row = reinterpret_cast<const __nv_bfloat16 *>(proj) + (size_t) (cr + t) * p.ld + h * d + i;
                rq[g] = *reinterpret_cast<const uint4 *>(row + p.q_off);
                rk[g] = *reinterpret_cast<const uint4 *>(row + p.k_off);
                if (per_channel) {
                    const float * zr = p.z + (size_t) (cr + t) * p.ld_z + h * d + i;
                    rz[g][0] = *reinterpret_cast<const float4 *>(zr);
                    rz[g][1] = *reinterpret_cast<const float4 *>(zr + 4);
                }
            }
        }
#pragma unroll
        for (int g = 0; g < VP; g++) {
            const int idx = tid + g * nthreads;
            if (idx < cnt * kDsCols) {
                const int t = idx / kDsCols, j = idx - t * kDsCols;
                rv[g] = col0 + j < dv ? reinterpret_cast<const unsigned short *>(proj)[(size_t) (cr + t) * p.ld + p.v_off + h * dv + col0 + j] : 0;
            }
        }
    };
    auto put = [&](int cnt) {                             // VEC: registers, transformed, into shared memory
#pragma unroll
        for (int g = 0; g < GP; g++) {
            const int pc = tid + g * nthreads;
            if (pc < cnt * pieces_per_token) {
                const int t = pc / pieces_per_token, i = (pc - t * pieces_per_token) * 8;
                float qf[8], kf[8];
                unpack8(rq[g], qf);
                unpack8(rk[g], kf);
                const float zf[8] = {rz[g][0].x, rz[g][0].y, rz[g][0].z, rz[g][0].w, rz[g][1].x, rz[g][1].y, rz[g][1].z, rz[g][1].w};
                float af[8];
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    if (p.act == 1) { qf[e] = silu_f32(qf[e]); kf[e] = silu_f32(kf[e]); }
                    qf[e] *= p.q_scale;
                    af[e] = per_channel ? decay_of(zf[e] + (p.z_bias != nullptr ? p.z_bias[h * d + i + e] : 0.0f), p.inv_tau) : 0.0f;
                }
                float4 * qd = reinterpret_cast<float4 *>(q_s + t * dpad + i);
                float4 * kd = reinterpret_cast<float4 *>(k_s + t * dpad + i);
                qd[0] = make_float4(qf[0], qf[1], qf[2], qf[3]); qd[1] = make_float4(qf[4], qf[5], qf[6], qf[7]);
                kd[0] = make_float4(kf[0], kf[1], kf[2], kf[3]); kd[1] = make_float4(kf[4], kf[5], kf[6], kf[7]);
                if (per_channel) {
                    float4 * ad = reinterpret_cast<float4 *>(a_s + t * dpad + i);
                    ad[0] = make_float4(af[0], af[1], af[2], af[3]); ad[1] = make_float4(af[4], af[5], af[6], af[7]);
                }
            }
        }
#pragma unroll
        for (int g = 0; g < VP; g++) {
            const int idx = tid + g * nthreads;
            if (idx < cnt * kDsCols) {
                float vv = __bfloat162float(__ushort_as_bfloat16(rv[g]));
                if (p.act == 1) vv = silu_f32(vv);
                v_s[idx] = vv;
            }
        }
    };
    auto fill = [&](int cr, int cnt) {                    // the general way: straight from global memory, one entry at a time
        for (int idx = tid; idx < cnt * d; idx += nthreads) {
            const int t = idx / d, i = idx - t * d;
            const A * row = proj + (size_t) (cr + t) * p.ld;
            float qv = to_f32(row[p.q_off + h * d + i]), kv = to_f32(row[p.k_off + h * d + i]);
            if (p.act == 1) { qv = silu_f32(qv); kv = silu_f32(kv); }
            q_s[t * dpad + i] = qv * p.q_scale;
            k_s[t * dpad + i] = kv;
            if (per_channel)
                a_s[t * dpad + i] = decay_of(p.z[(size_t) (cr + t) * p.ld_z + h * d + i] + (p.z_bias != nullptr ? p.z_bias[h * d + i] : 0.0f), p.inv_tau);
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
    };

    if (VEC && r0 < r1) fetch(r0, min(p.chunk, r1 - r0));
    // entries of a row beyond d (the lanes' padding) are zero for good
    for (int idx = tid; idx < p.chunk * (dpad - d); idx += nthreads) {
        const int t = idx / (dpad - d), i = d + idx - t * (dpad - d);
        q_s[t * dpad + i] = 0.0f;
        k_s[t * dpad + i] = 0.0f;
        if (per_channel) a_s[t * dpad + i] = 0.0f;
    }

    for (int cr = r0; cr < r1; cr += p.chunk) {
        const int cnt = min(p.chunk, r1 - cr);
        if (VEC) put(cnt); else fill(cr, cnt);
        __syncthreads();
        if (VEC && cr + p.chunk < r1) fetch(cr + p.chunk, min(p.chunk, r1 - cr - p.chunk));     // in flight while this chunk is walked
        for (int t4 = 0; t4 < cnt; t4 += 4) {
            float part[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                part[u] = 0.0f;
                const int t = t4 + u;
                if (t < cnt) {
                    const float vj = v_s[t * kDsCols + col];
                    const float4 * qr = reinterpret_cast<const float4 *>(q_s + (size_t) t * dpad) + lane;
                    const float4 * kr = reinterpret_cast<const float4 *>(k_s + (size_t) t * dpad) + lane;
                    const float4 * ar = reinterpret_cast<const float4 *>(a_s + (size_t) t * dpad) + lane;
                    float pa = 0.0f, pb = 0.0f;
#pragma unroll
                    for (int g = 0; g < EPL / 4; g++) {
                        const float4 qq = qr[g * L], kk = kr[g * L];
                        float4 aa = make_float4(a_head, a_head, a_head, a_head);
                        if (per_channel) aa = ar[g * L];
                        s[4 * g + 0] = fmaf(aa.x, s[4 * g + 0], __fmul_rn(kk.x, vj));
                        s[4 * g + 1] = fmaf(aa.y, s[4 * g + 1], __fmul_rn(kk.y, vj));
                        s[4 * g + 2] = fmaf(aa.z, s[4 * g + 2], __fmul_rn(kk.z, vj));
                        s[4 * g + 3] = fmaf(aa.w, s[4 * g + 3], __fmul_rn(kk.w, vj));
                        pa = fmaf(qq.x, s[4 * g + 0], pa);
                        pb = fmaf(qq.y, s[4 * g + 1], pb);
                        pa = fmaf(qq.z, s[4 * g + 2], pa);
                        pb = fmaf(qq.w, s[4 * g + 3], pb);
                    }
                    part[u] = pa + pb;
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
        __syncthreads();                                  // the chunk has been read by everyone
    }
    // ---- the state back (entries of a column's last piece beyond d stay zero: their k, q and decay are) ---------------------------
    if (col_ok) {
#pragma unroll
        for (int g = 0; g < EPL / 4; g++) {
            const int i4 = 4 * (g * L + lane);
            if (i4 < d4) *reinterpret_cast<float4 *>(st + i4) = make_float4(s[4 * g + 0], s[4 * g + 1], s[4 * g + 2], s[4 * g + 3]);
        }
    }
}

}  // namespace iian

using namespace iian;

// lanes that share a column of the state for heads of d key channels: `per_lane` entries a lane (8 or 16), at least 4 lanes
static int decay_scan_lanes(int d, int per_lane) {
    int L = 4;
    while (L < 32 && d > per_lane * L) L *= 2;
    return L;
}
static int g_decay_scan_per_lane = 0;          // 0: chosen per launch; 8 or 16: fixed (for measurements)
IIAN_API void iian_decay_scan_set_entries_per_lane(int per_lane) { g_decay_scan_per_lane = per_lane <= 0 ? 0 : per_lane <= 8 ? 8 : 16; }
IIAN_API int iian_decay_scan_lanes(int d) { return decay_scan_lanes(d, 16); }

// floats of one (slot, head) of the state: blocks of 16 columns of d4 = round_up(d, 4) floats each
IIAN_API long long iian_decay_scan_state_floats(int d, int dv) { return (long long) ((dv + kDsCols - 1) / kDsCols) * kDsCols * ((d + 3) & ~3); }

// proj: A rows [.. q (H * d) .. k (H * d) .. v (H * dv) ..] at the given column offsets, row stride ld.
// head_decay: f32 [H] (one constant decay per head) or null, then z: f32 rows of H * d (row stride ld_z), z_bias f32 [H * d]
// or null, inv_tau.  state: f32 [num_slots, H, ceil(dv / 16), 16, round_up(d, 4)].  out: f32 [n, H * dv].  max_q_len: the longest portion of
// the step (sizes the chunks; 0: unknown).
IIAN_API int iian_decay_scan(const void * proj, long long ld, int q_off, int k_off, int v_off, int act, float q_scale,
                             const float * head_decay, const float * z, long long ld_z, const float * z_bias, float inv_tau,
                             float * state, const int * cu_q, const int * state_slots, float * out, int act_dtype, int S, int H,
                             int d, int dv, int num_slots, int max_q_len, cudaStream_t stream) {
    if (S <= 0) return IIAN_OK;
    if (H <= 0 || d <= 0 || d > 512 || dv <= 0 || (act != 0 && act != 1)) return IIAN_ERR_SHAPE;
    if (head_decay == nullptr && z == nullptr) return IIAN_ERR_SHAPE;
    if (S > 65535 || H > 65535) return IIAN_ERR_LIMIT;
    if ((uintptr_t) state & 15) return IIAN_ERR_ALIGN;
    DecayScanParams p;
    p.proj = proj; p.ld = ld; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.act = act; p.q_scale = q_scale;
    p.head_decay = head_decay; p.z = z; p.ld_z = ld_z; p.z_bias = z_bias; p.inv_tau = inv_tau;
    p.state = state; p.cu_q = cu_q; p.state_slots = state_slots; p.out = out;
    p.H = H; p.d = d; p.dv = dv; p.num_slots = num_slots;
    // 16 entries a lane keep the instruction count low; where a step brings long portions of so few sequences that an SM gets
    // one CTA at most, 8 entries a lane (twice the warps) hide more of the chain's latency (0.78 -> 0.64 ms for one portion of
    // 2,048 tokens, 8 heads 128 x 256).  The 32-bit path keeps one form: its sums must not depend on what else is in the batch.
    int per_lane = 16;
    if (act_dtype == IIAN_BF16 && max_q_len >= 64 && (long long) ((dv + kDsCols - 1) / kDsCols) * H * S <= 160) per_lane = 8;
    if (g_decay_scan_per_lane) per_lane = g_decay_scan_per_lane;
    p.L = decay_scan_lanes(d, per_lane);
    const int epl = (d + p.L - 1) / p.L > 8 ? 16 : 8;
    p.dpad = p.L * epl;
    int chunk = d <= 128 ? 16 : d <= 256 ? 8 : 4;
    if (max_q_len > 0 && max_q_len < chunk) chunk = max_q_len;
    p.chunk = chunk;
    const size_t smem = ((size_t) chunk * p.dpad * (head_decay == nullptr ? 3 : 2) + (size_t) chunk * kDsCols) * sizeof(float);
    dim3 grid((dv + kDsCols - 1) / kDsCols, H, S), block(kDsCols * p.L);
    const bool vec = chunk * (d / 8) <= 2 * (int) block.x && chunk * kDsCols <= 4 * (int) block.x && act_dtype == IIAN_BF16 && d % 8 == 0 && ld % 8 == 0 && q_off % 8 == 0 && k_off % 8 == 0 && ((uintptr_t) proj & 15) == 0 &&
                     (head_decay != nullptr || (ld_z % 4 == 0 && ((uintptr_t) z & 15) == 0));
#define IIAN_DS(AT, E, V) return iian_launch(decay_scan_kernel<AT, E, V>, grid, block, smem, stream, p)
    if (act_dtype == IIAN_F32) { if (epl == 8) IIAN_DS(float, 8, false); IIAN_DS(float, 16, false); }
    if (act_dtype == IIAN_BF16) {
        if (vec) { if (epl == 8) IIAN_DS(__nv_bfloat16, 8, true); IIAN_DS(__nv_bfloat16, 16, true); }
        if (epl == 8) IIAN_DS(__nv_bfloat16, 8, false);
        IIAN_DS(__nv_bfloat16, 16, false);
    }
#undef IIAN_DS
    return IIAN_ERR_DTYPE;
}
