// The gated delta rule with a decay per key channel: a recurrent mixer whose state is a matrix S [dim, vdim] per head.
//
// Per token and head, with unit vectors q (times dim^-1/2) and k, a value v, a write strength beta in (0, 1) and a decay
// g in (0, 1) per key channel:
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// q, k and v come out of a short causal convolution over time (one filter per channel, the last tap is the current
// token's) followed by silu; the convolution's last `taps - 1` inputs are part of the state.
//
// The columns of S are independent: column j is a vector s_j of `dim` numbers with
//     s_j <- g * s_j;  u_j = beta (v_j - k . s_j);  s_j <- s_j + k u_j;  o_j = q . s_j = q . (g * s_j) + (q . k) u_j
// so a CTA owns kCols columns of one (sequence, head), kLanes lanes share a column (each holds every kLanes-th entry in
// registers), and both dot products of a token are taken from the decayed column in ONE pass and reduced together.
//
// Kernels:
//   delta_prep   per token and head: convolution + silu over the channels q | k | v (inputs of earlier tokens come from
//                the rows before it in the step, or from the state's tail), unit length of q and k per head, q . k, sigmoid
//                of the write strength, the decay exp(-exp(A) softplus(z + bias)).  Everything it leaves is float32.
//   delta_scan   the recurrence over a step's tokens of every sequence; the tokens' vectors come through two stages of
//                shared memory filled by cp.async a chunk ahead; the CTAs of a sequence also move the convolution's tail
//                on, a share of the channels each.
// State of a slot (float32): S as [heads, vdim, dim] (a column is contiguous), then the tail [taps - 1, channels].
#include "common.cuh"

namespace iian {

__device__ __forceinline__ float silu_f32(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f32(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

constexpr int kMaxTaps = 8;

// proj rows: [.. q (G * D) | k (G * D) | v (H * V) .. | b (H) ..] at col_off / b_off, row stride ld, activation type A.
// z: float32 [N, H * D] (the decay's pre-activation without its bias).  taps: float32 [C, n_taps], C = 2 G D + H V.
// Grid (N, G + H): CTA (t, u) with u < G prepares query/key head u of token t (convolution, silu, unit length, q . k);
// with u >= G the values of head u - G (convolution, silu), that head's decays and its write strength -- so that a step of
// a few single tokens still spreads over the GPU.
constexpr int kPrepThreads = 128;
constexpr int kPrepMaxDim = 512;

template <typename A>
__device__ __forceinline__ float delta_conv(const A * __restrict__ proj, long long ld, int col, long long t, int first,
                                            const float * __restrict__ tail, int C, int c, const float * __restrict__ taps,
                                            int n_taps) {
    const int back = n_taps - 1;
    float x[kMaxTaps];
#pragma unroll
    for (int j = 0; j < kMaxTaps; j++) {
        x[j] = 0.0f;
        if (j < n_taps) {
            const long long r = t - back + j;                          // the row that tap j multiplies
            if (r >= first) x[j] = to_f32(proj[(size_t) r * ld + col]);
            else {
                const int idx = (int) (r - first) + back;              // place in the tail: rows first - back .. first - 1
                if (tail != nullptr && idx >= 0) x[j] = tail[(size_t) idx * C + c];
            }
        }
    }
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxTaps; j++)
        if (j < n_taps) acc = fmaf(taps[(size_t) c * n_taps + j], x[j], acc);
    return acc;
}

template <typename A>
__global__ void __launch_bounds__(kPrepThreads)
delta_prep_kernel(const A * __restrict__ proj, long long ld, int col_off, int b_off,
                  const float * __restrict__ z, const float * __restrict__ taps, int n_taps,
                  const float * __restrict__ a_log, const float * __restrict__ dt_bias,
                  const float * __restrict__ state, long long state_stride, long long tail_off,
                  const int * __restrict__ seq_of_token, const int * __restrict__ cu_q,
                  const int * __restrict__ state_slots,
                  float * __restrict__ qn, float * __restrict__ kn, float * __restrict__ vv,
                  float * __restrict__ beta, float * __restrict__ decay, float * __restrict__ qk,
                  int H, int G, int D, int V, float q_scale) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float act_q[kPrepMaxDim], act_k[kPrepMaxDim];
    __shared__ float red[3][kPrepThreads / 32];
    const size_t t = blockIdx.x;
    const int u = blockIdx.y;
    const int s = seq_of_token[t];
    const int GD = G * D, HV = H * V, C = 2 * GD + HV;
    if (s < 0) return;                         // padding token: the scan writes zeros for it
    const int slot = state_slots[s];
    const int first = cu_q[s];                 // the step's first row of this sequence
    const float * tail = slot >= 0 ? state + (size_t) slot * state_stride + tail_off : nullptr;
    if (u < G) {
        float sq = 0.0f, sk = 0.0f, dot = 0.0f;
        for (int d = threadIdx.x; d < D; d += kPrepThreads) {
            const int cq = u * D + d, ck = GD + u * D + d;
            const float a = silu_f32(delta_conv(proj, ld, col_off + cq, (long long) t, first, tail, C, cq, taps, n_taps));
            const float b = silu_f32(delta_conv(proj, ld, col_off + ck, (long long) t, first, tail, C, ck, taps, n_taps));
            act_q[d] = a;
            act_k[d] = b;
        }
        // the three sums in the order the tiled kernel takes them (a lane over d = lane, lane + 32, ..., then the lanes), so
        // that a token's vectors are the same bits whichever kernel prepared them
        __syncthreads();
        if (threadIdx.x < 32) {
            sq = sk = dot = 0.0f;
            for (int d = threadIdx.x; d < D; d += 32) {
                const float a = act_q[d], b = act_k[d];
                sq = fmaf(a, a, sq);
                sk = fmaf(b, b, sk);
                dot = fmaf(a, b, dot);
            }
            sq = warp_sum(sq);
            sk = warp_sum(sk);
            dot = warp_sum(dot);
            if (threadIdx.x == 0) { red[0][0] = sq; red[1][0] = sk; red[2][0] = dot; }
        }
        __syncthreads();
        sq = red[0][0]; sk = red[1][0]; dot = red[2][0];
        const float iq = q_scale / sqrtf(sq + 1e-6f), ik = 1.0f / sqrtf(sk + 1e-6f);
        for (int d = threadIdx.x; d < D; d += kPrepThreads) {
            qn[t * GD + u * D + d] = act_q[d] * iq;
            kn[t * GD + u * D + d] = act_k[d] * ik;
        }
        if (threadIdx.x == 0) qk[t * G + u] = dot * iq * ik;
        return;
    }
    const int h = u - G;
    for (int j = threadIdx.x; j < V; j += kPrepThreads) {
        const int c = 2 * GD + h * V + j;
        vv[t * HV + h * V + j] = silu_f32(delta_conv(proj, ld, col_off + c, (long long) t, first, tail, C, c, taps, n_taps));
    }
    const float rate = expf(a_log[h]);
    for (int d = threadIdx.x; d < D; d += kPrepThreads) {
        const size_t e = (size_t) h * D + d;
        decay[t * (size_t) (H * D) + e] = expf(-rate * softplus_f32(z[t * (size_t) (H * D) + e] + dt_bias[e]));
    }
    if (threadIdx.x == 0) beta[t * H + h] = 1.0f / (1.0f + expf(-to_f32(proj[t * ld + b_off + h])));
}

// The same preparation for steps of many tokens.  Grid (ceil(N / T), G + H): a CTA takes T neighbouring rows of the step for
// one unit (a query/key head, or a value head with its decays and write strength).  The rows the convolution needs
// (T + taps - 1 of them) and the unit's filters first go to shared memory, every load independent of the others, together with
// the tokens' sequence numbers; then each warp takes tokens of its own, a lane the entries lane, lane + 32, ...  Inputs from
// before a sequence's first row in the step come from the state's tail as in the kernel above.  Results are the same bits.
// Shared memory: x [T + taps - 1][W] rows of the unit's W channels | filters [taps][W] | first [T] | slot [T] (ints).
constexpr int kPrepTileWarps = 4;
constexpr int kPrepTileFrom = 256;          // tokens in a step from which the tiled kernel runs (tiles of 8; of 16 from four times as many)
constexpr int kPrepPerLane = kPrepMaxDim / 32;

template <typename A>
__global__ void __launch_bounds__(kPrepTileWarps * 32)
delta_prep_tile_kernel(const A * __restrict__ proj, long long ld, int col_off, int b_off,
                       const float * __restrict__ z, const float * __restrict__ taps, int n_taps,
                       const float * __restrict__ a_log, const float * __restrict__ dt_bias,
                       const float * __restrict__ state, long long state_stride, long long tail_off,
                       const int * __restrict__ seq_of_token, const int * __restrict__ cu_q,
                       const int * __restrict__ state_slots,
                       float * __restrict__ qn, float * __restrict__ kn, float * __restrict__ vv,
                       float * __restrict__ beta, float * __restrict__ decay, float * __restrict__ qk,
                       int N, int T, int H, int G, int D, int V, float q_scale) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float psm[];
    const int u = blockIdx.y;
    const int GD = G * D, HV = H * V, C = 2 * GD + HV, HD = H * D;
    const int back = n_taps - 1, rows = T + back;
    const bool qk_unit = u < G;
    const int W = qk_unit ? 2 * D : V;                        // channels of this unit: q | k of a head, or a head's values
    float * xs = psm;                                        // [rows][W]
    float * ws = xs + (size_t) rows * W;                     // [n_taps][W]
    int * first_s = reinterpret_cast<int *>(ws + (size_t) W * n_taps);
    int * slot_s = first_s + T;
    const long long t0 = (long long) blockIdx.x * T;
    const int tid = threadIdx.x, nthr = blockDim.x;
    // channel w of the unit is channel chan(w) of the convolution
    auto chan = [&](int w) { return qk_unit ? (w < D ? u * D + w : GD + u * D + (w - D)) : 2 * GD + (u - G) * V + w; };
    if (tid < T) {
        const long long t = t0 + tid;
        int first = 0, slot = -2;                            // -2: no token (beyond the step, or padding)
        if (t < N) {
            const int sq = seq_of_token[t];
            if (sq >= 0) { first = cu_q[sq]; slot = state_slots[sq]; }
        }
        first_s[tid] = first;
        slot_s[tid] = slot;
    }
    for (int w = tid; w < W; w += nthr) {
        const int c = chan(w);
        const A * src = proj + col_off + c;
        for (int ri = 0; ri < rows; ri++) {
            const long long r = t0 - back + ri;
            xs[ri * W + w] = r >= 0 && r < N ? to_f32(src[(size_t) r * ld]) : 0.0f;
        }
        for (int j = 0; j < n_taps; j++) ws[j * W + w] = taps[(size_t) c * n_taps + j];      // [taps][W]: lanes read neighbours
    }
    __syncthreads();
    const int warp = tid >> 5, lane = tid & 31;
    // the convolution of channel w (convolution channel c) at the tile's token ti; `before` of its inputs lie ahead of the
    // sequence's first row in this step and come from the state's tail (or are zero)
    auto conv = [&](int ti, int before, const float * tail, int w, int c) {
        float acc = 0.0f;
        if (before <= 0) {
            for (int j = 0; j < n_taps; j++) acc = fmaf(ws[j * W + w], xs[(ti + j) * W + w], acc);
            return acc;
        }
        for (int j = 0; j < n_taps; j++) {
            float x = 0.0f;
            if (j >= before) x = xs[(ti + j) * W + w];
            else {
                const int idx = j - before + back;             // place in the tail: rows first - back .. first - 1
                if (tail != nullptr && idx >= 0) x = tail[(size_t) idx * C + c];
            }
            acc = fmaf(ws[j * W + w], x, acc);
        }
        return acc;
    };
    for (int ti = warp; ti < T; ti += kPrepTileWarps) {
        const int slot = slot_s[ti];
        if (slot == -2) continue;
        const long long t = t0 + ti;
        const int before = (int) (first_s[ti] - (t - back));        // inputs of this token that lie ahead of the step's rows
        const float * tail = slot >= 0 ? state + (size_t) slot * state_stride + tail_off : nullptr;
        if (qk_unit) {
            float aq[kPrepPerLane], ak[kPrepPerLane];
            float sq = 0.0f, sk = 0.0f, dot = 0.0f;
#pragma unroll
            for (int i = 0; i < kPrepPerLane; i++) {
                const int d = lane + 32 * i;
                aq[i] = ak[i] = 0.0f;
                if (d < D) {
                    aq[i] = silu_f32(conv(ti, before, tail, d, u * D + d));
                    ak[i] = silu_f32(conv(ti, before, tail, D + d, GD + u * D + d));
                    sq = fmaf(aq[i], aq[i], sq);
                    sk = fmaf(ak[i], ak[i], sk);
                    dot = fmaf(aq[i], ak[i], dot);
                }
            }
            sq = warp_sum(sq);
            sk = warp_sum(sk);
            dot = warp_sum(dot);
            const float iq = q_scale / sqrtf(sq + 1e-6f), ik = 1.0f / sqrtf(sk + 1e-6f);
#pragma unroll
            for (int i = 0; i < kPrepPerLane; i++) {
                const int d = lane + 32 * i;
                if (d < D) {
                    qn[t * GD + u * D + d] = aq[i] * iq;
                    kn[t * GD + u * D + d] = ak[i] * ik;
                }
            }
            if (lane == 0) qk[t * G + u] = dot * iq * ik;
        } else {
            const int h = u - G;
            const float rate = expf(a_log[h]);
            for (int d = lane; d < D; d += 32) {
                const size_t e = (size_t) h * D + d;
                decay[t * (size_t) HD + e] = expf(-rate * softplus_f32(z[t * (size_t) HD + e] + dt_bias[e]));
            }
            for (int j = lane; j < V; j += 32)
                vv[t * HV + h * V + j] = silu_f32(conv(ti, before, tail, j, 2 * GD + h * V + j));
            if (lane == 0) beta[t * H + h] = 1.0f / (1.0f + expf(-to_f32(proj[t * ld + b_off + h])));
        }
    }
}

constexpr int kCols = 16;        // columns of S a CTA owns
constexpr int kLanes = 8;        // lanes that share a column

__device__ __forceinline__ void dr_cp4(float * dst, const float * src, bool valid) {
    const unsigned d = (unsigned) __cvta_generic_to_shared(dst);
    const int n = valid ? 4 : 0;                             // src-size 0: the word is zero-filled, nothing is read
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void dr_cp16(float * dst, const float * src) {
    const unsigned d = (unsigned) __cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void dr_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void dr_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

// E: entries of a column a lane holds.  VEC (D a multiple of 4, the buffers 16-byte aligned): a lane holds groups of four
// neighbouring entries, d = 4 * lane + 32 * (i / 4) + i % 4, so that the state and the rows of q, k and the decays move
// 16 bytes at a time (E a multiple of 4); else entry d = lane + kLanes * i, word by word.  The tokens of a sequence pass
// through two stages of shared memory, `chunk` tokens each: while one is worked through, cp.async fills the other.
template <int E, bool VEC, typename A>
__global__ void __launch_bounds__(kCols * kLanes)
delta_scan_kernel(const float * __restrict__ qn, const float * __restrict__ kn, const float * __restrict__ vv,
                  const float * __restrict__ beta, const float * __restrict__ decay, const float * __restrict__ qk,
                  float * __restrict__ state, long long state_stride, long long tail_off,
                  const A * __restrict__ proj, long long ld, int col_off, int n_taps,
                  const int * __restrict__ cu_q, const int * __restrict__ state_slots, float * __restrict__ out,
                  int H, int G, int D, int V, int chunk) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float sm[];
    const int Dp = (D + 3) & ~3;                             // rows start on 16-byte boundaries
    const int stage_floats = chunk * (3 * Dp + kCols + 4);   // q | k | decay | v | beta, q . k (padded to 4 per token)
    const int cb = blockIdx.x, h = blockIdx.y, s = blockIdx.z;
    const int g = h / (H / G);
    const int col = threadIdx.x / kLanes, lane = threadIdx.x % kLanes;
    const int j = cb * kCols + col;            // this thread's column of S
    const int t0 = cu_q[s], t1 = cu_q[s + 1];
    const int slot = state_slots[s];
    const int HV = H * V, GD = G * D, HD = H * D;
    if (slot < 0) {                            // a padding sequence: zeros out, nothing kept
        for (int t = t0; t < t1; t++)
            if (lane == 0 && j < V) out[(size_t) t * HV + h * V + j] = 0.0f;
        return;
    }
    float * st = state + (size_t) slot * state_stride;

    auto fill = [&](int c0, int stage) {       // tokens c0 .. of the step into a stage
        const int nt = min(chunk, t1 - c0);
        float * s_q = sm + (size_t) stage * stage_floats;
        float * s_k = s_q + chunk * Dp;
        float * s_g = s_k + chunk * Dp;
        float * s_v = s_g + chunk * Dp;
        float * s_b = s_v + chunk * kCols;
        if (VEC) {
            const int per = D >> 2;
            for (int e = threadIdx.x; e < nt * per; e += blockDim.x) {
                const int tt = e / per, d = (e - tt * per) << 2;
                const size_t t = c0 + tt;
                dr_cp16(s_q + tt * Dp + d, qn + t * GD + g * D + d);
                dr_cp16(s_k + tt * Dp + d, kn + t * GD + g * D + d);
                dr_cp16(s_g + tt * Dp + d, decay + t * HD + h * D + d);
            }
        } else {
            for (int e = threadIdx.x; e < nt * D; e += blockDim.x) {
                const int tt = e / D, d = e - tt * D;
                const size_t t = c0 + tt;
                dr_cp4(s_q + tt * Dp + d, qn + t * GD + g * D + d, true);
                dr_cp4(s_k + tt * Dp + d, kn + t * GD + g * D + d, true);
                dr_cp4(s_g + tt * Dp + d, decay + t * HD + h * D + d, true);
            }
        }
        for (int e = threadIdx.x; e < nt * kCols; e += blockDim.x) {
            const int tt = e / kCols, c = e - tt * kCols;
            const int jj = cb * kCols + c;
            dr_cp4(s_v + e, vv + (size_t) (c0 + tt) * HV + h * V + (jj < V ? jj : 0), jj < V);
        }
        for (int e = threadIdx.x; e < nt; e += blockDim.x) {
            dr_cp4(s_b + 2 * e, beta + (size_t) (c0 + e) * H + h, true);
            dr_cp4(s_b + 2 * e + 1, qk + (size_t) (c0 + e) * G + g, true);
        }
    };
    if (t0 < t1) fill(t0, 0);
    dr_commit();

    // the convolution's tail moves on: the last taps - 1 inputs of the sequence so far (the sequence's CTAs share the channels)
    if (n_taps > 1) {
        const int C = 2 * GD + HV, back = n_taps - 1, L = t1 - t0;
        float * tail = st + tail_off;
        const int part = h * gridDim.x + cb, parts = gridDim.x * gridDim.y;
        for (int c = part * blockDim.x + threadIdx.x; c < C; c += parts * blockDim.x) {
            float keep[kMaxTaps];
#pragma unroll
            for (int i = 0; i < kMaxTaps - 1; i++) {
                if (i >= back) break;
                const int src = L - back + i;              // row of the step (relative to t0) that lands at place i
                keep[i] = src >= 0 ? to_f32(proj[(size_t) (t0 + src) * ld + col_off + c])
                                   : tail[(size_t) (src + back) * C + c];
            }
#pragma unroll
            for (int i = 0; i < kMaxTaps - 1; i++) {
                if (i >= back) break;
                tail[(size_t) i * C + c] = keep[i];
            }
        }
    }
    float S[E];
    float * scol = st + ((size_t) h * V + (j < V ? j : 0)) * D;
    static_assert(!VEC || E % 4 == 0, "groups of four entries");
    if (VEC) {
#pragma unroll
        for (int i = 0; i < E; i += 4) {
            const int d = 4 * lane + 4 * kLanes * (i >> 2);
            float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (j < V && d < D) x = *reinterpret_cast<const float4 *>(scol + d);
            S[i] = x.x; S[i + 1] = x.y; S[i + 2] = x.z; S[i + 3] = x.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < E; i++) {
            const int d = lane + kLanes * i;
            S[i] = (j < V && d < D) ? scol[d] : 0.0f;
        }
    }
    int stage = 0;
    for (int c0 = t0; c0 < t1; c0 += chunk, stage ^= 1) {
        const int nt = min(chunk, t1 - c0);
        if (c0 + chunk < t1) {
            fill(c0 + chunk, stage ^ 1);       // (the stage was read two chunks ago; the barrier below closed that)
            dr_commit();
            dr_wait<1>();
        } else {
            dr_wait<0>();
        }
        __syncthreads();
        const float * s_q = sm + (size_t) stage * stage_floats;
        const float * s_k = s_q + chunk * Dp;
        const float * s_g = s_k + chunk * Dp;
        const float * s_v = s_g + chunk * Dp;
        const float * s_b = s_v + chunk * kCols;
        for (int tt = 0; tt < nt; tt++) {
            const float * kq = s_k + tt * Dp;
            const float * qq = s_q + tt * Dp;
            const float * gg = s_g + tt * Dp;
            float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
            float kk[E];                       // the key's entries of this lane, kept for the write
            if (VEC) {
#pragma unroll
                for (int i = 0; i < E; i += 4) {
                    const int d = 4 * lane + 4 * kLanes * (i >> 2);
                    float4 g4 = make_float4(1.0f, 1.0f, 1.0f, 1.0f), k4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), q4 = k4;
                    if (d < D) {
                        g4 = *reinterpret_cast<const float4 *>(gg + d);
                        k4 = *reinterpret_cast<const float4 *>(kq + d);
                        q4 = *reinterpret_cast<const float4 *>(qq + d);
                    }
                    kk[i] = k4.x; kk[i + 1] = k4.y; kk[i + 2] = k4.z; kk[i + 3] = k4.w;
                    S[i] *= g4.x; S[i + 1] *= g4.y; S[i + 2] *= g4.z; S[i + 3] *= g4.w;
                    a0 = fmaf(k4.x, S[i], a0);     b0 = fmaf(q4.x, S[i], b0);
                    a1 = fmaf(k4.y, S[i + 1], a1); b1 = fmaf(q4.y, S[i + 1], b1);
                    a0 = fmaf(k4.z, S[i + 2], a0); b0 = fmaf(q4.z, S[i + 2], b0);
                    a1 = fmaf(k4.w, S[i + 3], a1); b1 = fmaf(q4.w, S[i + 3], b1);
                }
            } else {
#pragma unroll
                for (int i = 0; i < E; i += 2) {
                    const int d = lane + kLanes * i;
                    kk[i] = kk[i + 1] = 0.0f;
                    if (d < D) {
                        kk[i] = kq[d];
                        S[i] *= gg[d];
                        a0 = fmaf(kk[i], S[i], a0);
                        b0 = fmaf(qq[d], S[i], b0);
                    }
                    if (d + kLanes < D) {
                        kk[i + 1] = kq[d + kLanes];
                        S[i + 1] *= gg[d + kLanes];
                        a1 = fmaf(kk[i + 1], S[i + 1], a1);
                        b1 = fmaf(qq[d + kLanes], S[i + 1], b1);
                    }
                }
            }
            float a = a0 + a1, b = b0 + b1;
#pragma unroll
            for (int o = kLanes / 2; o > 0; o >>= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, o);
                b += __shfl_xor_sync(0xffffffffu, b, o);
            }
            const float u = s_b[2 * tt] * (s_v[tt * kCols + col] - a);
#pragma unroll
            for (int i = 0; i < E; i++) S[i] = fmaf(kk[i], u, S[i]);        // (entries beyond D stay zero: their key is zero)
            if (lane == 0 && j < V) out[(size_t) (c0 + tt) * HV + h * V + j] = fmaf(s_b[2 * tt + 1], u, b);
        }
        __syncthreads();                       // everyone is done with this stage before it is filled again
    }
    if (j < V) {
        if (VEC) {
#pragma unroll
            for (int i = 0; i < E; i += 4) {
                const int d = 4 * lane + 4 * kLanes * (i >> 2);
                if (d < D) *reinterpret_cast<float4 *>(scol + d) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < E; i++) {
                const int d = lane + kLanes * i;
                if (d < D) scol[d] = S[i];
            }
        }
    }
}

}  // namespace iian

using namespace iian;

// Floats of a slot's state: S [H, V, D], then the tail [taps - 1, 2 G D + H V].
IIAN_API long long iian_delta_state_floats(int H, int G, int D, int V, int n_taps) {
    return (long long) H * V * D + (long long) (n_taps - 1) * (2LL * G * D + (long long) H * V);
}

IIAN_API int iian_delta_prep(const void * proj, long long ld, int col_off, int b_off, int act_dtype, const float * z,
                             const float * taps, int n_taps, const float * a_log, const float * dt_bias, const float * state,
                             long long state_stride, const int * seq_of_token, const int * cu_q, const int * state_slots,
                             float * qn, float * kn, float * vv, float * beta, float * decay, float * qk, int N, int H, int G,
                             int D, int V, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0 || n_taps < 1 || n_taps > kMaxTaps) return IIAN_ERR_SHAPE;
    if (D > kPrepMaxDim) return IIAN_ERR_LIMIT;
    if (G + H > 65535) return IIAN_ERR_LIMIT;
    const long long tail_off = (long long) H * V * D;
    const float q_scale = 1.0f / sqrtf((float) D);
    // many tokens: tiles of T rows through shared memory; few: a CTA per token and unit, so that they spread over the GPU
    int T = N >= 4 * kPrepTileFrom ? 16 : N >= kPrepTileFrom ? 8 : 0;
    size_t smem = 0;
    const int W = 2 * D > V ? 2 * D : V;
    for (; T >= 4; T /= 2) {
        smem = ((size_t) (T + n_taps - 1) * W + (size_t) W * n_taps + 2 * T) * sizeof(float);
        if (smem <= 96 * 1024) break;
    }
    if (T >= 4) {
        const dim3 tgrid((N + T - 1) / T, G + H);
        if (act_dtype == IIAN_F32) {
            if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prep_tile_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
            return iian_launch(delta_prep_tile_kernel<float>, tgrid, dim3(kPrepTileWarps * 32), smem, stream, (const float *) proj, ld,
                               col_off, b_off, z, taps, n_taps, a_log, dt_bias, state, state_stride, tail_off, seq_of_token, cu_q,
                               state_slots, qn, kn, vv, beta, decay, qk, N, T, H, G, D, V, q_scale);
        }
        if (act_dtype == IIAN_BF16) {
            if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prep_tile_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
            return iian_launch(delta_prep_tile_kernel<__nv_bfloat16>, tgrid, dim3(kPrepTileWarps * 32), smem, stream,
                               (const __nv_bfloat16 *) proj, ld, col_off, b_off, z, taps, n_taps, a_log, dt_bias, state, state_stride,
                               tail_off, seq_of_token, cu_q, state_slots, qn, kn, vv, beta, decay, qk, N, T, H, G, D, V, q_scale);
        }
        return IIAN_ERR_DTYPE;
    }
    const dim3 grid(N, G + H);
    if (act_dtype == IIAN_F32)
        return iian_launch(delta_prep_kernel<float>, grid, dim3(kPrepThreads), 0, stream, (const float *) proj, ld, col_off, b_off, z,
                           taps, n_taps, a_log, dt_bias, state, state_stride, tail_off, seq_of_token, cu_q, state_slots, qn, kn,
                           vv, beta, decay, qk, H, G, D, V, q_scale);
    if (act_dtype == IIAN_BF16)
        return iian_launch(delta_prep_kernel<__nv_bfloat16>, grid, dim3(kPrepThreads), 0, stream, (const __nv_bfloat16 *) proj, ld,
                           col_off, b_off, z, taps, n_taps, a_log, dt_bias, state, state_stride, tail_off, seq_of_token, cu_q,
                           state_slots, qn, kn, vv, beta, decay, qk, H, G, D, V, q_scale);
    return IIAN_ERR_DTYPE;
}

template <int E, typename A>
static int launch_scan(const float * qn, const float * kn, const float * vv, const float * beta, const float * decay,
                       const float * qk, float * state, long long state_stride, const A * proj, long long ld, int col_off,
                       int n_taps, const int * cu_q, const int * state_slots, float * out, int S, int H, int G, int D, int V,
                       int max_q_len, bool vec, cudaStream_t stream) {
    const int Dp = (D + 3) & ~3;
    int chunk = D <= 256 ? 16 : 8;             // tokens per stage of shared memory
    if (max_q_len > 0 && max_q_len < chunk) chunk = max_q_len;         // single tokens: small stages, more CTAs per SM
    const size_t smem = (size_t) 2 * chunk * (3 * Dp + kCols + 4) * sizeof(float);
    if (smem > 200 * 1024) return IIAN_ERR_LIMIT;
    const dim3 grid((V + kCols - 1) / kCols, H, S);
    if constexpr (E % 4 == 0) if (vec) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(delta_scan_kernel<E, true, A>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        return iian_launch(delta_scan_kernel<E, true, A>, grid, dim3(kCols * kLanes), smem, stream, qn, kn, vv, beta, decay, qk, state,
                           state_stride, (long long) H * V * D, proj, ld, col_off, n_taps, cu_q, state_slots, out, H, G, D, V, chunk);
    }
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_scan_kernel<E, false, A>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
    return iian_launch(delta_scan_kernel<E, false, A>, grid, dim3(kCols * kLanes), smem, stream, qn, kn, vv, beta, decay, qk, state,
                       state_stride, (long long) H * V * D, proj, ld, col_off, n_taps, cu_q, state_slots, out, H, G, D, V, chunk);
}

template <typename A>
static int scan_by_depth(const float * qn, const float * kn, const float * vv, const float * beta, const float * decay,
                         const float * qk, float * state, long long state_stride, const A * proj, long long ld, int col_off,
                         int n_taps, const int * cu_q, const int * state_slots, float * out, int S, int H, int G, int D, int V,
                         int max_q_len, cudaStream_t stream) {
    const int e = (D + kLanes - 1) / kLanes;
    const bool vec = D % 4 == 0 && state_stride % 4 == 0 &&
                     (((uintptr_t) qn | (uintptr_t) kn | (uintptr_t) decay | (uintptr_t) state) & 15) == 0;
#define IIAN_SCAN(E) return launch_scan<E, A>(qn, kn, vv, beta, decay, qk, state, state_stride, proj, ld, col_off, n_taps, cu_q, \
                                              state_slots, out, S, H, G, D, V, max_q_len, vec, stream)
    if (e <= 2 && !vec) IIAN_SCAN(2);
    if (e <= 4) IIAN_SCAN(4);
    if (e <= 8) IIAN_SCAN(8);
    if (e <= 16) IIAN_SCAN(16);
    if (e <= 32) IIAN_SCAN(32);
    if (e <= 64) IIAN_SCAN(64);
#undef IIAN_SCAN
    return IIAN_ERR_LIMIT;
}

// out: float32 [N, H * V].  S sequences (grid z); a sequence with state slot -1 is padding.  max_q_len: the most tokens a
// sequence has in this step (0: unknown); it sizes the stages of shared memory.
IIAN_API int iian_delta_scan(const float * qn, const float * kn, const float * vv, const float * beta, const float * decay,
                             const float * qk, float * state, long long state_stride, const void * proj, long long ld,
                             int col_off, int act_dtype, int n_taps, const int * cu_q, const int * state_slots, float * out,
                             int S, int H, int G, int D, int V, int max_q_len, cudaStream_t stream) {
    if (S <= 0) return IIAN_OK;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0 || n_taps < 1 || n_taps > kMaxTaps || S > 65535 || H > 65535) return IIAN_ERR_SHAPE;
    if (act_dtype == IIAN_F32)
        return scan_by_depth<float>(qn, kn, vv, beta, decay, qk, state, state_stride, (const float *) proj, ld, col_off, n_taps,
                                    cu_q, state_slots, out, S, H, G, D, V, max_q_len, stream);
    if (act_dtype == IIAN_BF16)
        return scan_by_depth<__nv_bfloat16>(qn, kn, vv, beta, decay, qk, state, state_stride, (const __nv_bfloat16 *) proj, ld,
                                            col_off, n_taps, cu_q, state_slots, out, S, H, G, D, V, max_q_len, stream);
    return IIAN_ERR_DTYPE;
}
