// Mixers that carry a fixed-size state per request instead of a cache that grows:
//
//   causal_conv_silu   short causal convolution over time per channel (+ bias) and silu, with the last
//                      taps-1 inputs of a request kept in its state slot between steps; the residual form
//                      (causal_conv_residual) puts out x_t + conv(x)_t instead, without an activation
//   delta_scan         gated delta rule with one decay per head and key channel (or one per head):
//                        S <- diag(g_t) S ;  u = beta_t (v_t - S^T k_t) ;  S <- S + k_t u^T ;  o_t = S^T q_t
//                      and, without the correction, gated linear attention:
//                        S <- diag(g_t) S + k_t v_t^T ;  o_t = S^T q_t
//   ssd_scan           selective state-space recurrence with a scalar decay per head (Mamba-2):
//                        S <- exp(-A dt_t) S + dt_t B_t x_t^T ;  y_t = S^T C_t + D x_t
//   gated_group_rmsnorm  RMS norm over equal groups of a row, with a gate before (silu) or after (sigmoid) it
//
// The recurrences walk a request's tokens of the step in order, one block per (request, head, slice of
// 16 value columns); a thread holds an eighth of one column of S in registers, so that the products with
// k_t and q_t (or C_t) are sums inside a thread and over eight neighbouring lanes.  What a token needs
// besides S (unit vectors, decays, step sizes) is prepared for 8 tokens at a time by the whole block.
// All arithmetic is float, whatever the storage type of the activations; the state is float.  The order
// of the additions of a token depends on nothing but the sizes of the model, so a prompt cut into
// portions, decoded token by token or batched with others gives the same bits.
//
// State slots: state[slot * state_stride + offset ...]; rows of a step that belong to no request carry a
// spare slot of their own.

#include "common.cuh"

namespace mi {

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
// log(1 + e^x) without overflow; equal to x in float beyond 20
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

constexpr int kMaxTaps = 8;

// ---------------------------------------------------------------------------
// out[t, c] = silu(bias[c] + sum_j w[c, j] * in(t - (taps-1-j), c)), inputs before the step's first token
// come from the request's state (time-major: state[j * C + c] is the input at local position
// j - (taps-1)), zeros for a fresh request because a new slot is zeroed.
// ---------------------------------------------------------------------------
// RES: out = x_t + conv(x)_t, in the type OT, instead of silu(conv(x)_t).
template <typename WT, typename OT, bool RES>
__global__ void __launch_bounds__(256)
causal_conv_silu_kernel(const float* __restrict__ x, int ldx, const WT* __restrict__ w, const WT* __restrict__ bias,
                        const float* __restrict__ state, int64_t state_stride, const int* __restrict__ q_start,
                        const int* __restrict__ req_of_token, const int* __restrict__ state_slot,
                        OT* __restrict__ out, int ld_out, int C, int taps, int T) {
    wait_for_earlier_kernels();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float wt[kMaxTaps];
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) wt[j] = j < taps ? to_float(w[(int64_t)c * taps + j]) : 0.f;
    const float bv = bias ? to_float(bias[c]) : 0.f;
    const int per = (T + gridDim.y - 1) / gridDim.y;         // a block's tokens are neighbours in time: their inputs overlap
    for (int t = blockIdx.y * per; t < min(T, (blockIdx.y + 1) * per); ++t) {
        const int b = req_of_token[t];
        const int i = t - q_start[b];
        const float* st = state + (int64_t)state_slot[b] * state_stride;
        float acc = bv;
#pragma unroll
        for (int j = 0; j < kMaxTaps; ++j) {
            if (j < taps) {
                const int s = i - (taps - 1 - j);      // local position of the input of tap j
                const float v = s >= 0 ? x[(int64_t)(t - (taps - 1 - j)) * ldx + c] : st[(int64_t)(s + taps - 1) * C + c];
                acc += wt[j] * v;
            }
        }
        out[(int64_t)t * ld_out + c] = from_float<OT>(RES ? x[(int64_t)t * ldx + c] + acc : silu_f(acc));
    }
}

// The same for four neighbouring channels per thread, sixteen bytes per access: rows, state and output whose
// channel offsets and strides are multiples of four floats.
template <typename WT, typename OT, bool RES>
__global__ void __launch_bounds__(128)
causal_conv_silu_vec4_kernel(const float* __restrict__ x, int ldx, const WT* __restrict__ w, const WT* __restrict__ bias,
                             const float* __restrict__ state, int64_t state_stride, const int* __restrict__ q_start,
                             const int* __restrict__ req_of_token, const int* __restrict__ state_slot,
                             OT* __restrict__ out, int ld_out, int C, int taps, int T) {
    wait_for_earlier_kernels();
    const int c = 4 * (blockIdx.x * blockDim.x + threadIdx.x);
    if (c >= C) return;
    float wt[4][kMaxTaps];
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int j = 0; j < kMaxTaps; ++j) wt[k][j] = j < taps ? to_float(w[(int64_t)(c + k) * taps + j]) : 0.f;
    float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias) bv = make_float4(to_float(bias[c]), to_float(bias[c + 1]), to_float(bias[c + 2]), to_float(bias[c + 3]));
    const int per = (T + gridDim.y - 1) / gridDim.y;
    for (int t = blockIdx.y * per; t < min(T, (blockIdx.y + 1) * per); ++t) {
        const int b = req_of_token[t];
        const int i = t - q_start[b];
        const float* st = state + (int64_t)state_slot[b] * state_stride;
        float4 acc = bv;
#pragma unroll
        for (int j = 0; j < kMaxTaps; ++j) {
            if (j < taps) {
                const int s = i - (taps - 1 - j);
                const float4 v = *reinterpret_cast<const float4*>(
                    s >= 0 ? x + (int64_t)(t - (taps - 1 - j)) * ldx + c : st + (int64_t)(s + taps - 1) * C + c);
                acc.x += wt[0][j] * v.x; acc.y += wt[1][j] * v.y; acc.z += wt[2][j] * v.z; acc.w += wt[3][j] * v.w;
            }
        }
        if (RES) {
            const float4 xt = *reinterpret_cast<const float4*>(x + (int64_t)t * ldx + c);
            store4(out + (int64_t)t * ld_out + c, make_float4(xt.x + acc.x, xt.y + acc.y, xt.z + acc.z, xt.w + acc.w));
        } else {
            store4(out + (int64_t)t * ld_out + c, make_float4(silu_f(acc.x), silu_f(acc.y), silu_f(acc.z), silu_f(acc.w)));
        }
    }
}

// The last taps-1 inputs of every request after this step; one thread per (request, channel) moves its
// entries in ascending order, so an entry is read before it is overwritten.
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const float* __restrict__ x, int ldx, float* __restrict__ state, int64_t state_stride,
                         const int* __restrict__ q_start, const int* __restrict__ state_slot, int C, int taps) {
    wait_for_earlier_kernels();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= C) return;
    const int q0 = q_start[b], n = q_start[b + 1] - q0;
    float* st = state + (int64_t)state_slot[b] * state_stride;
    for (int j = 0; j < taps - 1; ++j) {
        const int s = n + j - (taps - 1);              // local position that becomes entry j
        st[(int64_t)j * C + c] = s >= 0 ? x[(int64_t)(q0 + s) * ldx + c] : st[(int64_t)(n + j) * C + c];
    }
}

// A step of ONE token per request: the norm in groups of the token's residual row, x + conv(x) over the request's
// last taps-1 normalised rows (its state) and this one, the rounded row out, and the state moved on by one token,
// in one launch (the three kernels that a step of any shape takes, for the shape that decoding repeats).  A block
// takes `chunk` columns of one request, all inside one group of the norm, whose root mean square it forms itself
// (blocks of one group form it alike).  w_conv float [C][taps].
template <typename OT>
__global__ void __launch_bounds__(128)
norm_conv_decode_kernel(const float* __restrict__ hidden, const float* __restrict__ norm_w, int groups, float eps,
                        const float* __restrict__ w_conv, float* __restrict__ state, int64_t state_stride,
                        const int* __restrict__ q_start, const int* __restrict__ state_slot, OT* __restrict__ out,
                        int C, int taps, int chunk) {
    __shared__ float scratch[32];
    wait_for_earlier_kernels();
    const int b = blockIdx.x, c_lo = blockIdx.y * chunk;
    const int64_t t = q_start[b];
    const float* x = hidden + t * C;
    const int gs = C / groups, g = c_lo / gs;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) { const float v = x[g * gs + i]; ss += v * v; }
    ss = block_sum(ss, scratch);
    const float rr = 1.0f / sqrtf(ss / (float)gs + eps);
    float* st = state + (int64_t)state_slot[b] * state_stride;
    for (int c = c_lo + threadIdx.x; c < c_lo + chunk; c += blockDim.x) {
        const float n = x[c] * rr * norm_w[c];
        float prev[kMaxTaps];
#pragma unroll
        for (int j = 0; j < kMaxTaps - 1; ++j) prev[j] = j + 1 < taps ? st[(int64_t)j * C + c] : 0.f;   // taps-1-j tokens back
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxTaps - 1; ++j) {
            if (j + 1 < taps) {
                acc += w_conv[(int64_t)c * taps + j] * prev[j];
                if (j > 0) st[(int64_t)(j - 1) * C + c] = prev[j];       // one token on
            }
        }
        acc += w_conv[(int64_t)c * taps + taps - 1] * n;
        if (taps > 1) st[(int64_t)(taps - 2) * C + c] = n;
        out[t * C + c] = from_float<OT>(n + acc);
    }
}

// ---------------------------------------------------------------------------
// The two recurrences.  Block = 128 threads = 16 value columns x 8 lanes; lane r of a column holds, of that
// column of S, the rows 4 (r + 8 m) .. 4 (r + 8 m) + 3 for m = 0 .. RP/4 - 1 (RP rows in all), so that the
// vectors a token brings are read from shared memory sixteen bytes at a time and a sum over rows is four
// independent chains inside a thread, then three exchanges among the eight lanes.  Tokens come 16 at a time:
// while the block walks one chunk, the raw rows of the next are on their way into a second buffer
// (cp.async), then the whole block turns them into what the recurrence reads (unit vectors, decays, step
// sizes), in place; a chunk's results go out together.
// ---------------------------------------------------------------------------
constexpr int kScanLanes = 8;
constexpr int kScanCols = 128 / kScanLanes;
constexpr int kScanChunk = 16;

__device__ __forceinline__ float lanes_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}

// asynchronous copy of one float from global to shared memory (any 4-byte alignment)
__device__ __forceinline__ void copy_async_f32(float* smem_dst, const float* src) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src));
}
// sixteen bytes; both addresses 16-byte aligned
__device__ __forceinline__ void copy_async_16(float* smem_dst, const float* src) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
// all groups but the most recent one have landed
__device__ __forceinline__ void copy_async_wait_but_one() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }

// loads from shared memory by its own 32-bit addresses (the delta rule's walk: 7 % shorter than through pointers;
// the Mamba-2 walk, with fewer loads per token, lost 4 % and keeps its pointers)
__device__ __forceinline__ float4 shared_f4(uint32_t a) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ float shared_f1(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(a) : "memory");
    return v;
}

// row of S that element (m, x) of lane r holds
__device__ __forceinline__ int scan_row(int r, int m, int x) { return 4 * (r + kScanLanes * m) + x; }

// What the delta rule reads per (token, head), made ready by a kernel of its own (all tokens at once, instead
// of once per slice of value columns inside the walk): prep[t][h] = [q | k | decay | beta, 0, 0, 0], the three
// vectors padded to DP rows with 0, 0 and 1.  qkv: [T, ld_qkv] float, q heads at column 0 (G x d), k heads at
// G*d; beta_raw: [T, ld_beta] (H columns); a_raw: [T, ld_a].  `form` says what the vectors are:
//   0  unit q (times q_scale), unit k; a decay per head and key channel, exp(-exp(a_log[h]) softplus(a + dt_bias))
//      with a and dt_bias laid out H x d
//   1  the same with ONE decay per head: a and dt_bias have H columns
//   2  q times q_scale and k as they are; a decay per key channel, sigmoid(a + dt_bias)^(1 / tau), laid out
//      H x d (a_log and beta_raw are not read; the write strength is 1)
enum DeltaForm : int { kDecayPerChannel = 0, kDecayPerHead = 1, kSigmoidDecay = 2 };

__global__ void __launch_bounds__(128)
delta_prepare_kernel(const float* __restrict__ qkv, int ld_qkv, const float* __restrict__ beta_raw, int ld_beta,
                     const float* __restrict__ a_raw, int ld_a, const float* __restrict__ a_log,
                     const float* __restrict__ dt_bias, float* __restrict__ prep, int H, int G, int d, int DP,
                     float q_scale, int form, float tau) {
    __shared__ float scratch[32];
    wait_for_earlier_kernels();
    const int64_t t = blockIdx.x;
    const int h = blockIdx.y, hk = h / (H / G);
    const float* qrow = qkv + t * ld_qkv + (int64_t)hk * d;
    const float* krow = qkv + t * ld_qkv + (int64_t)(G + hk) * d;
    float qn = q_scale, kn = 1.0f;
    if (form != kSigmoidDecay) {
        float qq = 0.f, kk = 0.f;
        for (int i = threadIdx.x; i < d; i += 128) { const float a = qrow[i], c = krow[i]; qq += a * a; kk += c * c; }
        qq = block_sum(qq, scratch);
        kk = block_sum(kk, scratch);
        qn = q_scale / sqrtf(qq + 1e-6f);
        kn = 1.0f / sqrtf(kk + 1e-6f);
    }
    const float neg_a = form == kSigmoidDecay ? 0.f : -expf(a_log[h]);
    const float head_decay = form == kDecayPerHead ? expf(neg_a * softplus_f(a_raw[t * ld_a + h] + dt_bias[h])) : 1.f;
    const float* arow = a_raw + t * ld_a + (int64_t)h * d;
    float* row = prep + (t * H + h) * (3 * DP + 4);
    for (int i = threadIdx.x; i < DP; i += 128) {
        float qv = 0.f, kv = 0.f, gv = 1.f;
        if (i < d) {
            qv = qrow[i] * qn;
            kv = krow[i] * kn;
            if (form == kDecayPerChannel) gv = expf(neg_a * softplus_f(arow[i] + dt_bias[(int64_t)h * d + i]));
            else if (form == kDecayPerHead) gv = head_decay;
            else gv = expf(-softplus_f(-(arow[i] + dt_bias[(int64_t)h * d + i])) / tau);   // log sigmoid(z) = -softplus(-z)
        }
        row[i] = qv; row[DP + i] = kv; row[2 * DP + i] = gv;
    }
    if (threadIdx.x < 4)
        row[3 * DP + threadIdx.x] = threadIdx.x == 0 ? (form == kSigmoidDecay ? 1.f : sigmoid_f(beta_raw[t * ld_beta + h])) : 0.f;
}

// The walk.  prep as delta_prepare_kernel leaves it; v heads at column v_col0 of qkv (H x dv).  out: [T, H*dv].
// Without DELTA the write is the value itself, u = v_t (gated linear attention): S^T k_t is never formed.
//
// Segments (segs > 1; gated linear attention only, whose transition is diagonal): a request's portion is cut into
// `segs` runs of seg_len tokens that are walked side by side, block z = request * segs + segment.  Segment 0 starts
// from the request's state, the others from zero, and every segment leaves its final state in seg_state
// [z][H][d][dv] instead of the slot.  The recurrence is linear in S, so what a later segment's read-outs lack is
// (b_t * q_t)^T S_start with b_t the product of the decays since the segment's start: gla_segment_decay_kernel forms
// b_t * q_t and the segments' whole decays, gla_segments_combine_kernel chains the final states into every
// segment's true start state (and the request's new state), delta_segments_correct_kernel adds the missing term.
template <int RP, bool DELTA>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* __restrict__ qkv, int ld_qkv, int64_t v_col0, const float* __restrict__ prep,
                  float* __restrict__ state, int64_t state_stride, const int* __restrict__ q_start,
                  const int* __restrict__ state_slot, float* __restrict__ out, int H, int d, int dv,
                  int segs, int seg_len, float* __restrict__ seg_state) {
    extern __shared__ __align__(16) float sm[];
    constexpr int DP = RP * kScanLanes;                 // rows, padded
    constexpr int MV = RP / 4;
    constexpr int ROW = 3 * DP + 4;                     // floats of one (token, head) of prep
    // two buffers of: prep rows [chunk][ROW], v of this slice [chunk][16]
    constexpr int kBuf = kScanChunk * (ROW + kScanCols);
    float* os = sm + 2 * kBuf;                          // [chunk][16] results of the chunk
    wait_for_earlier_kernels();
    const int z = blockIdx.z, b = segs > 1 ? z / segs : z, seg = segs > 1 ? z - b * segs : 0;
    const int h = blockIdx.y, col0 = blockIdx.x * kScanCols;
    const int tid = threadIdx.x;
    const int r = tid & (kScanLanes - 1), lc = tid / kScanLanes, col = col0 + lc;
    const bool col_ok = col < dv;
    const int qa = q_start[b], na = q_start[b + 1] - qa;
    if (seg > 0 && seg * seg_len >= na) return;                 // a request shorter than its segments
    const int q0 = qa + seg * seg_len, n = segs > 1 ? min(seg_len, na - seg * seg_len) : na;
    float* S = state + (int64_t)state_slot[b] * state_stride + (int64_t)h * d * dv;
    float s[RP];
#pragma unroll
    for (int m = 0; m < MV; ++m)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int i = scan_row(r, m, x);
            s[4 * m + x] = (seg == 0 && col_ok && i < d) ? S[(int64_t)i * dv + col] : 0.f;
        }
    const int64_t v_col = v_col0 + (int64_t)h * dv + col0;
    const int n_cols = min(kScanCols, dv - col0);

    auto fetch = [&](int c0, float* buf) {
        const int nc = min(kScanChunk, n - c0);
        float* vs = buf + kScanChunk * ROW;
        for (int idx = tid; idx < nc * (ROW / 4); idx += 128) {
            const int tt = idx / (ROW / 4), c = idx - tt * (ROW / 4);
            copy_async_16(buf + tt * ROW + 4 * c, prep + ((int64_t)(q0 + c0 + tt) * H + h) * ROW + 4 * c);
        }
        for (int idx = tid; idx < nc * n_cols; idx += 128) {
            const int tt = idx / n_cols, c = idx - tt * n_cols;
            copy_async_f32(vs + tt * kScanCols + c, qkv + (int64_t)(q0 + c0 + tt) * ld_qkv + v_col + c);
        }
    };

    fetch(0, sm);
    copy_async_commit();
    int which = 0;
    for (int c0 = 0; c0 < n; c0 += kScanChunk, which ^= 1) {
        const int nc = min(kScanChunk, n - c0);
        const float* rows = sm + which * kBuf;
        const float* vs = rows + kScanChunk * ROW;
        const uint32_t rows_a = static_cast<uint32_t>(__cvta_generic_to_shared(rows));
        const uint32_t vs_a = static_cast<uint32_t>(__cvta_generic_to_shared(vs));
        if (c0 + kScanChunk < n) fetch(c0 + kScanChunk, sm + (which ^ 1) * kBuf);     // read last two syncs ago
        copy_async_commit();
        copy_async_wait_but_one();
        __syncthreads();                                // this chunk's rows have landed for every thread
        // Four tokens at a time: the read-outs' sums over the lanes do not feed the recurrence, so the four of
        // them are exchanged together after the four steps instead of stalling each step.
        for (int t4 = 0; t4 < nc; t4 += 4) {
            float o_part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int u4 = 0; u4 < 4; ++u4) {
                const int tt = t4 + u4;
                if (tt < nc) {
                    const uint32_t qa = rows_a + (uint32_t)(tt * ROW + 4 * r) * 4u;       // this lane's first q
                    float4 k4[MV];
                    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                    for (int m = 0; m < MV; ++m) {
                        const float4 g4 = shared_f4(qa + (2 * DP + 4 * kScanLanes * m) * 4);
                        k4[m] = shared_f4(qa + (DP + 4 * kScanLanes * m) * 4);
                        s[4 * m] *= g4.x; s[4 * m + 1] *= g4.y; s[4 * m + 2] *= g4.z; s[4 * m + 3] *= g4.w;
                        if (DELTA) {
                            a0 += s[4 * m] * k4[m].x; a1 += s[4 * m + 1] * k4[m].y; a2 += s[4 * m + 2] * k4[m].z; a3 += s[4 * m + 3] * k4[m].w;
                        }
                    }
                    float u = shared_f1(vs_a + (uint32_t)(tt * kScanCols + lc) * 4u);
                    if (DELTA) {
                        const float acc = lanes_sum((a0 + a1) + (a2 + a3));
                        u = shared_f1(rows_a + (uint32_t)(tt * ROW + 3 * DP) * 4u) * (u - acc);
                    }
                    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
                    for (int m = 0; m < MV; ++m) {
                        const float4 q4 = shared_f4(qa + (4 * kScanLanes * m) * 4);
                        s[4 * m] += k4[m].x * u; s[4 * m + 1] += k4[m].y * u; s[4 * m + 2] += k4[m].z * u; s[4 * m + 3] += k4[m].w * u;
                        o0 += s[4 * m] * q4.x; o1 += s[4 * m + 1] * q4.y; o2 += s[4 * m + 2] * q4.z; o3 += s[4 * m + 3] * q4.w;
                    }
                    o_part[u4] = (o0 + o1) + (o2 + o3);
                }
            }
#pragma unroll
            for (int sh = 1; sh < kScanLanes; sh <<= 1)
#pragma unroll
                for (int u4 = 0; u4 < 4; ++u4) o_part[u4] += __shfl_xor_sync(0xffffffffu, o_part[u4], sh);
            if (r == 0) {
#pragma unroll
                for (int u4 = 0; u4 < 4; ++u4)
                    if (t4 + u4 < nc) os[(t4 + u4) * kScanCols + lc] = o_part[u4];
            }
        }
        __syncthreads();
        for (int idx = tid; idx < nc * kScanCols; idx += 128) {
            const int tt = idx / kScanCols, c = col0 + idx % kScanCols;
            if (c < dv) out[(int64_t)(q0 + c0 + tt) * H * dv + (int64_t)h * dv + c] = os[idx];
        }
    }
    if (segs > 1) S = seg_state + ((int64_t)z * H + h) * d * dv;       // the segment's final state, for the chain
#pragma unroll
    for (int m = 0; m < MV; ++m)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int i = scan_row(r, m, x);
            if (col_ok && i < d) S[(int64_t)i * dv + col] = s[4 * m + x];
        }
}

// Gated linear attention walked in segments: for every token the query times the product of the decays since its
// segment's start, qt[t][h][i] = q_t[i] * b_t[i] (what the start state must be read with), and per segment the whole
// product bend[z][h][i].  A thread per (segment, head, key channel) multiplies its way through the segment.
__global__ void __launch_bounds__(128)
gla_segment_decay_kernel(const float* __restrict__ prep, const int* __restrict__ q_start, float* __restrict__ qt,
                         float* __restrict__ bend, int H, int d, int DP, int segs, int seg_len) {
    wait_for_earlier_kernels();
    const int z = blockIdx.z, b = z / segs, seg = z - b * segs, h = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int qa = q_start[b], na = q_start[b + 1] - qa;
    if (i >= d || seg * seg_len >= na) return;
    const int n = min(seg_len, na - seg * seg_len);
    const int ROW = 3 * DP + 4;
    float acc = 1.f;
    // eight tokens' decays and queries are asked for before the first product: the chain is the products alone
    for (int t0 = 0; t0 < n; t0 += 8) {
        float g[8], q[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int64_t tok = qa + seg * seg_len + min(t0 + u, n - 1);
            const float* row = prep + (tok * H + h) * ROW;
            g[u] = row[2 * DP + i];
            q[u] = row[i];
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (t0 + u < n) {
                acc *= g[u];
                qt[((int64_t)(qa + seg * seg_len + t0 + u) * H + h) * d + i] = q[u] * acc;
            }
        }
    }
    bend[((int64_t)z * H + h) * d + i] = acc;
}

// The segments' final states chained into every segment's true start state: with U_p the state segment p reached
// from zero (segment 0: from the request's state) and b_p its whole decay per key channel, S_start[1] = U_0 and
// S_start[p + 1] = diag(b_p) S_start[p] + U_p.  Element by element; S_start[p] replaces U_p in seg_state once U_p has
// been read, and the state after the last segment goes to the request's slot.
__global__ void __launch_bounds__(256)
gla_segments_combine_kernel(float* __restrict__ seg_state, const float* __restrict__ bend, float* __restrict__ state,
                            int64_t state_stride, const int* __restrict__ q_start, const int* __restrict__ state_slot,
                            int H, int d, int dv, int segs, int seg_len) {
    wait_for_earlier_kernels();
    const int b = blockIdx.z, h = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;           // element i * dv + c of the head's state
    if (e >= d * dv) return;
    const int i = e / dv;
    const int na = q_start[b + 1] - q_start[b];
    const int nseg = min(segs, (na + seg_len - 1) / seg_len);
    float cur = seg_state[(((int64_t)b * segs) * H + h) * d * dv + e];
    for (int p = 1; p < nseg; ++p) {
        const int64_t zp = (int64_t)b * segs + p;
        float* U = seg_state + (zp * H + h) * d * dv + e;
        const float nxt = bend[(zp * H + h) * d + i] * cur + *U;
        *U = cur;
        cur = nxt;
    }
    state[(int64_t)state_slot[b] * state_stride + (int64_t)h * d * dv + e] = cur;
}

// out[t] += S_start[segment of t]^T qt[t] for the tokens of the segments behind the first.  A block takes 32 tokens
// of one segment and 64 value columns of one head: the start state's slice in shared memory, a warp four tokens, a
// lane two columns.
constexpr int kCorrectTokens = 32, kCorrectCols = 64;
__global__ void __launch_bounds__(256)
delta_segments_correct_kernel(const float* __restrict__ seg_state, const float* __restrict__ qt, float* __restrict__ out,
                              const int* __restrict__ q_start, int H, int d, int dv, int segs, int seg_len, int tiles,
                              int col_chunks) {
    extern __shared__ __align__(16) float corr_sm[];    // [d][64] start state, [8 warps][d][4 tokens] queries
    wait_for_earlier_kernels();
    const int b = blockIdx.z, h = blockIdx.y / col_chunks, cc = blockIdx.y % col_chunks;
    const int p = 1 + blockIdx.x / tiles, tile = blockIdx.x % tiles;
    const int qa = q_start[b], na = q_start[b + 1] - qa;
    const int t_lo = p * seg_len + tile * kCorrectTokens;
    const int t_hi = min(min(na, (p + 1) * seg_len), t_lo + kCorrectTokens);
    if (t_lo >= t_hi) return;
    const float* S0 = seg_state + (((int64_t)b * segs + p) * H + h) * d * dv;
    const int c0 = cc * kCorrectCols;
    float* Ssm = corr_sm;
    float* qsm = corr_sm + d * kCorrectCols;
    for (int idx = threadIdx.x; idx < d * kCorrectCols; idx += 256) {
        const int i = idx / kCorrectCols, c = c0 + idx % kCorrectCols;
        Ssm[idx] = c < dv ? S0[(int64_t)i * dv + c] : 0.f;
    }
    __syncthreads();
    // a warp takes the tokens t_lo + warp, + 8, + 16, + 24 together: a number of the state is fetched once for four
    // tokens, and the four queries' numbers of a row lie side by side in shared memory (one 16-byte load)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float4* qw = reinterpret_cast<float4*>(qsm) + warp * d;
    for (int j = lane; j < d; j += 32) {
        float q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int t = t_lo + warp + 8 * u;
            q[u] = t < t_hi ? qt[((int64_t)(qa + t) * H + h) * d + j] : 0.f;
        }
        qw[j] = make_float4(q[0], q[1], q[2], q[3]);
    }
    __syncwarp();
    float a[4][2];
#pragma unroll
    for (int u = 0; u < 4; ++u) a[u][0] = a[u][1] = 0.f;
    for (int j = 0; j < d; ++j) {
        const float4 q4 = qw[j];
        const float s0 = Ssm[j * kCorrectCols + lane], s1 = Ssm[j * kCorrectCols + 32 + lane];
        a[0][0] += q4.x * s0; a[0][1] += q4.x * s1;
        a[1][0] += q4.y * s0; a[1][1] += q4.y * s1;
        a[2][0] += q4.z * s0; a[2][1] += q4.z * s1;
        a[3][0] += q4.w * s0; a[3][1] += q4.w * s1;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int t = t_lo + warp + 8 * u;
        if (t < t_hi) {
            float* orow = out + ((int64_t)(qa + t) * H + h) * dv + c0;
            if (c0 + lane < dv) orow[lane] += a[u][0];
            if (c0 + 32 + lane < dv) orow[32 + lane] += a[u][1];
        }
    }
}

// xbc: [T, ld_x] float after the convolution: x heads at column 0 (H x P), B groups at H*P (G x N), C groups
// at H*P + G*N; dt_raw: [T, ld_dt] (H columns, before dt_bias and softplus).  out: [T, H*P] float.
template <int RP>
__global__ void __launch_bounds__(128)
ssd_scan_kernel(const float* __restrict__ xbc, int ld_x, const float* __restrict__ dt_raw, int ld_dt,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                float* __restrict__ state, int64_t state_stride, const int* __restrict__ q_start,
                const int* __restrict__ state_slot, float* __restrict__ out, int H, int G, int N, int P, int vec) {
    extern __shared__ __align__(16) float sm[];
    constexpr int NP = RP * kScanLanes;
    constexpr int MV = RP / 4;
    // two buffers of: B, C [chunk][NP] each, x of this slice [chunk][16], step size [chunk], decay [chunk]
    constexpr int kBuf = kScanChunk * (2 * NP + kScanCols + 2);
    float* os = sm + 2 * kBuf;                          // [chunk][16] results of the chunk
    wait_for_earlier_kernels();
    const int b = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * kScanCols;
    const int g = h / (H / G);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = tid & (kScanLanes - 1), lc = tid / kScanLanes, col = col0 + lc;
    const bool col_ok = col < P;
    const int q0 = q_start[b], n = q_start[b + 1] - q0;
    float* S = state + (int64_t)state_slot[b] * state_stride + (int64_t)h * N * P;
    float s[RP];
#pragma unroll
    for (int m = 0; m < MV; ++m)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int i = scan_row(r, m, x);
            s[4 * m + x] = (col_ok && i < N) ? S[(int64_t)i * P + col] : 0.f;
        }
    const float neg_a = -expf(a_log[h]);
    const float dskip = d_skip[h];
    const float bias = dt_bias[h];
    const int n_cols = min(kScanCols, P - col0);
    // rows beyond the state's size are never copied to: zero them once in both buffers
    if (N < NP)
        for (int idx = tid; idx < 2 * 2 * kScanChunk * (NP - N); idx += 128) {
            const int i = N + idx % (NP - N), row = idx / (NP - N);      // row: buffer, B or C, token
            sm[(row / (2 * kScanChunk)) * kBuf + (row % (2 * kScanChunk)) * NP + i] = 0.f;
        }

    auto fetch = [&](int c0, float* buf) {
        const int nc = min(kScanChunk, n - c0);
        float* Bs = buf;
        float* Cs = Bs + kScanChunk * NP;
        float* xs = Cs + kScanChunk * NP;
        float* ds = xs + kScanChunk * kScanCols;
        if (vec) {          // rows of B and C that start on 16-byte boundaries: four floats at a time
            const int N4 = N / 4;
            for (int idx = tid; idx < nc * N4; idx += 128) {
                const int tt = idx / N4, i = 4 * (idx - tt * N4);
                const float* brow = xbc + (int64_t)(q0 + c0 + tt) * ld_x + (int64_t)H * P + (int64_t)g * N;
                copy_async_16(Bs + tt * NP + i, brow + i);
                copy_async_16(Cs + tt * NP + i, brow + (int64_t)G * N + i);
            }
        } else {
            for (int idx = tid; idx < nc * N; idx += 128) {
                const int tt = idx / N, i = idx - tt * N;
                const float* brow = xbc + (int64_t)(q0 + c0 + tt) * ld_x + (int64_t)H * P + (int64_t)g * N;
                copy_async_f32(Bs + tt * NP + i, brow + i);
                copy_async_f32(Cs + tt * NP + i, brow + (int64_t)G * N + i);
            }
        }
        for (int idx = tid; idx < nc * n_cols; idx += 128) {
            const int tt = idx / n_cols, c = idx - tt * n_cols;
            copy_async_f32(xs + tt * kScanCols + c, xbc + (int64_t)(q0 + c0 + tt) * ld_x + (int64_t)h * P + col0 + c);
        }
        if (tid < nc) copy_async_f32(ds + tid, dt_raw + (int64_t)(q0 + c0 + tid) * ld_dt + h);
    };

    fetch(0, sm);
    copy_async_commit();
    int which = 0;
    for (int c0 = 0; c0 < n; c0 += kScanChunk, which ^= 1) {
        const int nc = min(kScanChunk, n - c0);
        float* Bs = sm + which * kBuf;
        float* Cs = Bs + kScanChunk * NP;
        float* xs = Cs + kScanChunk * NP;
        float* ds = xs + kScanChunk * kScanCols;
        float* as = ds + kScanChunk;
        if (c0 + kScanChunk < n) fetch(c0 + kScanChunk, sm + (which ^ 1) * kBuf);
        copy_async_commit();
        copy_async_wait_but_one();
        __syncthreads();
        // step sizes and decays, a thread per token (the step size is folded into x in the walk)
        if (tid < nc) {
            const float dt = softplus_f(ds[tid] + bias);
            ds[tid] = dt;
            as[tid] = expf(neg_a * dt);
        }
        __syncthreads();
        // Four tokens at a time: a token's read-out does not feed the recurrence, so the sums over the lanes of
        // four read-outs are exchanged together after the four steps.
        for (int t4 = 0; t4 < nc; t4 += 4) {
            float y_part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int u4 = 0; u4 < 4; ++u4) {
                const int tt = t4 + u4;
                if (tt < nc) {
                    const float4* Bq = reinterpret_cast<const float4*>(Bs + tt * NP);
                    const float4* Cq = reinterpret_cast<const float4*>(Cs + tt * NP);
                    const float a = as[tt], xv = ds[tt] * xs[tt * kScanCols + lc];     // decay; dt * x
                    float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
                    for (int m = 0; m < MV; ++m) {
                        const float4 b4 = Bq[r + kScanLanes * m], c4 = Cq[r + kScanLanes * m];
                        s[4 * m] = a * s[4 * m] + b4.x * xv; s[4 * m + 1] = a * s[4 * m + 1] + b4.y * xv;
                        s[4 * m + 2] = a * s[4 * m + 2] + b4.z * xv; s[4 * m + 3] = a * s[4 * m + 3] + b4.w * xv;
                        y0 += s[4 * m] * c4.x; y1 += s[4 * m + 1] * c4.y; y2 += s[4 * m + 2] * c4.z; y3 += s[4 * m + 3] * c4.w;
                    }
                    y_part[u4] = (y0 + y1) + (y2 + y3);
                }
            }
#pragma unroll
            for (int sh = 1; sh < kScanLanes; sh <<= 1)
#pragma unroll
                for (int u4 = 0; u4 < 4; ++u4) y_part[u4] += __shfl_xor_sync(0xffffffffu, y_part[u4], sh);
            if (r == 0) {
#pragma unroll
                for (int u4 = 0; u4 < 4; ++u4)
                    if (t4 + u4 < nc) os[(t4 + u4) * kScanCols + lc] = y_part[u4] + dskip * xs[(t4 + u4) * kScanCols + lc];
            }
        }
        __syncthreads();
        for (int idx = tid; idx < nc * kScanCols; idx += 128) {
            const int tt = idx / kScanCols, c = col0 + idx % kScanCols;
            if (c < P) out[(int64_t)(q0 + c0 + tt) * H * P + (int64_t)h * P + c] = os[idx];
        }
    }
#pragma unroll
    for (int m = 0; m < MV; ++m)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int i = scan_row(r, m, x);
            if (col_ok && i < N) S[(int64_t)i * P + col] = s[4 * m + x];
        }
}

// ---------------------------------------------------------------------------
// One block per (token, group of `gs` columns):
//   mode 0:  z = y * silu(gate);  out = z * rsqrt(mean(z^2) + eps) * w        (gate before the norm)
//   mode 1:  out = y * rsqrt(mean(y^2) + eps) * w * sigmoid(gate)             (gate after the norm)
//   mode 2:  out = y * rsqrt(mean(y^2) + eps) * w * silu(gate)
// w has `wlen` entries and column c of the row uses w[c % wlen].
// ---------------------------------------------------------------------------
template <typename AT, typename WT>
__global__ void __launch_bounds__(256)
gated_group_rmsnorm_kernel(const float* __restrict__ y, const float* __restrict__ gate, int ld_gate,
                           const WT* __restrict__ w, int wlen, AT* __restrict__ out, int n, int gs, int mode,
                           float eps, bool vec) {
    __shared__ float scratch[32];
    wait_for_earlier_kernels();
    const int t = blockIdx.x, c0 = blockIdx.y * gs;
    const float* yr = y + (int64_t)t * n + c0;
    const float* gr = gate + (int64_t)t * ld_gate + c0;
    AT* orow = out + (int64_t)t * n + c0;
    // vec: every row's groups start on 16-byte boundaries (decided for the whole launch from the sizes, so that
    // the order of a row's sum does not depend on where the row stands in a step): four floats per access
    float ss = 0.f;
    if (vec) {
        for (int i = 4 * threadIdx.x; i < gs; i += 4 * blockDim.x) {
            float4 v = *reinterpret_cast<const float4*>(yr + i);
            if (mode == 0) {
                const float4 g = *reinterpret_cast<const float4*>(gr + i);
                v.x *= silu_f(g.x); v.y *= silu_f(g.y); v.z *= silu_f(g.z); v.w *= silu_f(g.w);
            }
            ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
    } else {
        for (int i = threadIdx.x; i < gs; i += blockDim.x) {
            float v = yr[i];
            if (mode == 0) v *= silu_f(gr[i]);
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float rr = 1.0f / sqrtf(ss / (float)gs + eps);
    if (vec) {
        for (int i = 4 * threadIdx.x; i < gs; i += 4 * blockDim.x) {
            float4 v = *reinterpret_cast<const float4*>(yr + i);
            const float4 g = *reinterpret_cast<const float4*>(gr + i);
            if (mode == 0) { v.x *= silu_f(g.x); v.y *= silu_f(g.y); v.z *= silu_f(g.z); v.w *= silu_f(g.w); }
            const int wi = (c0 + i) % wlen;
            v.x *= rr * to_float(w[wi]); v.y *= rr * to_float(w[wi + 1]);
            v.z *= rr * to_float(w[wi + 2]); v.w *= rr * to_float(w[wi + 3]);
            if (mode == 1) { v.x *= sigmoid_f(g.x); v.y *= sigmoid_f(g.y); v.z *= sigmoid_f(g.z); v.w *= sigmoid_f(g.w); }
            if (mode == 2) { v.x *= silu_f(g.x); v.y *= silu_f(g.y); v.z *= silu_f(g.z); v.w *= silu_f(g.w); }
            orow[i] = from_float<AT>(v.x); orow[i + 1] = from_float<AT>(v.y);
            orow[i + 2] = from_float<AT>(v.z); orow[i + 3] = from_float<AT>(v.w);
        }
    } else {
        for (int i = threadIdx.x; i < gs; i += blockDim.x) {
            float v = yr[i];
            if (mode == 0) v *= silu_f(gr[i]);
            v = v * rr * to_float(w[(c0 + i) % wlen]);
            if (mode == 1) v *= sigmoid_f(gr[i]);
            if (mode == 2) v *= silu_f(gr[i]);
            orow[i] = from_float<AT>(v);
        }
    }
}

}  // namespace mi

using namespace mi;

extern "C" {

// form 0: silu(conv(x) + bias), float out; form 1: x + conv(x) in the type `odtype`
static int launch_causal_conv(const float* x, int ldx, const void* w, const void* bias, int wdtype, float* state,
                              int64_t state_stride, const int* q_start, const int* req_of_token, const int* state_slot,
                              void* out, int odtype, int ld_out, int C, int taps, int T, int B, bool residual,
                              cudaStream_t stream) {
    if (T <= 0 || C <= 0) return kOk;
    if (taps < 1 || taps > kMaxTaps) {
        set_last_error("causal convolution: %d taps are outside [1, %d]", taps, kMaxTaps);
        return kBadShape;
    }
    if (B > 65535) { set_last_error("causal convolution: %d requests exceed the grid limit", B); return kBadShape; }
    const int cb = (C + 255) / 256;
    // ranges of about 16 tokens per block, 8 for rows of up to 4,096 channels, whose blocks are few (2,048 tokens of
    // 1,024 and 2,048 channels: 15.3 -> 11.2 and 17.7 -> 15.8 us a launch; 4 tokens: 11.2 and 20.8 us); fewer when that
    // leaves SMs idle
    const int per_block = C <= 4096 ? 8 : 16;
    int ty = (T + per_block - 1) / per_block;
    if (ty * cb < 296) ty = T < (296 + cb - 1) / cb ? T : (296 + cb - 1) / cb;
    if (ty > 65535) ty = 65535;
    const bool vec4 = C % 4 == 0 && ldx % 4 == 0 && ld_out % 4 == 0 && state_stride % 4 == 0 &&
                      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(state)) & 15) == 0;
#define MI_CONV_LAUNCH(OT, RES)                                                                                       \
    do {                                                                                                              \
        if (vec4) {                                                                                                   \
            MI_DISPATCH_1(wdtype, WT,                                                                                 \
                launch_dependent(causal_conv_silu_vec4_kernel<WT, OT, RES>, dim3((C / 4 + 127) / 128, ty), dim3(128), 0, \
                                 stream, x, ldx, (const WT*)w, (const WT*)bias, (const float*)state, state_stride,    \
                                 q_start, req_of_token, state_slot, (OT*)out, ld_out, C, taps, T));                   \
        } else {                                                                                                      \
            MI_DISPATCH_1(wdtype, WT,                                                                                 \
                launch_dependent(causal_conv_silu_kernel<WT, OT, RES>, dim3(cb, ty), dim3(256), 0, stream, x, ldx,     \
                                 (const WT*)w, (const WT*)bias, (const float*)state, state_stride, q_start,           \
                                 req_of_token, state_slot, (OT*)out, ld_out, C, taps, T));                            \
        }                                                                                                             \
    } while (0)
    if (!residual) MI_CONV_LAUNCH(float, false);
    else if (odtype == kBF16) MI_CONV_LAUNCH(__nv_bfloat16, true);
    else if (odtype == kF32) MI_CONV_LAUNCH(float, true);
    else return kBadDType;
#undef MI_CONV_LAUNCH
    int launched = 1;
    if (taps > 1) {
        launch_dependent(conv_state_update_kernel, dim3(cb, B), dim3(256), 0, stream, x, ldx, state, state_stride,
                         q_start, state_slot, C, taps);
        launched = 2;
    }
    return finish_launch(residual ? "causal_conv_residual" : "causal_conv_silu", launched);
}

int mi_causal_conv_silu(const float* x, int ldx, const void* w, const void* bias, int wdtype, float* state,
                        int64_t state_stride, const int* q_start, const int* req_of_token, const int* state_slot,
                        float* out, int ld_out, int C, int taps, int T, int B, cudaStream_t stream) {
    return launch_causal_conv(x, ldx, w, bias, wdtype, state, state_stride, q_start, req_of_token, state_slot, out,
                              kF32, ld_out, C, taps, T, B, false, stream);
}

// out[t, c] = x[t, c] + sum_j w[c, j] * x(t - (taps-1-j), c) in the type `odtype`; state as above
int mi_causal_conv_residual(const float* x, int ldx, const void* w, int wdtype, float* state, int64_t state_stride,
                            const int* q_start, const int* req_of_token, const int* state_slot, void* out, int odtype,
                            int ld_out, int C, int taps, int T, int B, cudaStream_t stream) {
    return launch_causal_conv(x, ldx, w, nullptr, wdtype, state, state_stride, q_start, req_of_token, state_slot, out,
                              odtype, ld_out, C, taps, T, B, true, stream);
}

// One token per request (checked by the caller): norm in groups, x + conv(x), the state moved on, in one launch.
int mi_norm_conv_decode(const float* hidden, const float* norm_w, int groups, float eps, const float* w_conv,
                        float* state, int64_t state_stride, const int* q_start, const int* state_slot, void* out,
                        int odtype, int B, int C, int taps, cudaStream_t stream) {
    if (B <= 0 || C <= 0) return kOk;
    if (taps < 1 || taps > kMaxTaps || groups < 1 || C % groups || groups > 1024) {
        set_last_error("norm and convolution of a decode step: %d taps, %d columns in %d groups", taps, C, groups);
        return kBadShape;
    }
    // columns per block: a power of two that divides a group (at most 128, a column a thread), else a whole group
    const int gs = C / groups;
    int chunk = gs;
    for (int c = 128; c >= 32; c /= 2) if (gs % c == 0) { chunk = c; break; }
    if (C / chunk > 65535 || B > 65535) { set_last_error("norm and convolution of a decode step: too many blocks"); return kBadShape; }
    MI_DISPATCH_1(odtype, OT,
        launch_dependent(norm_conv_decode_kernel<OT>, dim3(B, C / chunk), dim3(128), 0, stream, hidden,
                         norm_w, groups, eps, w_conv, state, state_stride, q_start, state_slot, (OT*)out, C, taps, chunk));
    return finish_launch("norm_conv_decode");
}

#define MI_SCAN_DISPATCH(rows, ...)                                                     \
    do {                                                                                \
        if ((rows) <= 64) { constexpr int RP = 8; __VA_ARGS__; }                        \
        else if ((rows) <= 128) { constexpr int RP = 16; __VA_ARGS__; }                 \
        else { constexpr int RP = 32; __VA_ARGS__; }                                    \
    } while (0)

// floats of one (token, head) of the scratch that mi_delta_scan needs: T * H * this many
int mi_delta_scan_prep_row(int d) { return 3 * (d <= 64 ? 64 : (d <= 128 ? 128 : 256)) + 4; }

static int delta_scan_launch(const float* qkv, int ld_qkv, const float* beta_raw, int ld_beta, const float* a_raw, int ld_a,
                             const float* a_log, const float* dt_bias, float* state, int64_t state_stride,
                             const int* q_start, const int* state_slot, float* out, float* prep, int T, int B, int H, int G,
                             int d, int dv, float q_scale, int form, float tau, int segs, int seg_len, float* seg_state,
                             float* qt, float* bend, cudaStream_t stream) {
    if (B <= 0 || T <= 0) return kOk;
    if (d < 1 || d > 256 || dv < 1) { set_last_error("delta rule: key size %d outside [1, 256] or value size %d", d, dv); return kBadShape; }
    if (G < 1 || H % G) { set_last_error("delta rule: %d heads are not a multiple of %d key heads", H, G); return kBadShape; }
    if (B > 65535 || H > 65535) { set_last_error("delta rule: batch %d or heads %d exceed the grid limit", B, H); return kBadShape; }
    if (!prep || (reinterpret_cast<uintptr_t>(prep) & 15)) { set_last_error("delta rule: the scratch is missing or not 16-byte aligned"); return kBadShape; }
    if (form < 0 || form > 2 || (form == kSigmoidDecay && !(tau > 0.f)) || (form != kSigmoidDecay && (!beta_raw || !a_log))) {
        set_last_error("delta rule: form %d with tau %g, or a form that lacks its write strengths or decay rates", form, (double)tau);
        return kBadShape;
    }
    if (segs < 1 || (segs > 1 && (form != kSigmoidDecay || seg_len < 1 || !seg_state || !qt || !bend ||
                                  (int64_t)B * segs > 65535 || (int64_t)H * ((dv + kCorrectCols - 1) / kCorrectCols) > 65535))) {
        set_last_error("walk in segments: %d segments of %d tokens for %d requests (gated linear attention only, with its scratch)",
                       segs, seg_len, B);
        return kBadShape;
    }
    const int DP = d <= 64 ? 64 : (d <= 128 ? 128 : 256);
    launch_dependent(delta_prepare_kernel, dim3(T, H), dim3(128), 0, stream, qkv, ld_qkv, beta_raw, ld_beta, a_raw, ld_a,
                     a_log, dt_bias, prep, H, G, d, DP, q_scale, form, tau);
    if (segs > 1)
        launch_dependent(gla_segment_decay_kernel, dim3((d + 127) / 128, H, B * segs), dim3(128), 0, stream,
                         (const float*)prep, q_start, qt, bend, H, d, DP, segs, seg_len);
    const dim3 grid((dv + kScanCols - 1) / kScanCols, H, B * segs);
    MI_SCAN_DISPATCH(d, {
        const size_t smem = sizeof(float) * (2 * kScanChunk * (3 * RP * kScanLanes + 4 + kScanCols) + kScanChunk * kScanCols);
        if (form == kSigmoidDecay) {
            cudaFuncSetAttribute(delta_scan_kernel<RP, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            launch_dependent(delta_scan_kernel<RP, false>, grid, dim3(128), smem, stream, qkv, ld_qkv, (int64_t)2 * G * d,
                             (const float*)prep, state, state_stride, q_start, state_slot, out, H, d, dv, segs, seg_len,
                             seg_state);
        } else {
            cudaFuncSetAttribute(delta_scan_kernel<RP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            launch_dependent(delta_scan_kernel<RP, true>, grid, dim3(128), smem, stream, qkv, ld_qkv, (int64_t)2 * G * d,
                             (const float*)prep, state, state_stride, q_start, state_slot, out, H, d, dv, 1, 0,
                             (float*)nullptr);
        }
    });
    if (segs == 1) return finish_launch("delta_scan", 2);
    launch_dependent(gla_segments_combine_kernel, dim3((d * dv + 255) / 256, H, B), dim3(256), 0, stream, seg_state,
                     (const float*)bend, state, state_stride, q_start, state_slot, H, d, dv, segs, seg_len);
    const int tiles = (seg_len + kCorrectTokens - 1) / kCorrectTokens, chunks = (dv + kCorrectCols - 1) / kCorrectCols;
    const size_t corr_smem = sizeof(float) * ((size_t)d * kCorrectCols + 8 * 4 * d);
    cudaFuncSetAttribute(delta_segments_correct_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)corr_smem);
    launch_dependent(delta_segments_correct_kernel, dim3((segs - 1) * tiles, H * chunks, B), dim3(256), corr_smem, stream,
                     (const float*)seg_state, (const float*)qt, out, q_start, H, d, dv, segs, seg_len, tiles, chunks);
    return finish_launch("delta_scan", 5);
}

// form: see delta_prepare_kernel (0 and 1: the delta rule; 2: gated linear attention, which reads neither
// beta_raw nor a_log); tau: form 2 only
int mi_delta_scan_form(const float* qkv, int ld_qkv, const float* beta_raw, int ld_beta, const float* a_raw, int ld_a,
                       const float* a_log, const float* dt_bias, float* state, int64_t state_stride,
                       const int* q_start, const int* state_slot, float* out, float* prep, int T, int B, int H, int G,
                       int d, int dv, float q_scale, int form, float tau, cudaStream_t stream) {
    return delta_scan_launch(qkv, ld_qkv, beta_raw, ld_beta, a_raw, ld_a, a_log, dt_bias, state, state_stride, q_start,
                             state_slot, out, prep, T, B, H, G, d, dv, q_scale, form, tau, 1, 0, nullptr, nullptr, nullptr,
                             stream);
}

// Gated linear attention (form 2) with every request's portion walked as `segs` segments of seg_len tokens side by
// side (see delta_scan_kernel): seg_state holds B * segs * H * d * dv floats, qt T * H * d, bend B * segs * H * d.
// The sums of a token then run in another order than in the walk of one piece: the two agree within rounding, not
// bit for bit.
int mi_gla_scan_segments(const float* qkv, int ld_qkv, const float* a_raw, int ld_a, const float* dt_bias, float* state,
                         int64_t state_stride, const int* q_start, const int* state_slot, float* out, float* prep, int T,
                         int B, int H, int d, int dv, float q_scale, float tau, int segs, int seg_len, float* seg_state,
                         float* qt, float* bend, cudaStream_t stream) {
    return delta_scan_launch(qkv, ld_qkv, nullptr, 0, a_raw, ld_a, nullptr, dt_bias, state, state_stride, q_start,
                             state_slot, out, prep, T, B, H, H, d, dv, q_scale, kSigmoidDecay, tau, segs, seg_len, seg_state,
                             qt, bend, stream);
}

int mi_delta_scan(const float* qkv, int ld_qkv, const float* beta_raw, int ld_beta, const float* a_raw, int ld_a,
                  const float* a_log, const float* dt_bias, float* state, int64_t state_stride, const int* q_start,
                  const int* state_slot, float* out, float* prep, int T, int B, int H, int G, int d, int dv,
                  float q_scale, cudaStream_t stream) {
    return mi_delta_scan_form(qkv, ld_qkv, beta_raw, ld_beta, a_raw, ld_a, a_log, dt_bias, state, state_stride, q_start,
                              state_slot, out, prep, T, B, H, G, d, dv, q_scale, kDecayPerChannel, 1.0f, stream);
}

int mi_ssd_scan(const float* xbc, int ld_x, const float* dt_raw, int ld_dt, const float* dt_bias, const float* a_log,
                const float* d_skip, float* state, int64_t state_stride, const int* q_start, const int* state_slot,
                float* out, int B, int H, int G, int N, int P, cudaStream_t stream) {
    if (B <= 0) return kOk;
    if (N < 1 || N > 256 || P < 1) { set_last_error("state-space scan: state size %d outside [1, 256] or head size %d", N, P); return kBadShape; }
    if (G < 1 || H % G) { set_last_error("state-space scan: %d heads are not a multiple of %d groups", H, G); return kBadShape; }
    if (B > 65535 || H > 65535) { set_last_error("state-space scan: batch %d or heads %d exceed the grid limit", B, H); return kBadShape; }
    const dim3 grid((P + kScanCols - 1) / kScanCols, H, B);
    const int vec = (N % 4 == 0 && ld_x % 4 == 0 && (H * P) % 4 == 0 && (reinterpret_cast<uintptr_t>(xbc) & 15) == 0) ? 1 : 0;
    MI_SCAN_DISPATCH(N, {
        const size_t smem = sizeof(float) * (2 * kScanChunk * (2 * RP * kScanLanes + kScanCols + 2) + kScanChunk * kScanCols);
        cudaFuncSetAttribute(ssd_scan_kernel<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dependent(ssd_scan_kernel<RP>, grid, dim3(128), smem, stream, xbc, ld_x, dt_raw,
                         ld_dt, dt_bias, a_log, d_skip, state, state_stride, q_start, state_slot, out, H, G, N, P, vec);
    });
    return finish_launch("ssd_scan");
}

int mi_gated_group_rmsnorm(const float* y, const float* gate, int ld_gate, const void* w, int wdtype, int wlen,
                           void* out, int adtype, int T, int n, int groups, int mode, float eps, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return kOk;
    if (groups < 1 || n % groups || groups > 65535 || wlen < 1 || (mode < 0 || mode > 2)) {
        set_last_error("gated group norm: %d columns in %d groups, weight of %d, mode %d", n, groups, wlen, mode);
        return kBadShape;
    }
    const int gs = n / groups;
    const bool vec = gs % 4 == 0 && wlen % 4 == 0 && n % 4 == 0 && ld_gate % 4 == 0 &&
                     ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(gate)) & 15) == 0;
    const int work = vec ? gs / 4 : gs;      // a thread takes four floats where it can
    int threads = 32;
    while (threads < work && threads < 256) threads *= 2;
    MI_DISPATCH_2(adtype, AT, wdtype, WT,
        launch_dependent(gated_group_rmsnorm_kernel<AT, WT>, dim3(T, groups), dim3(threads), 0, stream, y, gate,
                         ld_gate, (const WT*)w, wlen, (AT*)out, n, gs, mode, eps, vec));
    return finish_launch("gated_group_rmsnorm");
}

}  // extern "C"
